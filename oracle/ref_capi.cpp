// TEST INFRASTRUCTURE ONLY. C entry points around the reference's *own, unmodified* CPU kernels.
//
// This file is compiled together with the reference sources where they lie (see Makefile in this
// directory) into oracle/_ref/librg_ref.so. Every function builds the reference kernel object the
// way the reference's unit tests do (e.g. src/04kernel/test/kernels/rms_normalization/test_cpu.cpp:8-20)
// and calls the lowered routine on host buffers. Only tests, the smoke check and the benchmark's
// CPU-baseline leg load this library; the product path never does.
#include "../src/kernels/gather/cpu_kernel.hh"
#include "../src/kernels/mat_mul/cpu_kernel.hh"
#include "../src/kernels/rms_normalization/cpu_kernel.hh"
#include "../src/kernels/simple_binary/cpu_kernel.hh"
#include "../src/kernels/simple_unary/cpu_kernel.hh"
#include "../src/kernels/softmax/cpu_kernel.hh"
#include <cstdint>
#include <optional>

using namespace refactor;
using namespace kernel;

static Shape mkShape(uint32_t const *dims, int rank) {
    Shape s;
    for (int i = 0; i < rank; ++i) s.push_back(dims[i]);
    return s;
}
static DataType mkType(int code) { return *DataType::parse(static_cast<uint8_t>(code)); }

extern "C" {

// RmsNormalizationCpu (src/04kernel/src/kernels/rms_normalization/cpu_kernel.cc:19-73). dtype: 1=F32, 11=F64.
int rg_ref_rms_norm(int dtype, void const *x, void const *w, void *y,
                    uint32_t const *shape, int rank, float eps) {
    auto t = Tensor::share(mkType(dtype), mkShape(shape, rank));
    auto k = RmsNormalizationCpu::build(eps, *t);
    if (!k) return 1;
    runtime::Resources res;
    auto r = k->lower(res).routine;
    void const *in[]{x, w};
    void *out[]{y};
    r(res, nullptr, in, out);
    return 0;
}

// SoftmaxCpu as built (src/04kernel/src/kernels/softmax/cpu_kernel.cc:27-70), integer-truncated row sum included.
int rg_ref_softmax(int dtype, void const *x, void *y, uint32_t const *shape, int rank, int axis) {
    auto t = Tensor::share(mkType(dtype), mkShape(shape, rank));
    auto k = SoftmaxCpu::build(SoftmaxInfo(*t, axis));
    if (!k) return 1;
    runtime::Resources res;
    auto r = k->lower(res).routine;
    void const *in[]{x};
    void *out[]{y};
    r(res, nullptr, in, out);
    return 0;
}

// MatMulCPU (src/04kernel/src/kernels/mat_mul/cpu_kernel.cc:28-91). c may be null (no bias).
int rg_ref_mat_mul(int dtype,
                   void const *a, uint32_t const *aShape, int aRank,
                   void const *b, uint32_t const *bShape, int bRank,
                   void const *c, uint32_t const *cShape, int cRank,
                   void *y, int transA, int transB, float alpha, float beta) {
    auto A = Tensor::share(mkType(dtype), mkShape(aShape, aRank));
    auto B = Tensor::share(mkType(dtype), mkShape(bShape, bRank));
    Arc<Tensor> C = c ? Tensor::share(mkType(dtype), mkShape(cShape, cRank)) : nullptr;
    auto k = MatMulCPU::build(MatMulInfo(
        *A, *B,
        C ? std::make_optional(std::cref(*C)) : std::nullopt,
        transA != 0, transB != 0, alpha, beta));
    if (!k) return 1;
    runtime::Resources res;
    auto r = k->lower(res).routine;
    void const *in[]{a, b, c};
    void *out[]{y};
    r(res, nullptr, in, out);
    return 0;
}

// GatherCpu (src/04kernel/src/kernels/gather/cpu_kernel.cc:24-42). idxType: 6=I32, 7=I64.
int rg_ref_gather(int dtype, void const *data, uint32_t const *dShape, int dRank,
                  int idxType, void const *idx, uint32_t const *iShape, int iRank,
                  void *out_, int axis) {
    auto D = Tensor::share(mkType(dtype), mkShape(dShape, dRank));
    auto I = Tensor::share(mkType(idxType), mkShape(iShape, iRank));
    auto k = GatherCpu::build(GatherInfo(axis, *D, *I));
    if (!k) return 1;
    runtime::Resources res;
    auto r = k->lower(res).routine;
    void const *in[]{data, idx};
    void *out[]{out_};
    r(res, nullptr, in, out);
    return 0;
}

// BinaryCpu (src/04kernel/src/kernels/simple_binary/cpu_kernel.cc:33-154). op: SimpleBinaryType value (0=Add, 2=Mul, 3=Div).
int rg_ref_binary(int op, int dtype,
                  void const *a, uint32_t const *aShape, int aRank,
                  void const *b, uint32_t const *bShape, int bRank, void *y) {
    auto A = Tensor::share(mkType(dtype), mkShape(aShape, aRank));
    auto B = Tensor::share(mkType(dtype), mkShape(bShape, bRank));
    auto k = BinaryCpu::build(static_cast<SimpleBinaryType>(op), *A, *B);
    if (!k) return 1;
    runtime::Resources res;
    auto r = k->lower(res).routine;
    void const *in[]{a, b};
    void *out[]{y};
    r(res, nullptr, in, out);
    return 0;
}

// SimpleUnaryCpu (src/04kernel/src/kernels/simple_unary/cpu_kernel.cc). op: SimpleUnaryType value (15=Sigmoid).
int rg_ref_unary(int op, int dtype, void const *x, void *y, uint32_t const *shape, int rank) {
    auto X = Tensor::share(mkType(dtype), mkShape(shape, rank));
    auto k = SimpleUnaryCpu::build(static_cast<SimpleUnaryType>(op), *X);
    if (!k) return 1;
    runtime::Resources res;
    auto r = k->lower(res).routine;
    void const *in[]{x};
    void *out[]{y};
    r(res, nullptr, in, out);
    return 0;
}

}// extern "C"
