// The adapters a RefactorGraph maintainer adds to bind the B200 kernel library (one per operator), written against
// the REFERENCE's own headers: kernel/kernel.h, kernel/tensor.h, kernel/collectors/*.h, kernel/attributes/*.h,
// runtime/resource.h.  tests/test_reference_headers_compile.py compiles this file with g++ -fsyntax-only against a reference
// checkout (include directories src/00common .. src/04kernel plus the two shims under oracle/shim), which is the proof that
// the C ABI of include/rg_b200.h fits the reference's Kernel / Routine / Resources interfaces as they are.
// One adapter per interface shape: a plain operator (RmsNormalization), an operator with attribute structs and a workspace
// (MatMul, through MatMulInfo), and an operator that needs a long-lived handle in Resources (AllReduce).
#include "kernel/attributes/communication.h"
#include "kernel/attributes/mat_mul_info.h"
#include "kernel/collectors/all_reduce.h"
#include "kernel/collectors/mat_mul.h"
#include "kernel/collectors/rms_normalization.h"
#include "kernel/kernel.h"
#include "kernel/tensor.h"
#include "rg_b200.h"
#include "runtime/resource.h"

namespace refactor::kernel {

    static void check(int rc, char const *what) {
        if (rc) RUNTIME_ERROR(fmt::format("{}: {}", what, rg_b200_status_string(rc)));
    }

    // ---- RmsNormalization: replaces RmsNormalizationCuda (src/04kernel/src/kernels/rms_normalization/cuda_kernel.cc) ----
    struct RmsNormalizationB200 final : public Kernel {
        rg_rms_norm_params info;
        explicit RmsNormalizationB200(rg_rms_norm_params p) noexcept : info(p) {}
        static KernelBox build(float epsilon, Tensor const &x) noexcept {
            if (!x.dataType.isFloat() || x.dataType == DataType::F64) return nullptr;
            rg_rms_norm_params p{};
            p.dtype = x.dataType.internal;// rg_dtype uses the reference's DataType codes
            p.dim = x.shape.back();
            p.rows = x.elementsSize() / p.dim;
            p.epsilon = epsilon;
            return std::make_unique<RmsNormalizationB200>(p);
        }
        static size_t typeId() noexcept {
            static uint8_t ID = 1;
            return reinterpret_cast<size_t>(&ID);
        }
        size_t kernelTypeId() const noexcept final { return typeId(); }
        std::string_view description() const noexcept final { return "RMS normalization on B200"; }
        RoutineWorkspace lower(Resources &) const final {
            return RoutineWorkspace(
                [info = info](Resources &, void *ws, void const *const *in, void *const *out) {
                    check(rg_b200_rms_norm(&info, ws, in, out, nullptr), "rg_b200_rms_norm");
                },
                rg_b200_rms_norm_workspace(&info));
        }
    };

    // ---- MatMul: replaces MatMulCublas (src/04kernel/src/kernels/mat_mul/cublas_kernel.cu); MatMulInfo carries m, k, n, the
    //      transposes, alpha / beta and the bias flag (src/04kernel/include/kernel/attributes/mat_mul_info.h) ----
    struct MatMulB200 final : public Kernel {
        rg_mat_mul_params info;
        explicit MatMulB200(rg_mat_mul_params p) noexcept : info(p) {}
        // weightIsConstant: B carries host data at lowering time (an initializer), so no kernel of the stream writes it and the
        // library may fetch its tiles while the previous kernel still runs — the reference-side route for RG_MM_B_STATIC
        static KernelBox build(MatMulInfo const &mm, bool weightIsConstant) noexcept {
            if (!mm.dataType.isFloat() || mm.dataType == DataType::F64) return nullptr;
            if (mm.broadcaster.outputsCount != 1) return nullptr;// batched products: flattened by a fuller adapter
            rg_mat_mul_params p{};
            p.dtype = mm.dataType.internal;
            p.m = mm.m, p.n = mm.n, p.k = mm.k;
            p.trans_a = mm.transA, p.trans_b = mm.transB;
            p.alpha = mm.alpha, p.beta = mm.beta;
            p.batch = 1;
            p.has_bias = mm.biasExpand.has_value();
            p.bias_row_stride = 0, p.bias_col_stride = 1;// the reference expands its bias to [m, n] first; a row bias needs no copy here
            if (weightIsConstant) p.flags |= RG_MM_B_STATIC;
            return std::make_unique<MatMulB200>(p);
        }
        static size_t typeId() noexcept {
            static uint8_t ID = 1;
            return reinterpret_cast<size_t>(&ID);
        }
        size_t kernelTypeId() const noexcept final { return typeId(); }
        std::string_view description() const noexcept final { return "MatMul on B200 (tcgen05 / streaming kernels)"; }
        RoutineWorkspace lower(Resources &) const final {
            return RoutineWorkspace(
                [info = info](Resources &, void *ws, void const *const *in, void *const *out) {
                    check(rg_b200_mat_mul(&info, ws, in, out, nullptr), "rg_b200_mat_mul");
                },
                rg_b200_mat_mul_workspace(&info));// the allocator turns the size into an offset (flat_allocator.cpp:34-36)
        }
    };

    // ---- AllReduce: replaces AllReduceNccl + NcclCommunicator.  The communicator is a runtime::Resource that whoever builds
    //      the Stream for this rank stores in Resources (the reference's own test does the same with NcclCommunicator,
    //      src/04kernel/test/kernels/all_reduce/test_allreduce_nccl.cpp:24); the routine fetches it at run time ----
    struct B200Communicator final : public runtime::Resource {
        rg_comm *comm;
        explicit B200Communicator(rg_comm *c) noexcept : comm(c) {}
        ~B200Communicator() override {
            if (comm) rg_b200_comm_destroy(comm);
        }
        static size_t typeId() noexcept {
            static uint8_t ID = 1;
            return reinterpret_cast<size_t>(&ID);
        }
        static runtime::ResourceBox build(rg_comm *c) noexcept { return std::make_unique<B200Communicator>(c); }
        size_t resourceTypeId() const noexcept final { return typeId(); }
        std::string_view description() const noexcept final { return "NVLink peer-memory communicator"; }
    };
    struct AllReduceB200 final : public Kernel {
        rg_all_reduce_params info;
        explicit AllReduceB200(rg_all_reduce_params p) noexcept : info(p) {}
        static KernelBox build(AllReduceType type, Tensor const &input, Tensor const &output) noexcept {
            if (input.elementsSize() != output.elementsSize() || input.dataType != output.dataType) return nullptr;// nccl_kernel.cc:14-17
            rg_all_reduce_params p{};
            p.dtype = input.dataType.internal;
            p.op = static_cast<int32_t>(type);
            p.count = input.elementsSize();
            return std::make_unique<AllReduceB200>(p);
        }
        static size_t typeId() noexcept {
            static uint8_t ID = 1;
            return reinterpret_cast<size_t>(&ID);
        }
        size_t kernelTypeId() const noexcept final { return typeId(); }
        std::string_view description() const noexcept final { return "AllReduce over NVLink peer memory on B200"; }
        RoutineWorkspace lower(Resources &) const final {
            return [info = info](Resources &res, void *, void const *const *in, void *const *out) {
                auto comm = res.fetch<B200Communicator>();
                if (!comm) RUNTIME_ERROR("AllReduce: no communicator in Resources");
                void const *in_[2] = {in[0], nullptr};
                check(rg_b200_all_reduce(comm->comm, &info, in_, out, nullptr), "rg_b200_all_reduce");
            };
        }
    };

    // ---- the collector lines (first candidate wins, src/05computation/src/graph.cc:48-49): what a maintainer writes inside
    //      `case decltype(_target)::Nvidia:` of each collector's filter() ----
    std::vector<KernelBox> b200_rms_normalization_candidates(float epsilon, TensorRefs inputs) {
        std::vector<KernelBox> ans;
        if (auto ptr = RmsNormalizationB200::build(epsilon, inputs[0]); ptr) ans.emplace_back(std::move(ptr));
        return ans;
    }
    std::vector<KernelBox> b200_mat_mul_candidates(float alpha, float beta, bool transA, bool transB, TensorRefs inputs) {
        std::vector<KernelBox> ans;
        MatMulInfo info(inputs[0], inputs[1],
                        inputs.size() == 2 ? std::nullopt : std::make_optional(std::reference_wrapper(inputs[2].get())),
                        transA, transB, alpha, beta);
        if (auto ptr = MatMulB200::build(info, inputs[1].get().data != nullptr); ptr) ans.emplace_back(std::move(ptr));
        return ans;
    }
    std::vector<KernelBox> b200_all_reduce_candidates(AllReduceType type, TensorRefs inputs, TensorRefs outputs) {
        std::vector<KernelBox> ans;
        if (auto ptr = AllReduceB200::build(type, inputs[0], outputs[0]); ptr) ans.emplace_back(std::move(ptr));
        return ans;
    }

}// namespace refactor::kernel
