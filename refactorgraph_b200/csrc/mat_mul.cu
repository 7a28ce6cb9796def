// rg_b200_mat_mul: routes a MatMul (MatMulInfo semantics, src/04kernel/src/attributes/mat_mul_info.cc:27-42)
// to one of the three hand-written kernels.  No vendor GEMM is linked.
#include "gemm_dispatch.cuh"
#include <cstdlib>

using namespace rg;

static bool gemv_shape(const rg_mat_mul_params *p) {
    return (p->dtype == RG_FP16 || p->dtype == RG_BF16) && !p->trans_a && p->trans_b && p->m <= 4 && p->batch == 1 &&
           !p->has_bias && p->alpha == 1.0f && p->k % 8 == 0 && p->k * 2u <= 32768u;
}

static int run_gemv(const rg_mat_mul_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    rg_linear_params lp = {};
    lp.dtype = p->dtype;
    lp.m = p->m, lp.n = p->n, lp.k = p->k;
    const void *lin[6] = {in[0], in[1], nullptr, nullptr, nullptr, nullptr};
    void *lout[3] = {out[0], nullptr, nullptr};
    return linear_stream(&lp, lin, lout, st);
}

// 5..32 rows of A against a K-major B: the weight-streaming kernel on the warp-level tensor path (RG_B200_SKINNY=0 keeps such
// products on the tcgen05 kernel)
static bool skinny_enabled() {
    static const bool on = [] {
        const char *e = std::getenv("RG_B200_SKINNY");
        return !(e && e[0] == '0');
    }();
    return on;
}
static bool skinny_shape(const rg_mat_mul_params *p) {
    if (p->trans_a || !p->trans_b || p->batch != 1 || p->m <= 4 || p->m > 32) return false;
    if (p->has_bias && (p->bias_col_stride > 1)) return false;
    return linear_skinny_shape(p->dtype, p->m, p->n, p->k);
}
// The automatic choice: up to 16 rows of A against few rows of B with a long k — the shape where the tcgen05 kernel has too
// few 128-row tiles and pays for a deep split (measured: 1280 x 8192 weights 13.0 us here, 18.3 us there; the other
// products of a decoder layer are 15-40 % faster on tcgen05).
static bool skinny_preferred(const rg_mat_mul_params *p) {
    return skinny_enabled() && skinny_shape(p) && p->m <= 16 && p->n <= 2560 && p->k >= 4096;
}
static int run_skinny(const rg_mat_mul_params *p, void *ws, const void *const *in, void *const *out, cudaStream_t st) {
    SkinnyCall c = {};
    c.dtype = p->dtype, c.m = p->m, c.n = p->n, c.k = p->k;
    c.epilogue = p->has_bias ? 1 : 0;
    c.alpha = p->alpha, c.beta = p->beta;
    c.c_row_stride = p->bias_row_stride, c.c_col_stride = p->bias_col_stride, c.y_row_stride = p->n;
    c.w_static = (p->flags & RG_MM_B_STATIC) != 0;
    const void *lin[5] = {in[0], in[1], p->has_bias ? in[2] : nullptr, nullptr, nullptr};
    void *lout[3] = {out[0], nullptr, nullptr};
    return linear_skinny(c, ws, lin, lout, st);
}

extern "C" {

size_t rg_b200_mat_mul_workspace(const rg_mat_mul_params *p) {
    // the tensor-core kernel's split-K path and the skinny kernel's k-split need scratch; sized for whichever could be chosen
    if (!p || (p->dtype != RG_FP16 && p->dtype != RG_BF16) || p->trans_a || !p->trans_b) return 0;
    size_t bytes = gemm_tc_workspace(p);
    if (skinny_shape(p)) {
        const size_t s = linear_skinny_workspace(p->dtype, p->m, p->n, p->k, p->has_bias ? 1 : 0, nullptr, 0);
        bytes = s > bytes ? s : bytes;
    }
    return bytes;
}

int rg_b200_mat_mul(const rg_mat_mul_params *p, void *ws, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !in[1] || !out[0]) return RG_ERR_NULL;
    if (p->has_bias && !in[2]) return RG_ERR_NULL;
    if (p->dtype != RG_F32 && p->dtype != RG_FP16 && p->dtype != RG_BF16) return RG_ERR_DTYPE;
    if (p->k == 0) return RG_ERR_SHAPE;
    if (p->m == 0 || p->n == 0 || p->batch == 0) return RG_OK;
    if (p->batch > 65535) return RG_ERR_SHAPE;
    auto st = static_cast<cudaStream_t>(stream);
    switch (p->force_kernel) {
        case 0: break;
        case 1: return gemm_simt(p, in, out, st);
        case 2: return gemv_shape(p) ? run_gemv(p, in, out, st) : RG_ERR_UNSUPPORTED;
        case 3: return gemm_tc_supported(p, in, out) ? gemm_tc(p, ws, in, out, st) : RG_ERR_UNSUPPORTED;
        case 4: return skinny_shape(p) ? run_skinny(p, ws, in, out, st) : RG_ERR_UNSUPPORTED;
        default: return RG_ERR_UNSUPPORTED;
    }
    if (gemv_shape(p) && aligned16(in[0]) && aligned16(in[1])) {
        const int rc = run_gemv(p, in, out, st);
        if (rc != RG_ERR_SHAPE && rc != RG_ERR_UNSUPPORTED) return rc;
    }
    if (skinny_preferred(p) && aligned16(in[0]) && aligned16(in[1]) && aligned16(out[0]) &&
        (ws || linear_skinny_workspace(p->dtype, p->m, p->n, p->k, p->has_bias ? 1 : 0, nullptr, 0) == 0)) {
        const int rc = run_skinny(p, ws, in, out, st);
        if (rc != RG_ERR_SHAPE && rc != RG_ERR_UNSUPPORTED) return rc;
    }
    if (gemm_tc_supported(p, in, out) && (ws || gemm_tc_workspace(p) == 0)) return gemm_tc(p, ws, in, out, st);
    return gemm_simt(p, in, out, st);
}
}
