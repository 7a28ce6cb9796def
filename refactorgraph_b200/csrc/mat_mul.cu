// rg_b200_mat_mul: routes a MatMul (MatMulInfo semantics, src/04kernel/src/attributes/mat_mul_info.cc:27-42)
// to one of the three hand-written kernels.  No vendor GEMM is linked.
#include "gemm_dispatch.cuh"

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

extern "C" {

size_t rg_b200_mat_mul_workspace(const rg_mat_mul_params *p) {
    // only the tensor-core kernel's split-K path needs scratch; sized for it whenever that kernel could be chosen
    if (!p || (p->dtype != RG_FP16 && p->dtype != RG_BF16) || p->trans_a || !p->trans_b) return 0;
    return gemm_tc_workspace(p);
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
        default: return RG_ERR_UNSUPPORTED;
    }
    if (gemv_shape(p) && aligned16(in[0]) && aligned16(in[1])) {
        const int rc = run_gemv(p, in, out, st);
        if (rc != RG_ERR_SHAPE && rc != RG_ERR_UNSUPPORTED) return rc;
    }
    if (gemm_tc_supported(p, in, out) && (ws || gemm_tc_workspace(p) == 0)) return gemm_tc(p, ws, in, out, st);
    return gemm_simt(p, in, out, st);
}
}
