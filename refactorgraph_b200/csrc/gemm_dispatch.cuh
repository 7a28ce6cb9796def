// Internal entry points behind rg_b200_mat_mul / rg_b200_linear.
#pragma once
#include "common.cuh"
namespace rg {
struct ArPeers;
int gemm_simt(const rg_mat_mul_params *p, const void *const *in, void *const *out, cudaStream_t st);
int linear_stream(const rg_linear_params *p, const void *const *in, void *const *out, cudaStream_t st);
// tcgen05/TMEM GEMM: Y[m,n] = alpha * A[m,k] * B[n,k]^T (+ beta*C), fp16/bf16, fp32 accumulation in TMEM.
int gemm_tc(const rg_mat_mul_params *p, void *ws, const void *const *in, void *const *out, cudaStream_t st);
int gemm_tc_swiglu(const rg_linear_params *p, const void *const *in, void *const *out, cudaStream_t st);
// SiLU gate on 5..64 tokens: weights on the instruction's M side, k-split plan of the skinny product (workspace as reported)
bool gemm_tc_swiglu_small_shape(const rg_linear_params *p);
size_t gemm_tc_swiglu_small_workspace(const rg_linear_params *p);
int gemm_tc_swiglu_small(const rg_linear_params *p, void *ws, const void *const *in, void *const *out, cudaStream_t st);
// QKV split + RoPE + cache append on 5..64 tokens, same orientation (a 128-row tile = one head of head_dim 128)
bool gemm_tc_qkv_rope_small_shape(const rg_linear_params *p);
size_t gemm_tc_qkv_rope_small_workspace(const rg_linear_params *p);
int gemm_tc_qkv_rope_small(const rg_linear_params *p, void *ws, const void *const *in, void *const *out, cudaStream_t st);
int gemm_tc_qkv_rope(const rg_linear_params *p, const void *const *in, void *const *out, cudaStream_t st);
size_t gemm_tc_workspace(const rg_mat_mul_params *p);// split-K partials + arrival counters (zero before first use)
// The product of up to 64 tokens whose 16-bit result goes, paired with the flag of the communicator's call in flight, into this
// rank's all-reduce slots on the peers instead of into Y (in = {A, B}); RG_ERR_UNSUPPORTED for any other shape
int gemm_tc_push(const rg_mat_mul_params *p, void *ws, const void *const *in, const ArPeers &peers, cudaStream_t st);
bool gemm_tc_supported(const rg_mat_mul_params *p, const void *const *in, void *const *out);
// Weight-streaming linear layer for 5..32 rows of X on the warp-level tensor path (linear_skinny.cu).
struct SkinnyCall {
    int dtype;
    uint32_t m, n, k;
    int epilogue;// 0 store, 1 alpha * acc + beta * C, 2 SiLU gate, 3 QKV split + RoPE + cache append
    float alpha, beta;
    uint32_t c_row_stride, c_col_stride, y_row_stride;
    uint32_t n_heads;
    float theta;
    rg_kv_layout kv;
    uint32_t tokens_per_seq;
    int w_static;// W is a weight: its stream may start before the previous kernel has finished
};
bool linear_skinny_shape(int dtype, uint32_t m, uint32_t n, uint32_t k);
size_t linear_skinny_workspace(int dtype, uint32_t m, uint32_t n, uint32_t k, int epilogue, const rg_kv_layout *kv, uint32_t n_heads);
// in = {X, W, C or NULL, positions or NULL, block_table or NULL}; out = {Y, k_cache or NULL, v_cache or NULL}
int linear_skinny(const SkinnyCall &c, void *ws, const void *const *in, void *const *out, cudaStream_t st);
// per-file error words: bounded waits that expired, and device-read indices that were out of range (clear: zero after reading)
int linear_error_word(bool clear);
int attn_error_word(bool clear);
int gemm_tc_error_word(bool clear);
int all_reduce_error_word(bool clear);
int mega_error_word(bool clear);
int linear_index_error_word(bool clear);
int elementwise_index_error_word(bool clear);
int gemm_tc_index_error_word(bool clear);
int mega_index_error_word(bool clear);
int attn_index_error_word(bool clear);
int gqa_index_error_word(bool clear);
int skinny_error_word(bool clear);
int attn_tc_error_word(bool clear);
int skinny_index_error_word(bool clear);
}// namespace rg
