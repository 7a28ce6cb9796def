// Internal entry points behind rg_b200_mat_mul / rg_b200_linear.
#pragma once
#include "common.cuh"
namespace rg {
int gemm_simt(const rg_mat_mul_params *p, const void *const *in, void *const *out, cudaStream_t st);
int linear_stream(const rg_linear_params *p, const void *const *in, void *const *out, cudaStream_t st);
// tcgen05/TMEM GEMM: Y[m,n] = alpha * A[m,k] * B[n,k]^T (+ beta*C), fp16/bf16, fp32 accumulation in TMEM.
int gemm_tc(const rg_mat_mul_params *p, void *ws, const void *const *in, void *const *out, cudaStream_t st);
int gemm_tc_swiglu(const rg_linear_params *p, const void *const *in, void *const *out, cudaStream_t st);
int gemm_tc_qkv_rope(const rg_linear_params *p, const void *const *in, void *const *out, cudaStream_t st);
size_t gemm_tc_workspace(const rg_mat_mul_params *p);// split-K partials + arrival counters (zero before first use)
bool gemm_tc_supported(const rg_mat_mul_params *p, const void *const *in, void *const *out);
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
}// namespace rg
