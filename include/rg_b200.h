/*
 * rg_b200.h — C ABI of the B200 (sm_100a) kernel library for the RefactorGraph decoder hot path.
 *
 * The reference has no C ABI: its boundary is C++ virtual dispatch
 * (InfoCollector::filter -> Kernel::lower(Resources&) -> RoutineWorkspace,
 *  src/04kernel/include/kernel/collector.h:10-20, kernel.h:12-23) and a routine of type
 *   void(Resources&, void* workspace, void const* const* inputs, void* const* outputs)
 * (src/03runtime/include/runtime/stream.h:10).  Every entry point below keeps that calling shape:
 * a POD parameter struct that is filled once at lower() time from the tensor shapes, then
 *   int rg_b200_X(const params*, void* workspace, const void* const* inputs, void* const* outputs, void* stream)
 * with raw DEVICE pointers in operator-input order, and
 *   size_t rg_b200_X_workspace(const params*)
 * for the byte count a kernel returns in RoutineWorkspace.  No torch types, no exceptions, no exit():
 * the return value is an rg_status and the C++ adapters turn non-zero into RUNTIME_ERROR.
 *
 * `stream` is a cudaStream_t passed as void* (NULL = legacy default stream, which is what the
 * reference launches on).  All launches are asynchronous; nothing here allocates device memory
 * except rg_b200_comm_create.
 */
#ifndef RG_B200_H
#define RG_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes. */
typedef enum rg_status {
    RG_OK = 0,
    RG_ERR_NULL = 1,        /* a required pointer is NULL */
    RG_ERR_SHAPE = 2,       /* shape outside what the kernel supports */
    RG_ERR_DTYPE = 3,       /* data type not supported by this kernel */
    RG_ERR_ALIGN = 4,       /* pointer or leading dimension not aligned as required */
    RG_ERR_CUDA = 5,        /* a CUDA runtime call or launch failed */
    RG_ERR_TIMEOUT = 6,     /* a bounded device-side or rendezvous wait ran out */
    RG_ERR_UNSUPPORTED = 7, /* valid request that this build has no kernel for */
    RG_ERR_LIMIT = 8        /* size beyond a stated fixed maximum */
} rg_status;

/* Data type codes = the reference's DataType enum (src/00common/include/common/data_type.h:14-35). */
typedef enum rg_dtype {
    RG_F32 = 1, RG_U8 = 2, RG_I8 = 3, RG_U16 = 4, RG_I16 = 5, RG_I32 = 6, RG_I64 = 7, RG_BOOL = 9,
    RG_FP16 = 10, RG_F64 = 11, RG_U32 = 12, RG_U64 = 13, RG_BF16 = 16
} rg_dtype;

const char *rg_b200_status_string(int status);
/* Library ABI version (bumped on any struct change). */
int rg_b200_version(void);
/* Number of kernels this library has launched in the calling process since load (all entry points). */
uint64_t rg_b200_launch_count(void);
/* Synchronises the current device and reports whether any kernel of this library gave up a bounded device-side
 * wait since load: 0 = none; otherwise bit 0 linear, bit 1 decode attention, bit 2 tensor-core GEMM, bit 3 all-reduce, bit 4 decode step,
 * bit 5 a device-read index (position, sequence length, token id, block-table entry) was out of range and the access
 * was skipped or clamped; negative = the device could not be queried.  The words are sticky until rg_b200_error_clear. */
int rg_b200_error_state(void);
/* Synchronises the current device and clears the words rg_b200_error_state reports (not a communicator's status:
 * see rg_b200_comm_status).  Returns RG_OK or RG_ERR_CUDA. */
int rg_b200_error_clear(void);

/* ---------------------------------------------------------------------------------------------
 * RmsNormalization.  Replaces RmsNormalizationCuda
 * (src/04kernel/src/kernels/rms_normalization/cuda_kernel.cc:24-131; CPU semantics cpu_kernel.cc:41-66):
 *   y[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps) * w[:]
 * inputs {x[rows,dim], w[dim]}, outputs {y[rows,dim]}.  Sum of squares is accumulated in fp32.
 * With add_residual != 0: inputs {x, w, r[rows,dim]}, outputs {y, s}; s = x + r (stored in dtype) and
 * the norm is taken of s — the residual-add + norm pair of a decoder layer in one pass. */
typedef struct rg_rms_norm_params {
    int32_t dtype; /* RG_F32, RG_FP16, RG_BF16 */
    uint32_t rows, dim;
    float epsilon;
    int32_t add_residual;
} rg_rms_norm_params;
size_t rg_b200_rms_norm_workspace(const rg_rms_norm_params *);
int rg_b200_rms_norm(const rg_rms_norm_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Softmax over the middle axis of [pre, mid, post].  Replaces SoftmaxCudnn / SoftmaxCuda
 * (src/04kernel/src/collectors/softmax.cc:22-29, src/04kernel/src/kernels/softmax/cuda_kernel.cu:21-105;
 * SoftmaxInfo src/04kernel/src/attributes/softmax_info.cc:6-13).  A true softmax (what the reference's
 * CUDA and cuDNN kernels compute), max/sum in fp32.  inputs {x}, outputs {y}. */
typedef struct rg_softmax_params {
    int32_t dtype; /* RG_F32, RG_FP16, RG_BF16 */
    uint32_t pre, mid, post;
} rg_softmax_params;
size_t rg_b200_softmax_workspace(const rg_softmax_params *);
int rg_b200_softmax(const rg_softmax_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * TopK (no reference counterpart: the reference has no TopK operator or kernel).
 * Per row of x[rows,n]: the k largest values in descending order, ties broken by the lower index,
 * NaN treated as smaller than every number.  inputs {x}, outputs {values[rows,k] (dtype of x, or fp32
 * probabilities when softmax != 0), indices[rows,k] int64}.  With softmax != 0 the values are
 * softmax(x)[idx] over the WHOLE row (max and sum of exp over all n, fp32).  k <= 64. */
typedef struct rg_topk_params {
    int32_t dtype;
    uint32_t rows, n, k;
    int32_t softmax;
} rg_topk_params;
size_t rg_b200_topk_workspace(const rg_topk_params *);
int rg_b200_topk(const rg_topk_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* Top-k sampling (no reference counterpart).  Draws one token per row from softmax(x/temperature)
 * restricted to the row's top-k set.  The uniform number for (seed, step, row) is a Philox-4x32-10
 * draw with key (seed lo, seed hi) and counter (row, 0, step lo, step hi); the token is the first entry
 * of the descending top-k list whose cumulative probability exceeds u.
 * inputs {x[rows,n], step (device uint64[1])}, outputs {token[rows] int64}. */
typedef struct rg_topk_sample_params {
    int32_t dtype;
    uint32_t rows, n, k;
    float temperature;
    uint64_t seed;
} rg_topk_sample_params;
size_t rg_b200_topk_sample_workspace(const rg_topk_sample_params *);
int rg_b200_topk_sample(const rg_topk_sample_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Gather along one axis (embedding lookup).  Replaces GatherCuda
 * (src/04kernel/src/kernels/gather/cuda_kernel.cc:32-56, src/04kernel/cuda/src/gather.cu:7-29) with
 * GatherInfo's fields (src/04kernel/src/attributes/gather_info.cc:19-27): out[p, i, :] = data[p, idx[i], :],
 * negative indices wrap by mid_in; byte-exact.  inputs {data, indices}, outputs {out}. */
typedef struct rg_gather_params {
    uint32_t prefix, mid_in, mid_out;
    uint64_t postfix_bytes;
    int32_t idx_dtype; /* RG_I32 or RG_I64 */
} rg_gather_params;
size_t rg_b200_gather_workspace(const rg_gather_params *);
int rg_b200_gather(const rg_gather_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Element-wise binary with multidirectional broadcast, rank <= 4.  Replaces BinaryCudnn / BinaryCuda
 * (src/04kernel/src/kernels/simple_binary/cuda_kernel.cc:42-136).  op uses the reference's
 * SimpleBinaryType values (src/04kernel/include/kernel/collectors/simple_binary.h:8-19): 0 Add, 1 Sub,
 * 2 Mul, 3 Div, 4 Pow, 5 And, 6 Or, 7 Xor, 8 Mod, 9 Fmod.  RG_F32 / RG_FP16 / RG_BF16: 0-4 and 9 (evaluated in fp32);
 * RG_U8 / RG_I8 / RG_I16 / RG_I32 / RG_U32 / RG_I64: 0-4, 8 and 9 (`%` of C++: sign of the dividend; a zero divisor gives 0);
 * RG_BOOL: 5-7.  Any other pair is RG_ERR_UNSUPPORTED.  Strides are in elements, 0 on a broadcast axis.
 * inputs {a, b}, outputs {y}. */
typedef struct rg_binary_params {
    int32_t op, dtype;
    uint32_t shape[4];
    uint32_t a_stride[4], b_stride[4];
} rg_binary_params;
size_t rg_b200_binary_workspace(const rg_binary_params *);
int rg_b200_binary(const rg_binary_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* Element-wise unary.  Replaces ActivationCudnn / SimpleUnaryCuda
 * (src/04kernel/src/kernels/simple_unary/cuda_kernel.cc:96-175).  op uses SimpleUnaryType values
 * (src/04kernel/include/kernel/collectors/simple_unary.h:8-30): 0 Abs, 1 Acos, 2 Acosh, 3 Asin, 4 Asinh, 5 Atan, 6 Atanh, 7 Cos,
 * 8 Cosh, 9 Sin, 10 Sinh, 11 Tan, 12 Tanh, 13 Relu, 14 Sqrt, 15 Sigmoid, 16 Erf, 17 Neg, 19 HardSwish, 20 Exp on RG_F32 / RG_FP16 /
 * RG_BF16 (evaluated in fp32); 18 Not on RG_BOOL; 100 = SiLU (x*sigmoid(x), the fused pair the decoder uses).
 * inputs {x}, outputs {y}. */
typedef struct rg_unary_params {
    int32_t op, dtype;
    uint64_t n;
} rg_unary_params;
size_t rg_b200_unary_workspace(const rg_unary_params *);
int rg_b200_unary(const rg_unary_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* Where (select): y = cond ? a : b with rank <= 4 broadcast.  Replaces WhereCuda
 * (src/04kernel/cuda/src/where.cu:7-36).  inputs {cond (bool/u8), a, b}, outputs {y}. */
typedef struct rg_where_params {
    int32_t dtype;
    uint32_t shape[4];
    uint32_t c_stride[4], a_stride[4], b_stride[4];
} rg_where_params;
size_t rg_b200_where_workspace(const rg_where_params *);
int rg_b200_where(const rg_where_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* Transpose (permuted copy), rank <= 4, byte-exact.  Replaces TransposeCuda
 * (src/04kernel/cuda/src/transpose.cu:7-28).  out has shape[i] = in_shape[perm[i]].  inputs {x}, outputs {y}. */
typedef struct rg_transpose_params {
    uint32_t elem_bytes; /* 1, 2, 4 or 8 */
    uint32_t rank;
    uint32_t in_shape[4];
    uint32_t perm[4];
} rg_transpose_params;
size_t rg_b200_transpose_workspace(const rg_transpose_params *);
int rg_b200_transpose(const rg_transpose_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Byte-exact data movement around the arithmetic.  Shapes are in elements of elem_bytes (1, 2, 4, 8 or 16).
 *
 * Concat / Split along one axis, the tensors seen as [outer, axis_len, inner].  Replace ConcatCuda and SplitCuda
 * (src/04kernel/src/kernels/concat/cuda_kernel.cc, src/04kernel/src/kernels/split/cuda_kernel.cc; SplitInfo,
 * src/04kernel/src/attributes/split_info.cc:6-28).  concat: inputs {part 0 .. part n_parts - 1}, outputs {whole};
 * split: inputs {whole}, outputs {part 0 ..}.  Parts of length 0 are allowed (their pointer is not read). */
#define RG_CONCAT_MAX_PARTS 32
typedef struct rg_concat_params {
    uint32_t elem_bytes;
    uint32_t n_parts;
    uint32_t outer, inner;
    uint32_t axis_len[RG_CONCAT_MAX_PARTS];
} rg_concat_params;
size_t rg_b200_concat_workspace(const rg_concat_params *);
int rg_b200_concat(const rg_concat_params *, void *ws, const void *const *in, void *const *out, void *stream);
size_t rg_b200_split_workspace(const rg_concat_params *);
int rg_b200_split(const rg_concat_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* Slice: y[i0, i1, ..] = x[start0 + i0 * step0, ..], 0 <= i_d < length_d; steps may be negative (the Dimensions {start, step,
 * length} of the reference's SliceCollector, src/04kernel/include/kernel/attributes/slice_info.h:8-13; replaces SliceCuda).  Every
 * addressed index must lie inside the input (RG_ERR_SHAPE otherwise: nothing is launched).  rank <= 6.  inputs {x}, outputs {y}. */
#define RG_MOVE_MAX_RANK 6
typedef struct rg_slice_params {
    uint32_t elem_bytes;
    uint32_t rank;
    uint32_t in_shape[RG_MOVE_MAX_RANK];
    int64_t start[RG_MOVE_MAX_RANK], step[RG_MOVE_MAX_RANK];
    uint32_t length[RG_MOVE_MAX_RANK];
} rg_slice_params;
size_t rg_b200_slice_workspace(const rg_slice_params *);
int rg_b200_slice(const rg_slice_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* Expand: broadcast x to out_shape; in_shape has the same rank (the caller pads it with leading 1s) and every dimension equals
 * the output's or is 1.  Replaces ExpandCuda (src/04kernel/src/kernels/expand/cuda_kernel.cc).  inputs {x}, outputs {y}. */
typedef struct rg_expand_params {
    uint32_t elem_bytes;
    uint32_t rank;
    uint32_t in_shape[RG_MOVE_MAX_RANK], out_shape[RG_MOVE_MAX_RANK];
} rg_expand_params;
size_t rg_b200_expand_workspace(const rg_expand_params *);
int rg_b200_expand(const rg_expand_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* Cast between RG_F32, RG_F64, RG_FP16, RG_BF16, RG_I8, RG_U8, RG_I16, RG_U16, RG_I32, RG_U32, RG_I64, RG_U64 and RG_BOOL (one byte
 * holding 0 or 1).  Replaces CastCuda (src/04kernel/src/kernels/cast/cuda_kernel.cc).  static_cast semantics: float -> integer
 * truncates toward zero, anything -> bool is `!= 0`; conversions to 16-bit floats round to nearest even.  inputs {x}, outputs {y}. */
typedef struct rg_cast_params {
    int32_t from, to;
    uint64_t n;
} rg_cast_params;
size_t rg_b200_cast_workspace(const rg_cast_params *);
int rg_b200_cast(const rg_cast_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * RotaryPositionEmbedding (no reference counterpart).  x[tokens, heads, head_dim], rotate-half pairing
 * (i, i + head_dim/2), angle = pos * theta^(-2i/head_dim) evaluated in fp32; pos = positions[token]
 * (device int64[tokens]).  inputs {x, positions}, outputs {y}. */
typedef struct rg_rope_params {
    int32_t dtype;
    uint32_t tokens, heads, head_dim;
    float theta; /* 10000 */
} rg_rope_params;
size_t rg_b200_rope_workspace(const rg_rope_params *);
int rg_b200_rope(const rg_rope_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* State update for device-resident generation loops (no reference counterpart: the reference feeds every step
 * from the host).  state[i] = (src ? src[i] : state[i]) + delta, int64, in place.  Lets a captured decode step
 * carry the sampled token and the position to the next replay without a host round trip.
 * inputs {src or NULL}, outputs {state}. */
typedef struct rg_state_update_params {
    uint32_t n;
    int64_t delta;
} rg_state_update_params;
size_t rg_b200_state_update_workspace(const rg_state_update_params *);
int rg_b200_state_update(const rg_state_update_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * MatMul: Y[b] = alpha * op(A[b]) * op(B[b]) + beta * C (C broadcast to [m,n]).  Replaces MatMulCublas
 * (src/04kernel/src/kernels/mat_mul/cublas_kernel.cu:9-100) with MatMulInfo's fields
 * (src/04kernel/src/attributes/mat_mul_info.cc:27-42).  Row-major.  Batch strides are in elements and are 0
 * for an operand that is broadcast over the batch (the reference's Broadcaster over the leading dims is
 * flattened by the adapter into `batch` strided launches).  fp32 accumulation for every type.
 * inputs {A, B, C or NULL}, outputs {Y}.
 * Kernel selection (all hand-written, no vendor GEMM):
 *   - fp16/bf16, transA=0, transB=1, m <= 4: HBM-streaming GEMV (bulk-copy smem ring),
 *   - fp16/bf16, transA=0, transB=1, 5 <= m <= 32, k a multiple of 128: the same weight streaming with the rows of A on the
 *     warp-level tensor path (k cut into parts whose partial tiles are summed in a fixed order; needs the workspace),
 *   - fp16/bf16, transA=0, transB=1, aligned, m*n large: tcgen05/TMEM tensor-core GEMM fed by TMA,
 *   - anything else: shared-memory tiled SIMT GEMM.
 * Workspace: rg_b200_mat_mul_workspace bytes (split-K partials and arrival counters of the skinny and tensor-core
 * kernels); it must be zero on first use and is left ready for the next call.  Without a workspace such products fall
 * back to the SIMT kernel. */
typedef struct rg_mat_mul_params {
    int32_t dtype; /* RG_F32, RG_FP16, RG_BF16 */
    uint32_t m, n, k;
    int32_t trans_a, trans_b;
    float alpha, beta;
    uint32_t batch;
    uint64_t stride_a, stride_b, stride_y; /* per-batch element strides (0 = broadcast) */
    int32_t has_bias;
    uint32_t bias_row_stride, bias_col_stride; /* element strides of C over (m, n); 0 = broadcast */
    uint64_t stride_c;
    int32_t force_kernel; /* 0 auto, 1 SIMT tile, 2 streaming GEMV, 3 tcgen05, 4 streaming skinny kernel (5..32 rows) */
    uint32_t flags;       /* RG_MM_B_STATIC: B is a weight - no kernel earlier in the stream writes it - so its tiles may be
                             fetched while the preceding kernel is still running (programmatic dependent launch) */
} rg_mat_mul_params;
#define RG_MM_B_STATIC 1u
size_t rg_b200_mat_mul_workspace(const rg_mat_mul_params *);
int rg_b200_mat_mul(const rg_mat_mul_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * KV-cache addressing shared by the fused linear layer and attention.
 * Contiguous (the reference Attention operator's cache edge, src/08-01llm/src/operators/attention.cc:53-66):
 *   cache[b, kv_head, t, d], t < max_seq.
 * Paged (block_table != NULL at call time): cache[block, kv_head, t % page, d] with
 *   block = block_table[b * max_blocks_per_seq + t / page]. */
typedef struct rg_kv_layout {
    uint32_t n_kv_heads, head_dim;
    uint32_t max_seq;            /* contiguous: tokens per (b, head) */
    uint32_t page_size;          /* paged: tokens per block (16) ; 0 = contiguous */
    uint32_t max_blocks_per_seq; /* paged: row length of the block table */
    uint32_t n_blocks;           /* paged: blocks in the cache; block-table entries are checked against it (0 = only their sign is checked) */
} rg_kv_layout;
/* Every kernel that reads a position, sequence length, token id or block-table entry from device memory checks it
 * against these bounds (and the vocabulary) before using it: an out-of-range value is never used for an access —
 * the store is skipped, or the read range is clamped — and bit 5 of rg_b200_error_state is set. */

/* QKV split + RoPE + cache append for batched decode (no reference counterpart; what the m <= 4 linear kernel does in
 * its epilogue, as a separate launch behind a tensor-core GEMM).  qkv[tokens, (n_heads + 2 n_kv_heads) * D]: q heads
 * are rotated to q[tokens, n_heads * D]; k heads are rotated and v heads copied into the caches of the token's sequence
 * (token / tokens_per_seq) at positions[token].
 * inputs {qkv, positions (int64[tokens]), block_table (int32) or NULL}, outputs {q, k_cache, v_cache}. */
typedef struct rg_qkv_rope_append_params {
    int32_t dtype;
    uint32_t tokens, n_heads;
    float theta;
    rg_kv_layout kv;
    uint32_t tokens_per_seq; /* 0 or 1: every token is its own sequence (decode); S: tokens [b*S, (b+1)*S) belong to sequence b (prefill) */
} rg_qkv_rope_append_params;
size_t rg_b200_qkv_rope_append_workspace(const rg_qkv_rope_append_params *);
int rg_b200_qkv_rope_append(const rg_qkv_rope_append_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* SiLU gate: y[r, j] = silu(x[r, j]) * x[r, f + j] for x[rows, 2f] — the Sigmoid, Mul, Mul triple of the reference
 * graph (src/04kernel/src/kernels/simple_unary/cuda_kernel.cc:96-175, simple_binary/cuda_kernel.cc:42-136) in one pass.
 * inputs {x}, outputs {y[rows, f]}. */
typedef struct rg_swiglu_params {
    int32_t dtype;
    uint32_t rows, f;
} rg_swiglu_params;
size_t rg_b200_swiglu_workspace(const rg_swiglu_params *);
int rg_b200_swiglu(const rg_swiglu_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* Fused decode linear layer  Y = epilogue( prologue(X) * W^T ),  W[n,k] row-major (the reference MatMul with
 * transB = 1), X[m,k].  One launch replaces RmsNormalization + MatMul + (Add | Sigmoid,Mul,Mul |
 * RoPE + cache append) of the reference graph.  m <= 4: every prologue and epilogue.  5 <= m <= 32 (batched decode, k a
 * multiple of 128): prologue 0 with every epilogue, on the streaming skinny kernel; needs rg_b200_linear_workspace bytes,
 * zero on first use and left ready for the next call.  m > 64, prologue 0, epilogue 3 and head_dim 128, or epilogue 2
 * (prefill): the product runs on the tcgen05 GEMM and the split, rotation and cache append / the SiLU gate are its epilogue.
 * W is taken to be a weight: no kernel earlier in the stream may write it (its stream starts before the previous kernel ends).
 *   prologue: 0 none; 1 RMSNorm with weight g[k] and epsilon (fp32 statistics).
 *   epilogue: 0 none                      outputs {Y[m,n]}
 *             1 residual add              inputs + {R[m,n]}; Y = R + X*W^T
 *             2 SiLU gate                 W = [gate rows 0..n/2) ; up rows n/2..n); Y[m,n/2] = silu(g)*u
 *             3 QKV split + RoPE + append W = [q heads | k heads | v heads]; q -> Y[m, n_heads*head_dim] rotated,
 *                                         k rotated and v stored into the caches at positions[m]
 * inputs  {X, W, g or NULL, R or NULL, positions (int64[m]) or NULL, block_table (int32) or NULL}
 * outputs {Y, k_cache or NULL, v_cache or NULL}. */
typedef struct rg_linear_params {
    int32_t dtype; /* RG_FP16, RG_BF16 */
    uint32_t m, n, k;
    int32_t prologue, epilogue;
    float epsilon;
    uint32_t n_heads; /* epilogue 3: query heads; n = (n_heads + 2*kv.n_kv_heads) * kv.head_dim */
    float theta;
    rg_kv_layout kv;
    uint32_t tokens_per_seq; /* epilogue 3 with m > 64: token t belongs to sequence t / tokens_per_seq (0 or 1: one token per sequence) */
} rg_linear_params;
size_t rg_b200_linear_workspace(const rg_linear_params *);
int rg_b200_linear(const rg_linear_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * One whole batch-1 decode step as a single persistent kernel (no reference counterpart: the reference runs a
 * decoder as ~900 separate launches per token, src/03runtime/src/stream.cc:60-69).  Same semantics as the graph
 *   Gather, [Linear(norm,QKV,RoPE,append), AttentionDecode, Linear(O,+res), Linear(norm,gate/up,SiLU), Linear(down,+res)] x layers,
 *   Linear(norm, LM head), TopK(k=1, softmax), token <- argmax, pos <- pos + 1,
 * with the weights streamed continuously across the phase boundaries (grid barriers instead of kernel launches).
 * Contiguous KV caches [1, n_kv_heads, max_seq, head_dim]; weights as for rg_b200_linear.
 * inputs  {token (int64[1], updated), pos (int64[1] = cached tokens, updated), embed[vocab,hidden], norm_f[hidden],
 *          lm_head[vocab,hidden], then per layer: norm1, wqkv, wo, norm2, wgu, wd, k_cache, v_cache}
 * outputs {next (int64[1]), prob (fp32[1], softmax probability of the chosen token), logits[vocab]}
 * The workspace must be zero on first use and is left ready for the next call.  Launched cooperatively with one CTA
 * per SM; grid-barrier waits are bounded (RG error state bit 4).  After rg_b200_error_state has reported bit 4 the
 * workspace's barrier state is undefined: zero-fill it again before the next call.  A step whose position is not below
 * max_seq, or whose token id is not below vocab, does nothing (outputs and state untouched) and sets bit 5. */
typedef struct rg_decode_step_params {
    int32_t dtype; /* RG_FP16, RG_BF16 */
    uint32_t layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, max_seq;
    float epsilon, theta;
} rg_decode_step_params;
size_t rg_b200_decode_step_workspace(const rg_decode_step_params *);
/* Diagnostics: timestamps (ns) of the last call, read back from its workspace: four per phase (entered, activations
 * ready, units consumed, epilogue done; phases per layer: QKV, attention, O, gate/up, down; then the LM head) plus a final
 * group whose first entry is the end of the last grid barrier.  Returns entries written. */
size_t rg_b200_decode_step_timeline(const rg_decode_step_params *, const void *ws, uint64_t *out_ns, size_t capacity);
int rg_b200_decode_step(const rg_decode_step_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Attention.  Completes AttentionCuda, which the reference declares without a definition
 * (src/04kernel/src/kernels/attention/cuda_kernel.hh:10-25); semantics follow the operator spec
 * src/08-01llm/README.md:29-63 and shape rules src/08-01llm/src/operators/attention.cc:37-128:
 * causal multi-head self-attention, q head h uses kv head h / (n_heads / n_kv_heads),
 * scores = q.k / sqrt(head_dim), query row i (absolute position past + i) sees keys j <= past + i,
 * softmax and accumulation in fp32.
 *
 * rg_b200_attention (reference tensor layout):
 *   inputs {q[N,n_heads,S,D], k[N,n_kv,S,D], v[N,n_kv,S,D], past_seq_len (device int64[1]) or NULL,
 *           k_cache[N,n_kv,max_seq,D] or NULL, v_cache or NULL}
 *   outputs {o[N,n_heads,S,D], k_cache_out or NULL, v_cache_out or NULL}
 * With caches: k, v are first written at [past, past+S) of the cache (in place when k_cache_out == k_cache,
 * else the whole live prefix is copied), then attention runs over [0, past+S). */
typedef struct rg_attention_params {
    int32_t dtype;
    uint32_t batch, n_heads, n_kv_heads, seq_len, head_dim, max_seq;
    int32_t has_cache;
} rg_attention_params;
size_t rg_b200_attention_workspace(const rg_attention_params *);
int rg_b200_attention(const rg_attention_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* Causal flash attention with explicit element strides (head_dim 128, fp16 / bf16): what rg_b200_attention runs for
 * prefill, exposed so that a fused QKV projection can be consumed in its token-major layout without transposes.
 * strides[12] = {q, k, v, o} x {sequence, head, token}; the head dimension is contiguous and every stride a multiple of 8.
 * Query row i of a sequence (absolute position past + i) attends keys j <= past + i, j < kv_capacity.
 * inputs {q, k, v, past_seq_len (device int64[1]) or NULL}, outputs {o}. */
typedef struct rg_attn_prefill_params {
    int32_t dtype;
    uint32_t batch, n_heads, n_kv_heads, seq_len, head_dim, kv_capacity;
    int64_t strides[12];
} rg_attn_prefill_params;
size_t rg_b200_attn_prefill_workspace(const rg_attn_prefill_params *);
int rg_b200_attn_prefill(const rg_attn_prefill_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* Split-K flash-decoding over a (paged or contiguous) KV cache, one new token per sequence.
 *   inputs {q[batch, n_heads, D], k_cache, v_cache, seq_lens (device int64[batch]; keys [0, len) are attended,
 *           the new token's k/v already appended), block_table (int32) or NULL}
 *   outputs {o[batch, n_heads, D]}
 * Workspace holds the per-split partial (max, sum, acc) records and one arrival counter per (sequence, head);
 * the counters must be zero on first use (rg_b200_attn_decode_workspace bytes, zero-filled once) and are
 * left zero by every call. */
typedef struct rg_attn_decode_params {
    int32_t dtype;
    uint32_t batch, n_heads;
    uint32_t max_len; /* upper bound of seq_lens, sizes the split count */
    rg_kv_layout kv;
} rg_attn_decode_params;
size_t rg_b200_attn_decode_workspace(const rg_attn_decode_params *);
int rg_b200_attn_decode(const rg_attn_decode_params *, void *ws, const void *const *in, void *const *out, void *stream);

/* Flash-decoding without caller-provided scratch.  No counterpart in the reference.
 * Same inputs, outputs and results as rg_b200_attn_decode, but the split-K scratch (arrival counters and partial
 * records) sits in a fixed array inside this library's device image, so the call needs no workspace pointer and
 * performs no device allocation of any kind.  It is meant for hosts that cannot hand a kernel fresh device
 * memory at the point of the call: a runtime whose pool already owns the GPU's free memory (the reference's
 * Nvidia device takes 90 % of it at start-up, src/02hardware/src/devices/nvidia/device.cc:24-35), a latency-bound
 * serving loop that must not hit the synchronisation cudaMalloc implies, or a plugin that is only given input
 * and output buffers.
 *   - Limit: rg_b200_attn_decode_workspace(p) must not exceed rg_b200_attn_decode_static_capacity() (8 MiB);
 *     larger requests return RG_ERR_LIMIT and launch nothing.  Every GPU that loads the library holds the array
 *     until the process exits.
 *   - The first call on each device looks up the array's device address (one-time set-up, with that device
 *     current); make that first call outside any stream capture.
 *   - All calls on a device share the one array.  Calls that may overlap on the GPU (different streams, or
 *     graph branches) race on it; serialise them.  The counters are cleared at the start of every call. */
size_t rg_b200_attn_decode_static_capacity(void);
int rg_b200_attn_decode_static(const rg_attn_decode_params *, const void *const *in, void *const *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * AllReduce across the GPUs of one box.  Replaces AllReduceNccl + NcclCommunicator
 * (src/04kernel/src/kernels/all_reduce/nccl_kernel.cu:9-19, src/04kernel/src/utilities/cuda/nccl_communicator.cu:11-44).
 * One process per GPU.  rg_b200_comm_create allocates this rank's symmetric buffer and returns an opaque
 * 64-byte IPC handle; the caller exchanges handles out of band (any host transport) and calls
 * rg_b200_comm_connect with all ranks' handles.  The reduction is a push over NVLink peer memory with ordinary
 * stores (every 32-bit word travels with the call's 32-bit flag; the receiver polls its own memory): up to 3 ranks every
 * rank sends its whole input to every peer (one-shot); from 4 ranks on each run of chunks has an owner rank that combines
 * and sends the finished values back (two-shot).  Values are combined in rank order, so every rank gets bit-identical
 * results.  No TMA and no multicast instruction touches peer memory.
 * dtype: RG_F32, RG_FP16, RG_BF16 (combined in fp32), RG_F64, RG_U8, RG_I8, RG_I32, RG_U32, RG_I64 (combined in their
 * own type; integer Sum / Prod wrap, integer Avg divides) — the set AllReduceNccl accepts (nccl_kernel.cc:14-17).
 * op uses AllReduceType (src/04kernel/include/kernel/attributes/communication.h:5-11): 0 Sum, 1 Avg, 2 Min, 3 Max, 4 Prod.
 * inputs {x, residual or NULL}, outputs {y}; y = reduce(x) (+ residual, added after the reduced value has been rounded
 * to the storage type); bytes <= the capacity given at create.  Every rank must issue the same sequence of calls.
 * Waits: a kernel waits for its peers' data for at most the bound set by rg_b200_comm_set_wait_ns (default 2 s),
 * measured from the moment THIS rank's kernel starts — so ranks must reach matching calls within that bound of one
 * another (raise it if one process may stall longer, e.g. while it instantiates a CUDA graph).  When the wait runs out
 * the kernel leaves its output untouched and sets the communicator's status word; from then on the communicator is out
 * of step with its peers: every later all-reduce on it is a no-op on the device, rg_b200_comm_status and
 * rg_b200_all_reduce return RG_ERR_TIMEOUT, and bit 3 of rg_b200_error_state stays set until the communicator is
 * destroyed and a new one is created on every rank.  Call numbers are 64-bit; the 32-bit flag derived from them is never 0. */
typedef struct rg_comm rg_comm;
int rg_b200_comm_create(int world, int rank, size_t capacity_bytes, rg_comm **out, void *handle64);
int rg_b200_comm_connect(rg_comm *, const void *all_handles /* world * 64 bytes */);
/* Same-process wiring: bases[r] = rg_b200_comm_base of rank r's communicator (peer access already enabled). */
void *rg_b200_comm_base(rg_comm *);
size_t rg_b200_comm_bytes(rg_comm *); /* size of the symmetric allocation behind rg_b200_comm_base (what a stand-in peer buffer must provide) */
int rg_b200_comm_connect_ptrs(rg_comm *, const void *const *bases);
/* Bound of the device-side wait for a peer, in nanoseconds (default 2 s). */
int rg_b200_comm_set_wait_ns(rg_comm *, uint64_t ns);
int rg_b200_comm_status(rg_comm *); /* RG_OK, or RG_ERR_TIMEOUT once a kernel gave up waiting for a peer (sticky); synchronises the device */
int rg_b200_comm_destroy(rg_comm *);
typedef struct rg_all_reduce_params {
    int32_t dtype, op;
    uint64_t count;
} rg_all_reduce_params;
int rg_b200_all_reduce(rg_comm *, const rg_all_reduce_params *, const void *const *in, void *const *out, void *stream);

/* Row-parallel product + all-reduce as two halves that meet in peer memory, replacing MatMulCublas followed by AllReduceNccl
 * (src/04kernel/src/kernels/mat_mul/cublas_kernel.cu:48-55, src/04kernel/src/kernels/all_reduce/nccl_kernel.cu:9-19) where a
 * tensor-parallel layer multiplies by its slice of Wo / Wdown and sums the partial results over the ranks:
 *   rg_b200_mat_mul_push  — the tcgen05 product of up to 64 tokens (A [m, k] activations, B [n, k] weights, transB, no C, batch 1,
 *     n a multiple of 8, fp16 / bf16) whose epilogue does not write Y: every finished pair of 16-bit values goes, with the flag
 *     of the communicator's call in flight, straight into this rank's input slot on every peer (one-shot) or on the rank that
 *     owns the run of chunks (two-shot), by ordinary 8-byte stores over NVLink.  inputs {A, B}; workspace as
 *     rg_b200_mat_mul_workspace of the same parameters.  RG_ERR_UNSUPPORTED for any other shape (call rg_b200_mat_mul and
 *     rg_b200_all_reduce instead), RG_ERR_LIMIT when m * n * 2 exceeds the communicator's capacity.
 *   rg_b200_all_reduce_recv — the receiving half: the all-reduce kernel without its send phase (this rank's own input is read
 *     from its slot like a peer's).  inputs {residual or NULL}, outputs {y}; count * element size a multiple of 16.  It is the
 *     call that advances the communicator's sequence, so every rg_b200_mat_mul_push must be followed by exactly one
 *     rg_b200_all_reduce_recv of the same element count on the same stream, on every rank.
 * The result carries the same bits as the tcgen05 product (rg_b200_mat_mul, force_kernel 3) followed by rg_b200_all_reduce. */
int rg_b200_mat_mul_push(rg_comm *, const rg_mat_mul_params *, void *ws, const void *const *in, void *stream);
int rg_b200_all_reduce_recv(rg_comm *, const rg_all_reduce_params *, const void *const *in, void *const *out, void *stream);

/* AllReduce(Sum) + residual + RmsNormalization in one launch: the three operators that follow a row-parallel product of a
 * tensor-parallel decoder layer (AllReduceNccl, nccl_kernel.cu:9-19; BinaryCuda Add; RmsNormalizationCuda,
 * src/04kernel/src/kernels/rms_normalization/cuda_kernel.cc:24-131).  inputs {x [rows, dim], residual [rows, dim] or NULL,
 * w [dim]}, outputs {y = sum over ranks of x (+ residual), n = y * rsqrt(mean(y^2) + epsilon) * w}; RG_FP16 / RG_BF16;
 * dim a multiple of 8 and at most 16384 (a row is held in the registers of one CTA); rows * dim * 2 <= the capacity given
 * at create.  y and n carry the same bits as rg_b200_all_reduce followed by rg_b200_rms_norm.  Counts as one call of the
 * communicator's sequence; waits and failure behave as for rg_b200_all_reduce. */
typedef struct rg_all_reduce_norm_params {
    int32_t dtype;
    uint32_t rows, dim;
    float epsilon;
} rg_all_reduce_norm_params;
int rg_b200_all_reduce_norm(rg_comm *, const rg_all_reduce_norm_params *, const void *const *in, void *const *out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* RG_B200_H */
