// Fused decode linear layer  Y = epilogue(prologue(X) * W^T)  for m <= 4 rows of X: the HBM-bound weight
// streaming kernel that carries ~92 % of the bytes of a batch-1 decode step.
//
// Design (sm_100a):
//  * persistent grid, one CTA per SM; CTA c owns a contiguous range of "units".  A unit is 1 or 2 segments of g
//    consecutive rows of W[n,k] — two segments when the epilogue needs a pair of rows in the same CTA
//    (gate row j with up row j for SiLU; row i with row i + D/2 of one head for rotate-half RoPE).
//  * one producer thread streams each unit's segments (contiguous in memory, <= 32 KiB) into a 3-stage shared
//    memory ring with cp.async.bulk (the 1-D TMA copy) completing on full[] mbarriers; 8 consumer warps wait,
//    read the stage with conflict-free 128-bit shared loads and release it through empty[] mbarriers.
//  * X lives in registers as fp32 (each thread owns the 16-byte chunks tid, tid+256, ... of the k axis), with
//    the RMSNorm prologue (fp32 sum of squares, block reduce) applied in place, so the normalised activations
//    never touch HBM.
//  * per-unit row sums are reduced inside each warp by a halving butterfly (V values cost V-1+log2(32/V)
//    shuffles, fixed order => deterministic) and parked in shared memory; the epilogue runs once at the end.
//  * programmatic dependent launch: the weight stream does not depend on the previous kernel, so the producer
//    starts immediately and only the consumers execute griddepcontrol.wait before touching activations.
//  * every mbarrier wait is bounded (~2 s); on expiry the kernel records an error word and leaves normally.
#include "gemm_dispatch.cuh"
#include <cstdlib>

namespace rg {

constexpr int LS_NW = 8;                      // consumer warps
constexpr int LS_CONSUMERS = LS_NW * 32;      // 256
constexpr int LS_THREADS = LS_CONSUMERS + 32; // + producer warp
constexpr int LS_STAGES = 3;
constexpr uint32_t LS_STAGE_BYTES = 32768;
constexpr uint32_t LS_PART_MAX_BYTES = 64 * 1024;

static __device__ int s_linear_error;// 0 ok; 1 consumer wait expired; 2 producer wait expired
static __device__ int s_linear_index_error;// a cache-append position or block-table entry was out of range (store skipped)

struct LinearArgs {
    const void *W, *X, *G, *R;
    const int64_t *pos;
    const int32_t *table;
    void *Y, *kc, *vc;
    uint32_t m, n, k;
    int prologue, epilogue;
    float eps;
    uint32_t n_heads;
    float log2_theta;
    rg_kv_layout kv;
    uint32_t units, g, segs;
};

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(LS_CONSUMERS) : "memory"); }

// first row of segment s of unit u, and how many of its g rows exist
__device__ __forceinline__ uint32_t unit_row(const LinearArgs &a, uint32_t u, uint32_t s, uint32_t &rows) {
    if (a.epilogue == 3) {
        const uint32_t D = a.kv.head_dim, half = D / 2, per_head = half / a.g;
        rows = a.g;
        return (u / per_head) * D + s * half + (u % per_head) * a.g;
    }
    const uint32_t span = a.epilogue == 2 ? a.n / 2 : a.n;
    const uint32_t r0 = u * a.g;
    rows = span - r0 < a.g ? span - r0 : a.g;
    return s * span + r0;
}

template<int V> __device__ __forceinline__ void reduce_halving(float (&vals)[V], int lane) {
    int o = 16;
#pragma unroll
    for (int cnt = V; cnt > 1; cnt >>= 1) {
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < cnt / 2; ++i) {
            const float send = up ? vals[i] : vals[i + cnt / 2];
            const float keep = up ? vals[i + cnt / 2] : vals[i];
            vals[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
        o >>= 1;
    }
    for (; o > 0; o >>= 1) vals[0] += __shfl_xor_sync(0xffffffffu, vals[0], o);
}
template<int V> struct Log2 { static constexpr int value = 1 + Log2<V / 2>::value; };
template<> struct Log2<1> { static constexpr int value = 0; };

template<class T, int M, int KCH, int R>
__global__ void __launch_bounds__(LS_THREADS) linear_stream_kernel(const LinearArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + LS_STAGES * LS_STAGE_BYTES);
    uint64_t *empty = full + LS_STAGES;
    float *red = reinterpret_cast<float *>(empty + LS_STAGES);// 16 floats
    int *failed = reinterpret_cast<int *>(red + 16);
    float *part = red + 32;                                    // [local slot][LS_NW]

    constexpr int V = R * M;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t u0 = static_cast<uint32_t>(static_cast<uint64_t>(a.units) * blockIdx.x / gridDim.x);
    const uint32_t u1 = static_cast<uint32_t>(static_cast<uint64_t>(a.units) * (blockIdx.x + 1) / gridDim.x);
    const uint32_t nu = u1 - u0;
    const uint32_t row_bytes = a.k * 2u;

    if (tid == 0) {
        for (int s = 0; s < LS_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], LS_NW);
        }
        *failed = 0;
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == LS_NW) {
        // ---------------- producer: one thread streams this CTA's units through the ring --------------------
        if (lane == 0) {
            const uint64_t policy = l2_policy_evict_first();
            const uint8_t *W = static_cast<const uint8_t *>(a.W);
            for (uint32_t i = 0; i < nu; ++i) {
                const uint32_t s = i % LS_STAGES, ph = (i / LS_STAGES) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u)) {
                    atomicExch(&s_linear_error, 2);
                    break;
                }
                uint32_t rows;
                unit_row(a, u0 + i, 0, rows);
                const uint32_t seg_bytes = rows * row_bytes;
                mbar_arrive_expect_tx(&full[s], seg_bytes * a.segs);
                for (uint32_t sg = 0; sg < a.segs; ++sg) {
                    uint32_t rr;
                    const uint32_t row = unit_row(a, u0 + i, sg, rr);
                    bulk_g2s_hint(smem + s * LS_STAGE_BYTES + sg * a.g * row_bytes,
                                  W + static_cast<uint64_t>(row) * row_bytes, seg_bytes, &full[s], policy);
                }
            }
        }
        return;
    }

    // -------------------- consumers ----------------------------------------------------------------------
    pdl_wait();// activations (X, R, positions) come from the previous kernel
    const uint32_t kchunks = a.k / 8;
    float x[M][KCH][8];
    {
        const T *X = static_cast<const T *>(a.X);
        float ss[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
            ss[m] = 0.f;
#pragma unroll
            for (int c = 0; c < KCH; ++c) {
                const uint32_t ci = tid + c * LS_CONSUMERS;
                if (ci < kchunks && m < static_cast<int>(a.m)) {
                    const uint4 raw = *reinterpret_cast<const uint4 *>(X + static_cast<size_t>(m) * a.k + ci * 8);
                    unpack8<T>(raw, x[m][c]);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) x[m][c][j] = 0.f;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) ss[m] += x[m][c][j] * x[m][c][j];
            }
        }
        if (a.prologue == 1) {
            const T *G = static_cast<const T *>(a.G);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float v = warp_sum(ss[m]);
                if (lane == 0) red[warp] = v;
                consumer_bar();
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < LS_NW; ++w) tot += red[w];
                consumer_bar();
                const float rstd = rsqrtf(tot / static_cast<float>(a.k) + a.eps);
#pragma unroll
                for (int c = 0; c < KCH; ++c) {
                    const uint32_t ci = tid + c * LS_CONSUMERS;
                    if (ci < kchunks) {
                        float gw[8];
                        unpack8<T>(*reinterpret_cast<const uint4 *>(G + ci * 8), gw);
#pragma unroll
                        for (int j = 0; j < 8; ++j) x[m][c][j] *= rstd * gw[j];
                    }
                }
            }
        }
    }

    bool ok = true;
    for (uint32_t i = 0; i < nu; ++i) {
        const uint32_t s = i % LS_STAGES, ph = (i / LS_STAGES) & 1u;
        if (!mbar_wait(&full[s], ph)) {
            ok = false;
            break;
        }
        const uint8_t *st = smem + s * LS_STAGE_BYTES;
        float acc[V];
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int c = 0; c < KCH; ++c) {
                const uint32_t ci = tid + c * LS_CONSUMERS;
                if (ci < kchunks) {
                    float w[8];
                    unpack8<T>(*reinterpret_cast<const uint4 *>(st + static_cast<size_t>(r) * row_bytes + ci * 16), w);
#pragma unroll
                    for (int m = 0; m < M; ++m)
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[r * M + m] = fmaf(w[j], x[m][c][j], acc[r * M + m]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        reduce_halving<V>(acc, static_cast<int>(lane));
        constexpr int NB = Log2<V>::value;
        if ((lane & ((32u >> NB) - 1u)) == 0) part[(i * V + (lane >> (5 - NB))) * LS_NW + warp] = acc[0];
    }
    if (!ok) {
        *failed = 1;
        atomicExch(&s_linear_error, 1);
    }
    consumer_bar();
    if (*failed) return;

    // -------------------- epilogue: one item = (local unit, row r within g, m) ------------------------------
    const uint32_t g = a.g, S = a.segs;
    T *Y = static_cast<T *>(a.Y);
    for (uint32_t e = tid; e < nu * g * M; e += LS_CONSUMERS) {
        const uint32_t m = e % M, r = (e / M) % g, lu = e / (M * g), u = u0 + lu;
        if (m >= a.m) continue;
        float val[2] = {0.f, 0.f};
        for (uint32_t sg = 0; sg < S; ++sg) {
            const float *p = part + ((lu * V) + (sg * g + r) * M + m) * LS_NW;
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < LS_NW; ++w) t += p[w];
            val[sg] = t;
        }
        uint32_t rows;
        const uint32_t row0 = unit_row(a, u, 0, rows);
        if (r >= rows) continue;
        if (a.epilogue == 0) {
            Y[static_cast<size_t>(m) * a.n + row0 + r] = Num<T>::from_f(val[0]);
        } else if (a.epilogue == 1) {
            const size_t o = static_cast<size_t>(m) * a.n + row0 + r;
            Y[o] = Num<T>::from_f(val[0] + Num<T>::to_f(static_cast<const T *>(a.R)[o]));
        } else if (a.epilogue == 2) {
            const float gt = val[0];
            Y[static_cast<size_t>(m) * (a.n / 2) + row0 + r] = Num<T>::from_f(gt / (1.f + expf(-gt)) * val[1]);
        } else {
            const uint32_t D = a.kv.head_dim, half = D / 2, nq = a.n_heads, nkv = a.kv.n_kv_heads;
            const uint32_t h = row0 / D, i = row0 % D + r;// i < half
            const int64_t t = a.pos[m];
            float lo = val[0], hi = val[1];
            if (h < nq + nkv) {
                const float inv_freq = exp2f(-a.log2_theta * (2.0f * static_cast<float>(i) / static_cast<float>(D)));
                float sn, cs;
                sincosf(static_cast<float>(t) * inv_freq, &sn, &cs);
                const float a0 = lo * cs - hi * sn, b0 = hi * cs + lo * sn;
                lo = a0, hi = b0;
            }
            if (h < nq) {
                T *q = Y + static_cast<size_t>(m) * nq * D + h * D;
                q[i] = Num<T>::from_f(lo);
                q[i + half] = Num<T>::from_f(hi);
            } else {
                const bool is_k = h < nq + nkv;
                const uint32_t kvh = is_k ? h - nq : h - nq - nkv;
                T *cache = static_cast<T *>(is_k ? a.kc : a.vc);
                size_t base;
                if (!kv_pos_ok(t, a.kv, a.table != nullptr)) {
                    s_linear_index_error = 1;
                    continue;
                }
                if (a.table) {
                    const uint32_t page = a.kv.page_size;
                    const int32_t blk = a.table[static_cast<size_t>(m) * a.kv.max_blocks_per_seq + static_cast<uint32_t>(t) / page];
                    if (!kv_block_ok(blk, a.kv)) {
                        s_linear_index_error = 1;
                        continue;
                    }
                    base = ((static_cast<size_t>(blk) * nkv + kvh) * page + static_cast<uint32_t>(t) % page) * D;
                } else {
                    base = ((static_cast<size_t>(m) * nkv + kvh) * a.kv.max_seq + static_cast<size_t>(t)) * D;
                }
                cache[base + i] = Num<T>::from_f(lo);
                cache[base + i + half] = Num<T>::from_f(hi);
            }
        }
    }
}

// ---- host ---------------------------------------------------------------------------------------
template<class Kern>
static int launch_stream_kernel(Kern kern, const LinearArgs &a, unsigned grid, size_t smem, cudaStream_t st) {
    RG_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(LS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    RG_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
    count_launch();
    return RG_OK;
}

static uint32_t pow2_floor(uint32_t v) {
    uint32_t p = 1;
    while (p * 2 <= v) p *= 2;
    return p;
}

struct LinearPlan {
    uint32_t g, segs, units, kch, grid;
    size_t smem;
};

static int linear_plan(const rg_linear_params *p, LinearPlan &pl) {
    if (p->dtype != RG_FP16 && p->dtype != RG_BF16) return RG_ERR_DTYPE;
    if (p->m == 0 || p->m > 4 || p->n == 0 || p->k == 0 || p->k % 8 != 0) return RG_ERR_SHAPE;
    if (p->prologue < 0 || p->prologue > 1 || p->epilogue < 0 || p->epilogue > 3) return RG_ERR_UNSUPPORTED;
    const uint32_t row_bytes = p->k * 2;
    pl.segs = p->epilogue >= 2 ? 2 : 1;
    if (row_bytes * pl.segs > LS_STAGE_BYTES) return RG_ERR_SHAPE;
    uint32_t g = pow2_floor(LS_STAGE_BYTES / (row_bytes * pl.segs));
    const uint32_t mm = p->m <= 1 ? 1 : p->m <= 2 ? 2 : 4;
    while (g > 1 && g * pl.segs * mm > 8) g /= 2;// keep V = R*M <= 8 accumulators
    if (g * pl.segs > 4) g = 4 / pl.segs;
    if (p->epilogue == 2) {
        if (p->n % 2 != 0) return RG_ERR_SHAPE;
        pl.units = (p->n / 2 + g - 1) / g;
    } else if (p->epilogue == 3) {
        const uint32_t D = p->kv.head_dim;
        if (D == 0 || D % 2 != 0 || p->n != (p->n_heads + 2 * p->kv.n_kv_heads) * D) return RG_ERR_SHAPE;
        while (g > 1 && (D / 2) % g != 0) g /= 2;
        pl.units = p->n / (2 * g);
    } else {
        pl.units = (p->n + g - 1) / g;
    }
    pl.g = g;
    const uint32_t need = (p->k / 8 + LS_CONSUMERS - 1) / LS_CONSUMERS;
    pl.kch = need <= 2 ? 2 : need <= 4 ? 4 : need <= 6 ? 6 : 8;
    if (need > 8) return RG_ERR_SHAPE;
    if (mm * pl.kch > 8) return RG_ERR_SHAPE;// x registers: M*KCH*8 <= 64 floats
    pl.grid = static_cast<uint32_t>(sm_count());
    if (pl.grid > pl.units) pl.grid = pl.units;
    const uint32_t max_local = (pl.units + pl.grid - 1) / pl.grid;
    const size_t part_bytes = static_cast<size_t>(max_local) * g * pl.segs * mm * LS_NW * 4;
    if (part_bytes > LS_PART_MAX_BYTES) return RG_ERR_SHAPE;
    pl.smem = LS_STAGES * LS_STAGE_BYTES + 2 * LS_STAGES * 8 + 32 * 4 + part_bytes;
    return RG_OK;
}

template<class T>
static int linear_dispatch(const LinearArgs &a, const LinearPlan &pl, uint32_t mm, cudaStream_t st) {
    const uint32_t R = pl.g * pl.segs;
#define RG_LS(M_, K_, R_)                                                                                     \
    if (mm == M_ && pl.kch == K_ && R == R_)                                                                  \
        return launch_stream_kernel(linear_stream_kernel<T, M_, K_, R_>, a, pl.grid, pl.smem, st);
#define RG_LS_R(M_, K_) RG_LS(M_, K_, 1) RG_LS(M_, K_, 2) RG_LS(M_, K_, 4)
    RG_LS_R(1, 2)
    RG_LS_R(1, 4)
    RG_LS_R(1, 6)
    RG_LS_R(1, 8)
    RG_LS_R(2, 2)
    RG_LS_R(2, 4)
    RG_LS(4, 2, 1)
    RG_LS(4, 2, 2)
#undef RG_LS_R
#undef RG_LS
    return RG_ERR_UNSUPPORTED;
}

int linear_stream(const rg_linear_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    LinearPlan pl;
    const int rc = linear_plan(p, pl);
    if (rc != RG_OK) return rc;
    LinearArgs a = {};
    a.X = in[0], a.W = in[1], a.G = in[2], a.R = in[3];
    a.pos = static_cast<const int64_t *>(in[4]);
    a.table = static_cast<const int32_t *>(in[5]);
    a.Y = out[0], a.kc = out[1], a.vc = out[2];
    if (!a.X || !a.W || !a.Y) return RG_ERR_NULL;
    if (p->prologue == 1 && !a.G) return RG_ERR_NULL;
    if (p->epilogue == 1 && !a.R) return RG_ERR_NULL;
    if (p->epilogue == 3 && (!a.pos || !a.kc || !a.vc)) return RG_ERR_NULL;
    if (p->epilogue == 3 && a.table && p->kv.page_size == 0) return RG_ERR_SHAPE;
    if (!aligned16(a.X) || !aligned16(a.W) || (a.G && !aligned16(a.G))) return RG_ERR_ALIGN;
    a.m = p->m, a.n = p->n, a.k = p->k;
    a.prologue = p->prologue, a.epilogue = p->epilogue;
    a.eps = p->epsilon, a.n_heads = p->n_heads;
    a.log2_theta = p->epilogue == 3 ? log2f(p->theta) : 0.f;
    a.kv = p->kv;
    a.units = pl.units, a.g = pl.g, a.segs = pl.segs;
    const uint32_t mm = p->m <= 1 ? 1 : p->m <= 2 ? 2 : 4;
    return p->dtype == RG_FP16 ? linear_dispatch<__half>(a, pl, mm, st) : linear_dispatch<__nv_bfloat16>(a, pl, mm, st);
}

int linear_error_word(bool clear) { return error_symbol(s_linear_error, clear); }
int linear_index_error_word(bool clear) { return error_symbol(s_linear_index_error, clear); }

}// namespace rg

using namespace rg;

extern "C" {
// 5..32 tokens without a norm prologue: the skinny weight-streaming kernel (linear_skinny.cu)
// SiLU gate on 5..64 tokens: the tcgen05 kernel with the weights on the M side, except for the few-rows / long-k shape the
// streaming skinny kernel is faster on (the rule of the plain product)
static bool linear_is_tc_swiglu_small(const rg_linear_params *p) {
    if (!gemm_tc_swiglu_small_shape(p)) return false;
    const bool skinny_wins = p->m <= 16 && p->n <= 2560 && p->k >= 4096 && linear_skinny_shape(p->dtype, p->m, p->n, p->k);
    return !skinny_wins;
}
// QKV split + RoPE + append on 5..64 tokens: the streaming skinny kernel where it applies (up to 32 tokens, k a multiple of 128);
// the tcgen05 form takes the rest.  Its epilogue is slow — 64 threads of a tile evaluate the rotation angles of every token on
// the last-arriving CTA's critical path: the batch-32 decode step measured 13.0 ms with it against 11.6 ms with the product
// followed by the separate rotation kernel — so the fusion pass only uses it on request.
static bool linear_is_tc_qkv_small(const rg_linear_params *p) {
    if (!gemm_tc_qkv_rope_small_shape(p)) return false;
    const bool skinny = p->m <= 32 && linear_skinny_shape(p->dtype, p->m, p->n, p->k);
    return !skinny;
}
static bool linear_is_skinny(const rg_linear_params *p) {
    return p->m > 4 && p->m <= 32 && p->prologue == 0 && linear_skinny_shape(p->dtype, p->m, p->n, p->k);
}
size_t rg_b200_linear_workspace(const rg_linear_params *p) {
    if (!p) return 0;
    if (linear_is_tc_swiglu_small(p)) return gemm_tc_swiglu_small_workspace(p);
    if (linear_is_tc_qkv_small(p)) return gemm_tc_qkv_rope_small_workspace(p);
    if (!linear_is_skinny(p)) return 0;
    return linear_skinny_workspace(p->dtype, p->m, p->n, p->k, p->epilogue, &p->kv, p->n_heads);
}
int rg_b200_linear(const rg_linear_params *p, void *ws, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out) return RG_ERR_NULL;
    if (linear_is_tc_swiglu_small(p)) return gemm_tc_swiglu_small(p, ws, in, out, static_cast<cudaStream_t>(stream));
    if (linear_is_tc_qkv_small(p)) return gemm_tc_qkv_rope_small(p, ws, in, out, static_cast<cudaStream_t>(stream));
    if (linear_is_skinny(p)) {
        SkinnyCall c = {};
        c.dtype = p->dtype, c.m = p->m, c.n = p->n, c.k = p->k, c.epilogue = p->epilogue;
        c.alpha = 1.f, c.beta = 1.f;
        const uint32_t n_out = p->epilogue == 2 ? p->n / 2 : p->epilogue == 3 ? p->n_heads * p->kv.head_dim : p->n;
        c.c_row_stride = n_out, c.c_col_stride = 1, c.y_row_stride = n_out;
        c.n_heads = p->n_heads, c.theta = p->theta, c.kv = p->kv, c.tokens_per_seq = p->tokens_per_seq;
        c.w_static = 1;// as for the m <= 4 kernel: W is a weight, nothing earlier in the stream writes it
        const void *lin[5] = {in[0], in[1], in[3], in[4], in[5]};
        return linear_skinny(c, ws, lin, out, static_cast<cudaStream_t>(stream));
    }
    // many tokens (prefill): the QKV projection runs on the tensor cores with the same epilogue
    if (p->m > 64 && p->epilogue == 3) return gemm_tc_qkv_rope(p, in, out, static_cast<cudaStream_t>(stream));
    if (p->m > 64 && p->epilogue == 2) return gemm_tc_swiglu(p, in, out, static_cast<cudaStream_t>(stream));
    return linear_stream(p, in, out, static_cast<cudaStream_t>(stream));
}
}
