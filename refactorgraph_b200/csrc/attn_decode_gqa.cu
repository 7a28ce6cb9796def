// Split-K flash-decoding for grouped-query attention (head_dim 128, fp16 / bf16, 2..16 query heads per KV head).
//
// The plain decode kernel runs one CTA per (sequence, QUERY head), so with 8 query heads per KV head every K/V tile is
// fetched eight times (from L2).  Here one CTA owns a run of 64-key tiles of one (sequence, KV head) and serves all
// query heads of the group at once: the group's queries are the (zero-padded) 16 rows of an mma.sync.m16n8k16 tile, so
// a K/V tile is loaded once (16-byte cp.async, XOR-swizzled, double-buffered; contiguous or paged cache) and reused by
// every query head.  Each warp takes 16 of the tile's 64 keys with its own online-softmax state; the four states are
// merged in shared memory, the per-split records go to the workspace and the last CTA of a (sequence, KV head) to
// arrive merges the splits (self-resetting counter), exactly like attn_decode_kernel.
#include "common.cuh"

namespace rg {

constexpr int GQ_THREADS = 128, GQ_TILE = 64, GQ_D = 128;
constexpr int GQ_STAGES = 3;// K/V tile buffers: two tiles in flight while one is consumed (2 CTAs per SM)
constexpr int GQ_REC = GQ_D + 4;// floats per split record: max, sum, 2 pad, accumulator (16-byte aligned)

static __device__ int s_gqa_index_error;// a sequence length or block-table entry was out of range (length clamped, block 0 read instead)
int gqa_index_error_word(bool clear) { return error_symbol(s_gqa_index_error, clear); }

struct GqaArgs {
    const void *q, *kc, *vc;
    const int64_t *lens;
    const int32_t *table;
    void *o;
    float *part;
    unsigned *cnt;
    uint32_t batch, n_heads, tiles_per_split, max_splits, max_len;
    rg_kv_layout kv;
    float scale_log2e;
};

template<class T> struct GMma;
template<> struct GMma<__half> {
    static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
};
template<> struct GMma<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
};
__device__ __forceinline__ void g_ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void g_ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void g_cp_async16(uint32_t dst, const void *src, bool valid) {
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ uint32_t g_sw(uint32_t r, uint32_t c) { return r * 256u + ((c ^ (r & 7u)) << 4); }

template<class T>
__global__ void __launch_bounds__(GQ_THREADS) attn_decode_gqa_kernel(const GqaArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sQ = smem_u32(smem), sK = sQ + 4096, sV = sK + GQ_STAGES * 16384;
    float *mbuf = reinterpret_cast<float *>(smem + 4096);// [4 warps][16 rows][D + 2], aliases the K/V tiles after the loop
    __shared__ int s_last;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const uint32_t nkv = a.kv.n_kv_heads, gq = a.n_heads / nkv, h0 = kvh * gq;

    pdl_launch_dependents();
    pdl_wait();
    const int64_t len64 = a.lens[b];
    const uint32_t len = kv_len_clamped(len64, a.max_len, a.kv, a.table != nullptr, &s_gqa_index_error);
    const uint32_t ntiles = (len + GQ_TILE - 1) / GQ_TILE;
    const uint32_t nsplit = (ntiles + a.tiles_per_split - 1) / a.tiles_per_split;
    T *O = static_cast<T *>(a.o) + (static_cast<size_t>(b) * a.n_heads + h0) * GQ_D;
    if (len == 0) {
        if (split == 0)
            for (uint32_t i = threadIdx.x; i < gq * GQ_D; i += GQ_THREADS) O[i] = Num<T>::from_f(0.f);
        return;
    }
    if (split >= nsplit) return;
    const uint32_t t0 = split * a.tiles_per_split;
    const uint32_t t1 = t0 + a.tiles_per_split < ntiles ? t0 + a.tiles_per_split : ntiles;
    const T *Q = static_cast<const T *>(a.q) + (static_cast<size_t>(b) * a.n_heads + h0) * GQ_D;
    const T *KC = static_cast<const T *>(a.kc), *VC = static_cast<const T *>(a.vc);

    auto load_tile = [&](uint32_t tile, uint32_t buf) {
        // 64 keys x 16 chunks for K and for V, 8 + 8 chunks per thread; keys >= len are zero-filled
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t id = threadIdx.x + i * GQ_THREADS, r = id >> 4, c = id & 15u;
            const uint32_t key = tile * GQ_TILE + r;
            const bool valid = key < len;
            size_t off = 0;
            if (valid) {
                if (a.table) {
                    const uint32_t page = a.kv.page_size;
                    int32_t blk = a.table[static_cast<size_t>(b) * a.kv.max_blocks_per_seq + key / page];
                    if (!kv_block_ok(blk, a.kv)) s_gqa_index_error = 1, blk = 0;
                    off = ((static_cast<size_t>(blk) * nkv + kvh) * page + key % page) * GQ_D;
                } else {
                    off = ((static_cast<size_t>(b) * nkv + kvh) * a.kv.max_seq + key) * GQ_D;
                }
            }
            g_cp_async16(sK + buf * 16384 + g_sw(r, c), KC + off + c * 8, valid);
            g_cp_async16(sV + buf * 16384 + g_sw(r, c), VC + off + c * 8, valid);
        }
    };
    // queries of the group: 16 rows x 16 chunks, rows >= gq zero
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint32_t id = threadIdx.x + i * GQ_THREADS, r = id >> 4, c = id & 15u;
        g_cp_async16(sQ + g_sw(r, c), Q + static_cast<size_t>(r < gq ? r : 0) * GQ_D + c * 8, r < gq);
    }
    load_tile(t0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");// group 0: queries + first tile
    if (t0 + 1 < t1) load_tile(t0 + 1, 1);
    asm volatile("cp.async.commit_group;" ::: "memory");// group 1: second tile (possibly empty)
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();

    uint32_t qf[8][4];
    {
        const uint32_t m = lane >> 3, rin = lane & 7u;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) g_ldsm_x4(qf[kk], sQ + g_sw((m & 1u) * 8 + rin, 2 * kk + (m >> 1)));
    }
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    for (uint32_t tile = t0; tile < t1; ++tile) {
        // on entry tile `tile` has landed and every thread is past the previous tile's math, so the buffer that tile held
        // ((i + 2) % 3) can take tile + 2: two tiles stay in flight while this one is consumed
        const uint32_t buf = (tile - t0) % GQ_STAGES;
        if (tile + 2 < t1) load_tile(tile + 2, (tile - t0 + 2) % GQ_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const uint32_t sKb = sK + buf * 16384, sVb = sV + buf * 16384;
        const uint32_t m = lane >> 3, rin = lane & 7u;
        // S = Q K^T for this warp's 16 keys (two 8-key blocks)
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            uint32_t kf[4];
            g_ldsm_x4(kf, sKb + g_sw(warp * 16 + (m >> 1) * 8 + rin, 2 * kk + (m & 1u)));
            GMma<T>::run(s[0], qf[kk], kf[0], kf[1]);
            GMma<T>::run(s[1], qf[kk], kf[2], kf[3]);
        }
        const uint32_t key0 = tile * GQ_TILE + warp * 16;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t key = key0 + nb * 8 + 2 * t + (e & 1);
                s[nb][e] = key < len ? s[nb][e] * a.scale_log2e : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[nb][e]);
            }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            corr[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
        }
        float p[2][4], rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                p[nb][e] = (m_run[r] == -INFINITY) ? 0.f : exp2f(s[nb][e] - m_run[r]);
                rs[r] += p[nb][e];
            }
        const uint32_t pf[4] = {GMma<T>::pack(p[0][0], p[0][1]), GMma<T>::pack(p[0][2], p[0][3]), GMma<T>::pack(p[1][0], p[1][1]),
                                GMma<T>::pack(p[1][2], p[1][3])};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
            l_run[r] = l_run[r] * corr[r] + rs[r];
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            o[i][0] *= corr[0], o[i][1] *= corr[0];
            o[i][2] *= corr[1], o[i][3] *= corr[1];
        }
#pragma unroll
        for (int db = 0; db < 16; db += 2) {
            uint32_t vf[4];
            g_ldsm_x4_t(vf, sVb + g_sw(warp * 16 + (m & 1u) * 8 + rin, db + (m >> 1)));
            GMma<T>::run(o[db], pf, vf[0], vf[1]);
            GMma<T>::run(o[db + 1], pf, vf[2], vf[3]);
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");// all but the newest group: the next tile is there
        __syncthreads();
    }
    // ---- merge the four warps (each saw a quarter of every tile) ----
    {
        float *mine = mbuf + static_cast<size_t>(warp) * 16 * (GQ_D + 2);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float *row = mine + (g + 8 * r) * (GQ_D + 2);
            if (t == 0) row[0] = m_run[r], row[1] = l_run[r];
#pragma unroll
            for (int db = 0; db < 16; ++db) {
                row[2 + db * 8 + 2 * t] = o[db][2 * r];
                row[2 + db * 8 + 2 * t + 1] = o[db][2 * r + 1];
            }
        }
    }
    __syncthreads();
    const size_t rec0 = (static_cast<size_t>(b) * a.n_heads + h0) * a.max_splits;
    for (uint32_t r = 0; r < gq; ++r) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mbuf[(static_cast<size_t>(w) * 16 + r) * (GQ_D + 2)]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float *row = mbuf + (static_cast<size_t>(w) * 16 + r) * (GQ_D + 2);
            const float f = row[0] == -INFINITY ? 0.f : exp2f(row[0] - M);
            L += row[1] * f;
            acc += row[2 + threadIdx.x] * f;
        }
        if (nsplit == 1) {
            O[r * GQ_D + threadIdx.x] = Num<T>::from_f(acc / L);
        } else {
            float *rec = a.part + (rec0 + static_cast<size_t>(r) * a.max_splits + split) * GQ_REC;
            rec[4 + threadIdx.x] = acc;
            if (threadIdx.x == 0) rec[0] = M, rec[1] = L;
        }
    }
    if (nsplit == 1) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&a.cnt[static_cast<size_t>(b) * nkv + kvh], 1u) == nsplit - 1 ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // The last CTA of the group merges the records: warp w takes heads w, w + 4, ...; a lane reads one record header per
    // round (all headers in one round trip), then owns four output dims and streams the records with independent
    // 16-byte loads (a dependent chain of loads here costs a round trip to L2 per split).
    for (uint32_t r = warp; r < gq; r += GQ_THREADS / 32) {
        const float *base = a.part + (rec0 + static_cast<size_t>(r) * a.max_splits) * GQ_REC;
        float M = -INFINITY;
        for (uint32_t s0 = 0; s0 < nsplit; s0 += 32)
            if (s0 + lane < nsplit) M = fmaxf(M, __ldcg(base + static_cast<size_t>(s0 + lane) * GQ_REC));
        M = warp_max(M);
        float den = 0.f;
        float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t s0 = 0; s0 < nsplit; s0 += 32) {
            float2 ml = make_float2(-INFINITY, 0.f);
            if (s0 + lane < nsplit) ml = __ldcg(reinterpret_cast<const float2 *>(base + static_cast<size_t>(s0 + lane) * GQ_REC));
            const float w = ml.x == -INFINITY ? 0.f : exp2f(ml.x - M);
            den += ml.y * w;
            const uint32_t cnt = nsplit - s0 < 32 ? nsplit - s0 : 32;
#pragma unroll 8
            for (uint32_t j = 0; j < cnt; ++j) {
                const float wj = __shfl_sync(0xffffffffu, w, j);
                const float4 v = __ldcg(reinterpret_cast<const float4 *>(base + static_cast<size_t>(s0 + j) * GQ_REC + 4 + lane * 4));
                num.x += v.x * wj, num.y += v.y * wj, num.z += v.z * wj, num.w += v.w * wj;
            }
        }
        const float inv = 1.f / warp_sum(den);
        T ov[4] = {Num<T>::from_f(num.x * inv), Num<T>::from_f(num.y * inv), Num<T>::from_f(num.z * inv), Num<T>::from_f(num.w * inv)};
        *reinterpret_cast<uint2 *>(O + r * GQ_D + lane * 4) = *reinterpret_cast<const uint2 *>(ov);
    }
    if (threadIdx.x == 0) a.cnt[static_cast<size_t>(b) * nkv + kvh] = 0u;
}

struct GqaPlan {
    uint32_t tiles_per_split, max_splits;
    size_t cnt_bytes, part_bytes;
};
static GqaPlan gqa_plan(const rg_attn_decode_params *p) {
    GqaPlan pl;
    const uint32_t total_tiles = (p->max_len + GQ_TILE - 1) / GQ_TILE;
    const uint64_t groups = static_cast<uint64_t>(p->batch) * p->kv.n_kv_heads;
    // All CTAs of the launch should be resident together (2 per SM with three 32 KiB tile buffers): one CTA more than the slots and the launch takes two
    // rounds (16 sequences x 4 KV heads: 7 splits = 448 CTAs on 444 slots took 41 us).
    const uint64_t slots = 2ull * sm_count();
    uint32_t want = static_cast<uint32_t>(slots / (groups ? groups : 1));
    if (want < 1) want = 1;
    if (want > total_tiles) want = total_tiles ? total_tiles : 1;
    pl.tiles_per_split = total_tiles ? (total_tiles + want - 1) / want : 1;
    pl.max_splits = total_tiles ? (total_tiles + pl.tiles_per_split - 1) / pl.tiles_per_split : 1;
    pl.cnt_bytes = (groups * 4 + 255) / 256 * 256;
    pl.part_bytes = static_cast<size_t>(p->batch) * p->n_heads * pl.max_splits * GQ_REC * 4;
    return pl;
}

bool attn_decode_gqa_applies(const rg_attn_decode_params *p) {
    if (p->kv.head_dim != GQ_D || p->kv.n_kv_heads == 0) return false;
    const uint32_t gq = p->n_heads / p->kv.n_kv_heads;
    static const uint32_t gq_min = getenv("RG_B200_GQA_MIN") ? static_cast<uint32_t>(atoi(getenv("RG_B200_GQA_MIN"))) : 2u;
    return gq >= gq_min && gq <= 16 && (p->dtype == RG_FP16 || p->dtype == RG_BF16);
}
size_t attn_decode_gqa_workspace(const rg_attn_decode_params *p) {
    const GqaPlan pl = gqa_plan(p);
    return pl.cnt_bytes + pl.part_bytes;
}
size_t attn_decode_gqa_counter_bytes(const rg_attn_decode_params *p) { return gqa_plan(p).cnt_bytes; }

int attn_decode_gqa_launch(const rg_attn_decode_params *p, void *ws, const void *const *in, void *const *out, cudaStream_t st, bool pdl) {
    const GqaPlan pl = gqa_plan(p);
    GqaArgs a = {};
    a.q = in[0], a.kc = in[1], a.vc = in[2];
    a.lens = static_cast<const int64_t *>(in[3]);
    a.table = static_cast<const int32_t *>(in[4]);
    a.o = out[0];
    a.cnt = static_cast<unsigned *>(ws);
    a.part = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + pl.cnt_bytes);
    a.batch = p->batch, a.n_heads = p->n_heads;
    a.tiles_per_split = pl.tiles_per_split, a.max_splits = pl.max_splits, a.max_len = p->max_len;
    a.kv = p->kv;
    a.scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(GQ_D));
    const size_t smem = 4096 + 2 * GQ_STAGES * 16384;
    void (*kern)(const GqaArgs) = p->dtype == RG_FP16 ? attn_decode_gqa_kernel<__half> : attn_decode_gqa_kernel<__nv_bfloat16>;
    RG_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.max_splits, p->kv.n_kv_heads, p->batch);
    cfg.blockDim = dim3(GQ_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    RG_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
    count_launch();
    return RG_OK;
}

}// namespace rg
