// Attention for the decoder path.  The reference declares AttentionCuda::lower without defining it
// (src/04kernel/src/kernels/attention/cuda_kernel.hh:23-25); semantics are the operator spec
// src/08-01llm/README.md:29-63: causal multi-head self-attention with an optional KV cache, query head h uses
// kv head h / (n_heads / n_kv_heads), scores scaled by 1/sqrt(head_dim), fp32 softmax and accumulation.
//
//  * attn_decode_kernel  — split-K flash-decoding for one new token per sequence over a contiguous or paged
//    cache.  Each CTA owns a run of 64-token tiles of one (sequence, head); K and V tiles are staged into a
//    double-buffered shared-memory ring by cp.async.bulk (one copy per tile, or per 16-token page) completing on
//    mbarriers; scores, online softmax and P*V run from shared memory with conflict-free 128-bit loads; the
//    per-split (max, sum, acc) records go to the workspace and the last CTA to arrive merges them.
//  * kv_append_kernel / attn_rows_kernel — cache append and a general (prefill or decode) kernel on the
//    reference tensor layout, one warp per query row with online softmax.
#include "common.cuh"
#include <cstdlib>

namespace rg {

static __device__ int s_attn_error;
static __device__ int s_attn_index_error;// a sequence length or block-table entry was out of range (length clamped, block 0 read instead)

constexpr int AD_THREADS = 128;
constexpr int AD_TILE = 64;

struct DecodeArgs {
    const void *q, *kc, *vc;
    const int64_t *lens;
    const int32_t *table;
    void *o;
    float *part;
    unsigned *cnt;
    uint32_t batch, n_heads, tiles_per_split, max_splits, max_len;
    rg_kv_layout kv;
    float scale;
};

template<class T, int D>
__global__ void __launch_bounds__(AD_THREADS) attn_decode_kernel(const DecodeArgs a) {
    constexpr int CPR = D / 8;            // 16-byte chunks per row
    constexpr int CPT = CPR / 2;          // chunks per thread in the QK phase (2 threads per token)
    constexpr int NTG = AD_THREADS / CPR; // token groups in the PV phase
    constexpr uint32_t TILE_BYTES = AD_TILE * D * 2;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *stage = smem;// [2][K tile | V tile]
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + 4 * TILE_BYTES);
    float *qs = reinterpret_cast<float *>(full + 2);// [D]
    float *sc = qs + D;                             // [AD_TILE] scores then probabilities
    float *red = sc + AD_TILE;                      // [NTG][D]
    __shared__ int s_last;

    const uint32_t split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const uint32_t tid = threadIdx.x, lane = tid & 31;
    const uint32_t nkv = a.kv.n_kv_heads, kvh = h / (a.n_heads / nkv);

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();

    const int64_t len64 = a.lens[b];
    const uint32_t len = kv_len_clamped(len64, a.max_len, a.kv, a.table != nullptr, &s_attn_index_error);
    const uint32_t ntiles = (len + AD_TILE - 1) / AD_TILE;
    const uint32_t nsplit = (ntiles + a.tiles_per_split - 1) / a.tiles_per_split;
    T *o = static_cast<T *>(a.o) + (static_cast<size_t>(b) * a.n_heads + h) * D;
    if (len == 0) {
        if (split == 0 && tid < D) o[tid] = Num<T>::from_f(0.f);
        return;
    }
    if (split >= nsplit) return;
    const uint32_t t0 = split * a.tiles_per_split;
    const uint32_t t1 = t0 + a.tiles_per_split < ntiles ? t0 + a.tiles_per_split : ntiles;

    if (tid < D) qs[tid] = Num<T>::to_f(static_cast<const T *>(a.q)[(static_cast<size_t>(b) * a.n_heads + h) * D + tid]);

    auto issue = [&](uint32_t t, uint32_t s) {
        // thread 0 only: stage tile t into buffer s
        const uint32_t tok0 = t * AD_TILE;
        const uint32_t ntok = len - tok0 < AD_TILE ? len - tok0 : AD_TILE;
        uint8_t *ks = stage + s * 2 * TILE_BYTES, *vs = ks + TILE_BYTES;
        const uint8_t *kc = static_cast<const uint8_t *>(a.kc), *vc = static_cast<const uint8_t *>(a.vc);
        mbar_arrive_expect_tx(&full[s], 2u * ntok * D * 2u);
        if (!a.table) {
            const size_t off = ((static_cast<size_t>(b) * nkv + kvh) * a.kv.max_seq + tok0) * D * 2;
            bulk_g2s(ks, kc + off, ntok * D * 2u, &full[s]);
            bulk_g2s(vs, vc + off, ntok * D * 2u, &full[s]);
        } else {
            const uint32_t page = a.kv.page_size;
            const uint32_t step = page < AD_TILE ? page : AD_TILE;// tokens per copy
            for (uint32_t done = 0; done < ntok; done += step) {
                const uint32_t tok = tok0 + done;
                const uint32_t n = ntok - done < step ? ntok - done : step;
                int32_t blk = a.table[static_cast<size_t>(b) * a.kv.max_blocks_per_seq + tok / page];
                if (!kv_block_ok(blk, a.kv)) s_attn_index_error = 1, blk = 0;
                const size_t off = ((static_cast<size_t>(blk) * nkv + kvh) * page + tok % page) * D * 2;
                bulk_g2s(ks + done * D * 2, kc + off, n * D * 2u, &full[s]);
                bulk_g2s(vs + done * D * 2, vc + off, n * D * 2u, &full[s]);
            }
        }
    };

    float m_run = -INFINITY, l_run = 0.f;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    const uint32_t cg = tid % CPR, tg = tid / CPR;
    bool ok = true;

    if (tid == 0) issue(t0, 0);
    __syncthreads();// qs visible
    for (uint32_t t = t0; t < t1; ++t) {
        const uint32_t it = t - t0, s = it & 1u;
        if (tid == 0 && t + 1 < t1) issue(t + 1, s ^ 1u);
        // every thread waits (bounded) and the outcome is made uniform before anyone proceeds
        if (!__syncthreads_and(mbar_wait(&full[s], (it >> 1) & 1u) ? 1 : 0)) {
            ok = false;
            break;
        }
        const uint32_t tok0 = t * AD_TILE;
        const uint32_t ntok = len - tok0 < AD_TILE ? len - tok0 : AD_TILE;
        const uint8_t *ks = stage + s * 2 * TILE_BYTES, *vs = ks + TILE_BYTES;
        // ---- scores: two threads per token ----
        {
            const uint32_t tk = tid >> 1, hf = tid & 1u;
            const uint32_t sw = (D == 128) ? (tid & 7u) : ((tid >> 1) & 3u);
            float dot = 0.f;
            if (tk < ntok) {
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    const uint32_t cc = hf * CPT + (static_cast<uint32_t>(c) ^ sw);
                    float kf[8];
                    unpack8<T>(*reinterpret_cast<const uint4 *>(ks + tk * (D * 2) + cc * 16), kf);
                    const float4 q0 = *reinterpret_cast<const float4 *>(qs + cc * 8);
                    const float4 q1 = *reinterpret_cast<const float4 *>(qs + cc * 8 + 4);
                    dot += kf[0] * q0.x + kf[1] * q0.y + kf[2] * q0.z + kf[3] * q0.w + kf[4] * q1.x + kf[5] * q1.y +
                           kf[6] * q1.z + kf[7] * q1.w;
                }
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            if (hf == 0) sc[tk] = tk < ntok ? dot * a.scale : -INFINITY;
        }
        __syncthreads();
        // ---- online softmax statistics (every warp computes the same numbers) ----
        const float s0 = sc[lane], s1 = sc[lane + 32];
        const float tmax = warp_max(fmaxf(s0, s1));
        const float m_new = fmaxf(m_run, tmax);
        const float p0 = expf(s0 - m_new), p1 = expf(s1 - m_new);
        const float corr = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
        l_run = l_run * corr + warp_sum(p0 + p1);
        m_run = m_new;
        __syncthreads();// all reads of the raw scores done
        if (tid < 32) {
            sc[lane] = p0;
            sc[lane + 32] = p1;
        }
        __syncthreads();
        // ---- P*V: thread = (chunk cg of the row, token group tg) ----
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= corr;
        for (uint32_t tk = tg; tk < ntok; tk += NTG) {
            const float p = sc[tk];
            float vf[8];
            unpack8<T>(*reinterpret_cast<const uint4 *>(vs + tk * (D * 2) + cg * 16), vf);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = fmaf(p, vf[j], acc[j]);
        }
        __syncthreads();// stage s and sc[] free for reuse
    }
    if (!ok) {
        atomicExch(&s_attn_error, 1);
        return;
    }
    // ---- reduce the NTG token groups ----
#pragma unroll
    for (int j = 0; j < 8; ++j) red[tg * D + cg * 8 + j] = acc[j];
    __syncthreads();
    float out = 0.f;
    if (tid < D) {
#pragma unroll
        for (int g = 0; g < NTG; ++g) out += red[g * D + tid];
    }
    if (nsplit == 1) {
        if (tid < D) o[tid] = Num<T>::from_f(out / l_run);
        return;
    }
    const size_t rec = (static_cast<size_t>(b) * a.n_heads + h) * a.max_splits;
    float *mine = a.part + (rec + split) * (D + 2);
    if (tid < D) mine[2 + tid] = out;
    if (tid == 0) {
        mine[0] = m_run;
        mine[1] = l_run;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned old = atomicAdd(&a.cnt[static_cast<size_t>(b) * a.n_heads + h], 1u);
        s_last = (old == nsplit - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid < D) {
        // whole warps (D is 64 or 128): a lane reads one record header per round, so all headers cost one round trip to
        // L2; the accumulator loads of different splits are independent and unrolled
        const float *base = a.part + rec * (D + 2);
        float mx = -INFINITY;
        for (uint32_t s0 = 0; s0 < nsplit; s0 += 32)
            if (s0 + lane < nsplit) mx = fmaxf(mx, __ldcg(base + static_cast<size_t>(s0 + lane) * (D + 2)));
        mx = warp_max(mx);
        float num = 0.f, den = 0.f;
        for (uint32_t s0 = 0; s0 < nsplit; s0 += 32) {
            float2 ml = make_float2(-INFINITY, 0.f);
            if (s0 + lane < nsplit) ml = __ldcg(reinterpret_cast<const float2 *>(base + static_cast<size_t>(s0 + lane) * (D + 2)));
            const float w = ml.x == -INFINITY ? 0.f : expf(ml.x - mx);
            den += ml.y * w;
            const uint32_t cnt = nsplit - s0 < 32 ? nsplit - s0 : 32;
#pragma unroll 8
            for (uint32_t j = 0; j < cnt; ++j) num += __ldcg(base + static_cast<size_t>(s0 + j) * (D + 2) + 2 + tid) * __shfl_sync(0xffffffffu, w, j);
        }
        o[tid] = Num<T>::from_f(num / warp_sum(den));
    }
    if (tid == 0) a.cnt[static_cast<size_t>(b) * a.n_heads + h] = 0u;
}


// ---- flash-decoding, head_dim 128, 16-bit caches: warp-independent tiles, scores on the warp-level tensor path ------------
// 160 threads: warps 0-3 consume, lane 0 of warp 4 produces.  A 64-token K/V tile (32 KiB) is staged by cp.async.bulk (one copy
// per tile, or per 16-token page) into a ring of 2 stages (3 CTAs per SM) guarded by full/empty mbarriers.  Consumer warp w owns tokens
// [16w, 16w + 16) of every tile = the 16 rows of one mma.sync.m16n8k16 whose B operand is the query: row r reads its 32-byte
// k-chunks in the order s ^ (r % 8) with the 16-byte halves swapped for chunks >= 4 (no bank conflicts although rows lie 256
// bytes apart), column n of B holds the query permuted the same way, so C[r][r % 8] is the score of row r.  Every warp keeps its
// own online-softmax state (no CTA-wide barrier per tile); P.V runs on the FMA pipe, a lane owning 4 output dims.  The four
// warp states are merged through shared memory at the end; split records and the last-arriver merge are as in the general kernel.
constexpr int AM_THREADS = 160;
constexpr uint32_t AM_TILE_BYTES = AD_TILE * 128 * 2;// one of K, V

template<class T, int AM_STAGES>
__global__ void __launch_bounds__(AM_THREADS) attn_decode_mma_kernel(const DecodeArgs a) {
    constexpr int D = 128;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + AM_STAGES * 2 * AM_TILE_BYTES);
    uint64_t *empty = full + AM_STAGES;
    float *red = reinterpret_cast<float *>(empty + AM_STAGES);// [4 warps][D + 2]
    __shared__ int s_last, s_fail;

    const uint32_t split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t nkv = a.kv.n_kv_heads, kvh = h / (a.n_heads / nkv);
    if (tid == 0) {
        for (int s = 0; s < AM_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 4);
        }
        s_fail = 0;
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();

    const int64_t len64 = a.lens[b];
    const uint32_t len = kv_len_clamped(len64, a.max_len, a.kv, a.table != nullptr, &s_attn_index_error);
    const uint32_t ntiles = (len + AD_TILE - 1) / AD_TILE;
    const uint32_t nsplit = (ntiles + a.tiles_per_split - 1) / a.tiles_per_split;
    T *o = static_cast<T *>(a.o) + (static_cast<size_t>(b) * a.n_heads + h) * D;
    if (len == 0) {
        if (split == 0 && tid < D) o[tid] = Num<T>::from_f(0.f);
        return;
    }
    if (split >= nsplit) return;
    const uint32_t t0 = split * a.tiles_per_split;
    const uint32_t t1 = t0 + a.tiles_per_split < ntiles ? t0 + a.tiles_per_split : ntiles;

    if (warp == 4) {
        if (lane == 0) {
            const uint8_t *kc = static_cast<const uint8_t *>(a.kc), *vc = static_cast<const uint8_t *>(a.vc);
            for (uint32_t t = t0, it = 0; t < t1; ++t, ++it) {
                const uint32_t s = it % AM_STAGES, par = (it / AM_STAGES) & 1u;
                if (!mbar_wait(&empty[s], par ^ 1u)) {
                    atomicExch(&s_attn_error, 1);
                    break;
                }
                const uint32_t tok0 = t * AD_TILE, ntok = len - tok0 < AD_TILE ? len - tok0 : AD_TILE;
                uint8_t *ks = smem + s * 2 * AM_TILE_BYTES, *vs = ks + AM_TILE_BYTES;
                mbar_arrive_expect_tx(&full[s], 2u * ntok * D * 2u);
                if (!a.table) {
                    const size_t off = ((static_cast<size_t>(b) * nkv + kvh) * a.kv.max_seq + tok0) * D * 2;
                    bulk_g2s(ks, kc + off, ntok * D * 2u, &full[s]);
                    bulk_g2s(vs, vc + off, ntok * D * 2u, &full[s]);
                } else {
                    const uint32_t page = a.kv.page_size, step = page < AD_TILE ? page : AD_TILE;
                    for (uint32_t done = 0; done < ntok; done += step) {
                        const uint32_t tok = tok0 + done, n = ntok - done < step ? ntok - done : step;
                        int32_t blk = a.table[static_cast<size_t>(b) * a.kv.max_blocks_per_seq + tok / page];
                        if (!kv_block_ok(blk, a.kv)) s_attn_index_error = 1, blk = 0;
                        const size_t off = ((static_cast<size_t>(blk) * nkv + kvh) * page + tok % page) * D * 2;
                        bulk_g2s(ks + done * D * 2, kc + off, n * D * 2u, &full[s]);
                        bulk_g2s(vs + done * D * 2, vc + off, n * D * 2u, &full[s]);
                    }
                }
            }
        }
        return;
    }

    // ---- consumers ----
    const uint32_t gq = lane >> 2, kq = lane & 3u;
    const bool own = kq == (gq >> 1);// this lane's c[gq & 1] / c[2 + (gq & 1)] are the scores of rows gq / gq + 8
    uint32_t qb[8][2];
    {
        const T *qh = static_cast<const T *>(a.q) + (static_cast<size_t>(b) * a.n_heads + h) * D;
#pragma unroll
        for (int st = 0; st < 8; ++st) {
            const uint32_t ch = static_cast<uint32_t>(st) ^ gq, hs = (ch >> 2) & 1u;
            const T *qp = qh + (ch * 16 + 2 * kq);
            qb[st][0] = *reinterpret_cast<const uint32_t *>(qp + (hs ? 8 : 0));
            qb[st][1] = *reinterpret_cast<const uint32_t *>(qp + (hs ? 0 : 8));
        }
    }
    float m_w = -INFINITY, l_w = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    bool ok = true;
    for (uint32_t t = t0, it = 0; t < t1; ++t, ++it) {
        const uint32_t s = it % AM_STAGES;
        if (!mbar_wait(&full[s], (it / AM_STAGES) & 1u)) {
            ok = false;
            break;
        }
        const uint32_t tok0 = t * AD_TILE, ntok = len - tok0 < AD_TILE ? len - tok0 : AD_TILE;
        const uint8_t *ks = smem + s * 2 * AM_TILE_BYTES, *vs = ks + AM_TILE_BYTES;
        const uint32_t rA = warp * 16 + gq, rB = rA + 8;
        const bool vA = rA < ntok, vB = rB < ntok;
        float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int st = 0; st < 8; ++st) {
            const uint32_t ch = static_cast<uint32_t>(st) ^ gq, hs = (ch >> 2) & 1u;
            const uint32_t off = ch * 32 + kq * 4, o0 = off + (hs ? 16u : 0u), o1 = off + (hs ? 0u : 16u);
            uint32_t af[4];
            af[0] = vA ? *reinterpret_cast<const uint32_t *>(ks + rA * 256 + o0) : 0u;
            af[2] = vA ? *reinterpret_cast<const uint32_t *>(ks + rA * 256 + o1) : 0u;
            af[1] = vB ? *reinterpret_cast<const uint32_t *>(ks + rB * 256 + o0) : 0u;
            af[3] = vB ? *reinterpret_cast<const uint32_t *>(ks + rB * 256 + o1) : 0u;
            if (st & 1) mma16816<T>(c2, af, qb[st][0], qb[st][1]);
            else
                mma16816<T>(c, af, qb[st][0], qb[st][1]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) c[e] += c2[e];
        const float sa = (own && vA) ? ((gq & 1u) ? c[1] : c[0]) * a.scale : -INFINITY;
        const float sb = (own && vB) ? ((gq & 1u) ? c[3] : c[2]) * a.scale : -INFINITY;
        const float m_new = fmaxf(m_w, warp_max(fmaxf(sa, sb)));
        // a warp whose 16 rows all lie past the end of the sequence keeps m = -inf and adds nothing
        const float pa = (sa == -INFINITY) ? 0.f : __expf(sa - m_new);
        const float pb = (sb == -INFINITY) ? 0.f : __expf(sb - m_new);
        const float corr = (m_w == -INFINITY) ? 0.f : __expf(m_w - m_new);
        l_w = l_w * corr + warp_sum(pa + pb);
        m_w = m_new;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] *= corr;
        uint2 vraw[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t tok = warp * 16 + j;// rows 0..7 carry pa, rows 8..15 pb
            vraw[j] = make_uint2(0u, 0u);
            if (tok < ntok) vraw[j] = *reinterpret_cast<const uint2 *>(vs + tok * 256 + lane * 8);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float pt = __shfl_sync(0xffffffffu, j < 8 ? pa : pb, (j & 7) * 4 + (j & 7) / 2);
            const float2 lo = unpack2<T>(vraw[j].x), hi = unpack2<T>(vraw[j].y);
            acc[0] = fmaf(pt, lo.x, acc[0]);
            acc[1] = fmaf(pt, lo.y, acc[1]);
            acc[2] = fmaf(pt, hi.x, acc[2]);
            acc[3] = fmaf(pt, hi.y, acc[3]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    if (!ok) {
        atomicExch(&s_attn_error, 1);
        s_fail = 1;
    }
    // ---- merge the four warps ----
    float *wst = red + warp * (D + 2);
    if (lane == 0) wst[0] = m_w, wst[1] = l_w;
#pragma unroll
    for (int e = 0; e < 4; ++e) wst[2 + lane * 4 + e] = acc[e];
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (s_fail) return;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, red[w * (D + 2)]);
    float out = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const float mw = red[w * (D + 2)];
        const float f = mw == -INFINITY ? 0.f : __expf(mw - M);
        L += red[w * (D + 2) + 1] * f;
        out += red[w * (D + 2) + 2 + tid] * f;
    }
    if (nsplit == 1) {
        o[tid] = Num<T>::from_f(out / L);
        return;
    }
    const size_t rec = (static_cast<size_t>(b) * a.n_heads + h) * a.max_splits;
    float *mine = a.part + (rec + split) * (D + 2);
    mine[2 + tid] = out;
    if (tid == 0) {
        mine[0] = M;
        mine[1] = L;
    }
    __threadfence();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (tid == 0) {
        const unsigned old = atomicAdd(&a.cnt[static_cast<size_t>(b) * a.n_heads + h], 1u);
        s_last = (old == nsplit - 1) ? 1 : 0;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (!s_last) return;
    __threadfence();
    {
        const float *base = a.part + rec * (D + 2);
        float mx = -INFINITY;
        for (uint32_t s0 = 0; s0 < nsplit; s0 += 32)
            if (s0 + lane < nsplit) mx = fmaxf(mx, __ldcg(base + static_cast<size_t>(s0 + lane) * (D + 2)));
        mx = warp_max(mx);
        float num = 0.f, den = 0.f;
        for (uint32_t s0 = 0; s0 < nsplit; s0 += 32) {
            float2 ml = make_float2(-INFINITY, 0.f);
            if (s0 + lane < nsplit) ml = __ldcg(reinterpret_cast<const float2 *>(base + static_cast<size_t>(s0 + lane) * (D + 2)));
            const float w = ml.x == -INFINITY ? 0.f : expf(ml.x - mx);
            den += ml.y * w;
            const uint32_t cnt = nsplit - s0 < 32 ? nsplit - s0 : 32;
#pragma unroll 8
            for (uint32_t j = 0; j < cnt; ++j) num += __ldcg(base + static_cast<size_t>(s0 + j) * (D + 2) + 2 + tid) * __shfl_sync(0xffffffffu, w, j);
        }
        o[tid] = Num<T>::from_f(num / warp_sum(den));
    }
    if (tid == 0) a.cnt[static_cast<size_t>(b) * a.n_heads + h] = 0u;
}

struct DecodePlan {
    uint32_t tiles_per_split, max_splits;
    size_t part_bytes, cnt_bytes;
};
static DecodePlan decode_plan(const rg_attn_decode_params *p) {
    DecodePlan pl;
    const uint32_t total_tiles = (p->max_len + AD_TILE - 1) / AD_TILE;
    const uint64_t rows = static_cast<uint64_t>(p->batch) * p->n_heads;
    uint32_t want = static_cast<uint32_t>(4ull * sm_count() / (rows ? rows : 1));// rounded down: the CTAs of a launch fit the slots
    if (want < 1) want = 1;
    if (want > total_tiles) want = total_tiles ? total_tiles : 1;
    pl.tiles_per_split = total_tiles ? (total_tiles + want - 1) / want : 1;
    // Long sequences are cut into runs of at most 16 tiles even when there are enough (sequence, head) rows to fill the GPU:
    // with lengths between 512 and 4096 tokens, whole-sequence CTAs leave the last wave to the few longest sequences
    // (batch 32 x 32 heads, 16-token pages: 302 us unsplit, 274 / 263 / 265 / 286 us with runs of 32 / 16 / 8 / 4 tiles).
    if (pl.tiles_per_split > 16) pl.tiles_per_split = 16;
    pl.max_splits = total_tiles ? (total_tiles + pl.tiles_per_split - 1) / pl.tiles_per_split : 1;
    pl.cnt_bytes = (rows * 4 + 255) / 256 * 256;
    pl.part_bytes = rows * pl.max_splits * (p->kv.head_dim + 2) * 4;
    return pl;
}

template<class T, int D>
static int decode_launch(const rg_attn_decode_params *p, void *ws, const void *const *in, void *const *out,
                         cudaStream_t st, bool pdl) {
    const DecodePlan pl = decode_plan(p);
    DecodeArgs a = {};
    a.q = in[0], a.kc = in[1], a.vc = in[2];
    a.lens = static_cast<const int64_t *>(in[3]);
    a.table = static_cast<const int32_t *>(in[4]);
    a.o = out[0];
    a.cnt = static_cast<unsigned *>(ws);
    a.part = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + pl.cnt_bytes);
    a.batch = p->batch, a.n_heads = p->n_heads;
    a.tiles_per_split = pl.tiles_per_split, a.max_splits = pl.max_splits, a.max_len = p->max_len;
    a.kv = p->kv;
    a.scale = 1.0f / sqrtf(static_cast<float>(D));
    // The tensor-path kernel pays for its larger prologue only when there is enough work to stream (batch-1 launches of
    // ~1000 tiles measured 17.4 us against 15.5 us for the general kernel; batch 32 x 32 heads 203 us against 263 us).
    static const int mma_env = std::getenv("RG_B200_ATTN_MMA") ? atoi(std::getenv("RG_B200_ATTN_MMA")) : -1;
    const uint64_t work_tiles = static_cast<uint64_t>(p->batch) * p->n_heads * ((p->max_len + AD_TILE - 1) / AD_TILE);
    const int stages = mma_env >= 2 ? mma_env : 2;// batch-32 launch: 203 / 235 / 385 us with 2 / 3 / 4 stages (3 / 2 / 1 CTAs per SM)
    const bool mma = D == 128 && sizeof(T) == 2 && mma_env != 0 && (mma_env > 0 || work_tiles >= 8192);
    const size_t smem = mma ? stages * 2 * AM_TILE_BYTES + 2 * stages * 8 + 4 * (128 + 2) * 4
                            : 4 * AD_TILE * D * 2 + 16 + (D + AD_TILE + (AD_THREADS / (D / 8)) * D) * 4;
    void (*kern)(const DecodeArgs) = attn_decode_kernel<T, D>;
    if constexpr (D == 128 && sizeof(T) == 2) {
        if (mma) kern = stages == 2 ? attn_decode_mma_kernel<T, 2> : stages == 4 ? attn_decode_mma_kernel<T, 4> : attn_decode_mma_kernel<T, 3>;
    }
    RG_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.max_splits, p->n_heads, p->batch);
    cfg.blockDim = dim3(mma ? AM_THREADS : AD_THREADS);
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

// ---- reference-layout kernels -----------------------------------------------------------------------
// cache[n, h, past + s, :] = x[n, h, s, :]
template<class T>
__global__ void kv_append_kernel(const T *__restrict__ k, const T *__restrict__ v, T *__restrict__ kc,
                                 T *__restrict__ vc, const int64_t *__restrict__ past_p, uint32_t nh, uint32_t S,
                                 uint32_t D, uint32_t max_seq, uint64_t total) {
    const uint32_t past = past_clamped(past_p, max_seq);
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
         t += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t d = static_cast<uint32_t>(t % D);
        const uint64_t r = t / D;
        const uint32_t s = static_cast<uint32_t>(r % S);
        const uint64_t nhh = r / S;// n*nh + h
        if (past + s >= max_seq) continue;
        const uint64_t dst = (nhh * max_seq + past + s) * D + d;
        kc[dst] = k[t];
        vc[dst] = v[t];
    }
}
// copy the live prefix [0, past) of a cache into another buffer (out-of-place cache outputs)
template<class T>
__global__ void kv_prefix_copy_kernel(const T *__restrict__ src, T *__restrict__ dst,
                                      const int64_t *__restrict__ past_p, uint32_t D, uint32_t max_seq,
                                      uint64_t heads) {
    const uint32_t past = past_clamped(past_p, max_seq);
    const uint64_t per = static_cast<uint64_t>(past) * D, total = heads * per;
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
         t += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint64_t hh = t / per, r = t % per;
        dst[hh * max_seq * D + r] = src[hh * max_seq * D + r];
    }
}

// One warp per query row; lane owns EP = D/32 consecutive dims.  K/V rows are [.., kv_stride_tokens, D].
template<class T, int EP>
__global__ void __launch_bounds__(128) attn_rows_kernel(const T *__restrict__ q, const T *__restrict__ K,
                                                        const T *__restrict__ V, T *__restrict__ o,
                                                        const int64_t *__restrict__ past_p, uint32_t batch,
                                                        uint32_t n_heads, uint32_t n_kv, uint32_t S,
                                                        uint32_t kv_tokens /* tokens per (n, kv head) in K/V */,
                                                        float scale) {
    constexpr int D = EP * 32;
    const uint32_t past = past_clamped(past_p, kv_tokens);
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);// (n, h, i)
    if (row >= static_cast<uint64_t>(batch) * n_heads * S) return;
    const uint32_t i = static_cast<uint32_t>(row % S);
    const uint32_t h = static_cast<uint32_t>((row / S) % n_heads);
    const uint32_t n = static_cast<uint32_t>(row / S / n_heads);
    const uint32_t kvh = h / (n_heads / n_kv);
    const T *Kb = K + (static_cast<size_t>(n) * n_kv + kvh) * kv_tokens * D;
    const T *Vb = V + (static_cast<size_t>(n) * n_kv + kvh) * kv_tokens * D;
    float qv[EP], acc[EP];
#pragma unroll
    for (int e = 0; e < EP; ++e) {
        qv[e] = Num<T>::to_f(q[row * D + lane * EP + e]) * scale;
        acc[e] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const uint32_t last = past + i;// keys 0..last inclusive
    for (uint32_t j = 0; j <= last && j < kv_tokens; ++j) {
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < EP; ++e) dot += qv[e] * Num<T>::to_f(Kb[static_cast<size_t>(j) * D + lane * EP + e]);
        dot = warp_sum(dot);
        const float mn = fmaxf(m, dot);
        const float corr = m == -INFINITY ? 0.f : expf(m - mn);
        const float p = expf(dot - mn);
        l = l * corr + p;
#pragma unroll
        for (int e = 0; e < EP; ++e)
            acc[e] = acc[e] * corr + p * Num<T>::to_f(Vb[static_cast<size_t>(j) * D + lane * EP + e]);
        m = mn;
    }
#pragma unroll
    for (int e = 0; e < EP; ++e) o[row * D + lane * EP + e] = Num<T>::from_f(acc[e] / l);
}

// grouped-query variant (attn_decode_gqa.cu): one CTA serves all query heads of a KV head
bool attn_decode_gqa_applies(const rg_attn_decode_params *p);
size_t attn_decode_gqa_workspace(const rg_attn_decode_params *p);
size_t attn_decode_gqa_counter_bytes(const rg_attn_decode_params *p);
int attn_decode_gqa_launch(const rg_attn_decode_params *p, void *ws, const void *const *in, void *const *out, cudaStream_t st, bool pdl);

int attn_prefill_ref_layout(int dtype, const void *q, const void *K, const void *V, void *o, const int64_t *past, uint32_t batch,
                            uint32_t n_heads, uint32_t n_kv, uint32_t S, uint32_t kv_tokens, cudaStream_t st);

template<class T>
static int attention_launch(const rg_attention_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    auto q = static_cast<const T *>(in[0]);
    auto k = static_cast<const T *>(in[1]);
    auto v = static_cast<const T *>(in[2]);
    auto past = static_cast<const int64_t *>(in[3]);
    auto o = static_cast<T *>(out[0]);
    const T *K = k, *V = v;
    uint32_t kv_tokens = p->seq_len;
    const unsigned cap = static_cast<unsigned>(sm_count()) * 8;
    if (p->has_cache) {
        auto kci = static_cast<const T *>(in[4]);
        auto vci = static_cast<const T *>(in[5]);
        auto kco = static_cast<T *>(out[1]);
        auto vco = static_cast<T *>(out[2]);
        if (!kco || !vco) return RG_ERR_NULL;
        const uint64_t heads = static_cast<uint64_t>(p->batch) * p->n_kv_heads;
        if (kci && kci != kco) {
            kv_prefix_copy_kernel<T><<<cap, 256, 0, st>>>(kci, kco, past, p->head_dim, p->max_seq, heads);
            kv_prefix_copy_kernel<T><<<cap, 256, 0, st>>>(vci, vco, past, p->head_dim, p->max_seq, heads);
            count_launch(2);
        }
        const uint64_t total = heads * p->seq_len * p->head_dim;
        if (total) {
            const uint64_t want = (total + 255) / 256;
            kv_append_kernel<T><<<static_cast<unsigned>(want > cap ? cap : want), 256, 0, st>>>(
                k, v, kco, vco, past, p->n_kv_heads, p->seq_len, p->head_dim, p->max_seq, total);
            count_launch();
        }
        K = kco, V = vco, kv_tokens = p->max_seq;
    }
    const uint64_t rows = static_cast<uint64_t>(p->batch) * p->n_heads * p->seq_len;
    if (rows == 0) return RG_OK;
    // tensor-core flash kernel for 16-bit types at head_dim 128 once there is a tile's worth of query rows
    if (sizeof(T) == 2 && p->head_dim == 128 && p->seq_len >= 16 && aligned16(q) && aligned16(K) && aligned16(V) && aligned16(o))
        return attn_prefill_ref_layout(p->dtype, q, K, V, o, past, p->batch, p->n_heads, p->n_kv_heads, p->seq_len, kv_tokens, st);
    const unsigned grid = static_cast<unsigned>((rows + 3) / 4);
    const float scale = 1.0f / sqrtf(static_cast<float>(p->head_dim));
#define RG_ATT(EP) attn_rows_kernel<T, EP><<<grid, 128, 0, st>>>(q, K, V, o, past, p->batch, p->n_heads, p->n_kv_heads, p->seq_len, kv_tokens, scale)
    switch (p->head_dim) {
        case 32: RG_ATT(1); break;
        case 64: RG_ATT(2); break;
        case 128: RG_ATT(4); break;
        case 256: RG_ATT(8); break;
        default: return RG_ERR_SHAPE;
    }
#undef RG_ATT
    count_launch();
    return launch_status();
}

int attn_error_word(bool clear) { return error_symbol(s_attn_error, clear); }
int attn_index_error_word(bool clear) { return error_symbol(s_attn_index_error, clear); }

}// namespace rg

using namespace rg;

static bool attn_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = std::getenv("RG_B200_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

extern "C" {

size_t rg_b200_attention_workspace(const rg_attention_params *) { return 0; }
int rg_b200_attention(const rg_attention_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !in[1] || !in[2] || !out[0]) return RG_ERR_NULL;
    if (p->n_kv_heads == 0 || p->n_heads % p->n_kv_heads != 0) return RG_ERR_SHAPE;
    if (p->has_cache && p->max_seq < p->seq_len) return RG_ERR_SHAPE;
    auto st = static_cast<cudaStream_t>(stream);
    switch (p->dtype) {
        case RG_F32: return attention_launch<float>(p, in, out, st);
        case RG_FP16: return attention_launch<__half>(p, in, out, st);
        case RG_BF16: return attention_launch<__nv_bfloat16>(p, in, out, st);
        default: return RG_ERR_DTYPE;
    }
}

size_t rg_b200_attn_decode_workspace(const rg_attn_decode_params *p) {
    if (!p) return 0;
    const DecodePlan pl = decode_plan(p);
    size_t bytes = pl.cnt_bytes + pl.part_bytes;
    if (attn_decode_gqa_applies(p)) {
        const size_t g = attn_decode_gqa_workspace(p);
        bytes = g > bytes ? g : bytes;
    }
    return bytes;
}
int rg_b200_attn_decode(const rg_attn_decode_params *p, void *ws, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !in[1] || !in[2] || !in[3] || !out[0] || !ws) return RG_ERR_NULL;
    if (p->kv.n_kv_heads == 0 || p->n_heads % p->kv.n_kv_heads != 0 || p->max_len == 0) return RG_ERR_SHAPE;
    if (p->batch == 0) return RG_OK;
    if (p->batch > 65535 || p->n_heads > 65535) return RG_ERR_SHAPE;
    if (in[4]) {
        const uint32_t pg = p->kv.page_size;
        if (pg == 0 || !((pg < AD_TILE && AD_TILE % pg == 0) || pg % AD_TILE == 0)) return RG_ERR_SHAPE;
    } else if (p->kv.max_seq < p->max_len) {
        return RG_ERR_SHAPE;
    }
    if (!aligned16(in[1]) || !aligned16(in[2])) return RG_ERR_ALIGN;
    auto st = static_cast<cudaStream_t>(stream);
    const bool pdl = attn_pdl_enabled();
    if (attn_decode_gqa_applies(p)) return attn_decode_gqa_launch(p, ws, in, out, st, pdl);
    if (p->dtype == RG_FP16) {
        if (p->kv.head_dim == 128) return decode_launch<__half, 128>(p, ws, in, out, st, pdl);
        if (p->kv.head_dim == 64) return decode_launch<__half, 64>(p, ws, in, out, st, pdl);
        return RG_ERR_SHAPE;
    }
    if (p->dtype == RG_BF16) {
        if (p->kv.head_dim == 128) return decode_launch<__nv_bfloat16, 128>(p, ws, in, out, st, pdl);
        if (p->kv.head_dim == 64) return decode_launch<__nv_bfloat16, 64>(p, ws, in, out, st, pdl);
        return RG_ERR_SHAPE;
    }
    return RG_ERR_DTYPE;
}

// ---- allocation-free variant ---------------------------------------------------------------------------------
// Scratch for rg_b200_attn_decode_static: arrival counters followed by the per-split partial records, held in
// device memory that belongs to this library image instead of to the caller.  Every GPU that loads the library
// carries these 8 MiB until the process exits.
#define RG_DECODE_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char s_decode_scratch[RG_DECODE_STATIC_SCRATCH_BYTES];

size_t rg_b200_attn_decode_static_capacity(void) { return RG_DECODE_STATIC_SCRATCH_BYTES; }

int rg_b200_attn_decode_static(const rg_attn_decode_params *p, const void *const *in, void *const *out, void *stream) {
    // Validation first: nothing is written to the shared array for a request that cannot run.
    if (!p || !in || !out || !in[0] || !in[1] || !in[2] || !in[3] || !out[0]) return RG_ERR_NULL;
    if (p->kv.n_kv_heads == 0 || p->n_heads % p->kv.n_kv_heads != 0 || p->max_len == 0) return RG_ERR_SHAPE;
    if (p->batch == 0) return RG_OK;
    if (p->batch > 65535 || p->n_heads > 65535) return RG_ERR_SHAPE;
    // The limit is the size the workspace entry point asks for: the larger of the general and the grouped-query
    // kernel's layouts, whichever of the two the dispatch below picks.
    const size_t need = rg_b200_attn_decode_workspace(p);
    if (need > RG_DECODE_STATIC_SCRATCH_BYTES) return RG_ERR_LIMIT;
    // In host code `s_decode_scratch` names a host-side shadow of the symbol, not device memory, so the device
    // address is looked up once per device (with that device current) and remembered.
    static void *scratch_of_device[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return RG_ERR_CUDA;
    if (!scratch_of_device[dev]) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, s_decode_scratch) != cudaSuccess || !ptr) return RG_ERR_CUDA;
        scratch_of_device[dev] = ptr;
    }
    void *ws = scratch_of_device[dev];
    auto st = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left, and the previous call may have used the other kernel's layout:
    // clear the arrival counters of both (each sits at the start of the array).
    const DecodePlan pl = decode_plan(p);
    size_t cnt = pl.cnt_bytes;
    if (attn_decode_gqa_applies(p)) {
        const size_t g = attn_decode_gqa_counter_bytes(p);
        cnt = g > cnt ? g : cnt;
    }
    if (cnt > need) cnt = need;
    if (cudaMemsetAsync(ws, 0, cnt, st) != cudaSuccess) return RG_ERR_CUDA;
    return rg_b200_attn_decode(p, ws, in, out, stream);
}
}
