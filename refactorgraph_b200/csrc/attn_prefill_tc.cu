// Causal flash attention for prefill on the fifth-generation tensor cores (head_dim 128, fp16 / bf16).
// Two kernels: attn_prefill_q2_kernel (further down; two query tiles per CTA, the default) and attn_prefill_tc_kernel (one query tile
// per CTA, RG_B200_ATTN_Q2=0), described first because the second builds on what was measured on it.
// Semantics: src/08-01llm/README.md:29-63 (causal multi-head self-attention, query head h uses KV head h / (heads / kv_heads),
// scores scaled by 1/sqrt(head_dim), softmax and accumulation in fp32).
//
// One CTA = 128 query rows of one (sequence, head) and walks the 128-key tiles at or below its causal diagonal:
//   warp 4 (one thread)  TMA producer: Q once, then K and V tiles (two d-halves of [128 rows x 64 columns], 128-byte swizzle)
//                        into double-buffered shared-memory stages, completion on mbarriers;
//   warp 5 (one thread)  issues tcgen05.mma: S = Q K^T (both operands K-major, 8 instructions of M128 N128 K16) into one of two
//                        128-column accumulators in tensor memory, and O_tile = P V (A = P from shared memory, K-major; B = V as
//                        it lies in the cache, i.e. MN-major, 8 instructions) into a third; S of the NEXT tile is issued
//                        before the wait for P, so it runs while the softmax warps work;
//   warps 0-7            two threads per query row (warps w and w + 4 share tensor-memory lane quarter w, one takes key / d columns
//                        0-63, the other 64-127): tcgen05.ld of the scores, online softmax in fp32 with ex2.approx, P written to
//                        shared memory in the swizzled K-major layout the second product reads, O_tile read back with tcgen05.ld
//                        and added to the thread's 64 fp32 accumulators.  The two threads of a row swap their half-row maxima
//                        through shared memory once per tile.  The running maximum is only moved (and the accumulators rescaled)
//                        when a row's maximum grows by more than 2^8 in the exponent's units — probabilities then stay below 256,
//                        exact in fp32 and far inside the 16-bit range — so most tiles skip the rescaling altogether.
// Keeping O in registers instead of in tensor memory avoids a read-modify-write of the accumulator whenever the maximum
// changes; the price is one tcgen05.ld of the tile per key tile.
// Measured on [4, 32, 2048, 128] bf16: 208.4 us = 660 TFLOP/s (the warp-level mma.sync kernel: 565 us = 243 TFLOP/s).  The steps:
// one row per thread (four softmax warps) 306 TFLOP/s on one sequence, two threads per row 392 (499 on four sequences); P and
// O_tile double-buffered, so that tile j's second product runs under tile j + 1's exponentials (the accumulators take O_tile
// two tiles late, times whatever rescaling happened in between): 523; persistent CTAs, one per SM, that fetch the next item's
// Q / K / V under the current item's tail and set tensor memory and barriers up once: 563; items dealt back and forth over the
// CTAs instead of round-robin (the heaviest CTA carries 119 key tiles instead of 125, the mean is 117.6): 579; the output staged
// through shared memory and written two whole rows per instruction instead of 32 half rows: 660.  Keeping a
// thread's 64 scores in registers between the maximum pass and the exponential pass (one tcgen05.ld round instead of two) spills
// at the 168 registers a 320-thread CTA gets and measured 532.  A head-major item order (all query tiles of a head in flight
// together, so that K / V come from L2: ncu shows 3.2 x the algorithmic bytes in DRAM traffic, 41 % of DRAM peak) measured 568:
// the loads are not what the kernel waits for.  Cycle counters in a softmax warp, per key tile, before the
// double buffering: ~1480 in the exponential pass (the special-function unit's 16 results per clock bound it at 1024), ~330
// reading the scores for the maximum, ~200 in the pair exchange, ~190 adding O_tile, ~800 waiting for the tensor core.
// Taking a quarter or half of the exponentials from a cubic on the FMA pipe instead of the special-function unit measured 556
// and 539 (against 574 the same day): the pass is not bound by that unit alone.  Packed fp32 instructions (fma / add .f32x2) and
// the three-input maximum in the softmax warps, a sixth fewer instructions: 647 against 646; the causal mask compiled out of the
// tiles that need none: no change (the compiler had done it); both halves of a tile requested from tensor memory before one wait in
// the maximum pass: 618 against 650.  What the counters show (ncu, two sequences): issue slots 51 % busy, the special-function
// pipe 33 % over the kernel but ~75 % inside the exponential pass, where all eight softmax warps arrive together because one
// barrier releases each tile's scores; spreading that pass out in time needs two query tiles per CTA on alternating phases, with
// O kept in tensor memory to make room in the register file.
// Every wait is bounded; on expiry the kernel records an error word, releases its tensor memory and leaves.
#include "tcgen05.cuh"
#include <cstdlib>

namespace rg {

constexpr int AT_BM = 128, AT_BN = 128, AT_D = 128, AT_SW = 8, AT_THREADS = (AT_SW + 2) * 32;
constexpr uint32_t AT_TILE_BYTES = 128 * 128 * 2;// one [128 x 128] 16-bit tile = two [128 x 64] swizzled halves

static __device__ int s_attn_tc_error;

struct AttnTcArgs {
    void *o;
    int64_t o_sn, o_sh, o_st;
    uint32_t n_heads, n_kv, S, kv_len;
    float scale_log2e;
    int is_bf16;
    uint32_t v_lbo, v_sbo;// descriptor offsets of the MN-major V operand (bytes)
    uint32_t q_tiles, batch;
};

// Work item i of the launch: query tile qt of (sequence n, head h), heaviest tiles (far from the start of the sequence) first.
// CTA c takes one item of every band of G consecutive items, walking the bands back and forth (item c of even bands, G - 1 - c of
// odd ones), so that the weights it collects add up to within ~1 % of every other CTA's.
__device__ __forceinline__ uint32_t at_item_of(uint32_t band, uint32_t n_items) {// >= n_items: this CTA has none in this band
    return band * gridDim.x + ((band & 1u) ? gridDim.x - 1 - blockIdx.x : blockIdx.x);
}
struct AtItem {
    uint32_t q0, h, n, kvh, ntiles;
};
__device__ __forceinline__ AtItem at_item(const AttnTcArgs &a, uint32_t i) {
    const uint32_t hn = a.n_heads * a.batch, qt = a.q_tiles - 1 - i / hn, r = i % hn;
    AtItem it;
    it.q0 = qt * AT_BM, it.h = r % a.n_heads, it.n = r / a.n_heads;
    it.kvh = it.h / (a.n_heads / a.n_kv);
    // keys any row of this tile may see: [0, q0 + 128) cut at kv_len
    const uint32_t last_key = it.q0 + AT_BM < a.kv_len ? it.q0 + AT_BM : a.kv_len;
    it.ntiles = (last_key + AT_BN - 1) / AT_BN;
    return it;
}

__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t z, uint32_t w, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar))
        : "memory");
}
// Shared-memory descriptor with explicit leading / stride byte offsets, 128-byte swizzle (see smem_desc_sw128 for the fields)
__device__ __forceinline__ uint64_t smem_desc_sw128_ex(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// A bounded wait whose outcome is the same for every lane of the warp (the .sync.aligned tensor-memory instructions behind
// it must be executed by the whole warp or by none of it)
__device__ __forceinline__ bool at_warp_wait(uint64_t *bar, uint32_t parity) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity) ? 1 : 0) != 0;
}
// Barrier of the 64 threads that share named barrier `id` which also ORs a predicate over them: both warps of a lane quarter
// get the same answer, so they take the same way out when a wait has failed (a plain flag read could differ between them and
// leave one warp at a barrier the other never reaches).
__device__ __forceinline__ bool at_pair_sync_or(uint32_t id, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.u32 q, %2, 0;\n"
        "bar.red.or.pred p, %1, 64, q;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(r)
        : "r"(id), "r"(pred ? 1u : 0u)
        : "memory");
    return r != 0;
}
template<class T> __device__ __forceinline__ uint32_t at_pack2(float lo, float hi);
template<> __device__ __forceinline__ uint32_t at_pack2<__half>(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}
template<> __device__ __forceinline__ uint32_t at_pack2<__nv_bfloat16>(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

template<class T>
__global__ void __launch_bounds__(AT_THREADS, 1) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                                                        const __grid_constant__ CUtensorMap map_v, const AttnTcArgs a) {
    // Seven 32 KiB tiles leave no room for alignment slack below the 227 KiB a CTA may have: the swizzled tiles need the dynamic
    // shared memory to start on a 1 KiB boundary, which is checked below (it does when the kernel has no static shared memory).
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sQ = smem;                          // 32 KiB
    uint8_t *sK = sQ + AT_TILE_BYTES;            // 2 x 32 KiB
    uint8_t *sV = sK + 2 * AT_TILE_BYTES;        // 2 x 32 KiB
    uint8_t *sP = sV + 2 * AT_TILE_BYTES;        // 2 x 32 KiB
    uint64_t *bars = reinterpret_cast<uint64_t *>(sP + 2 * AT_TILE_BYTES);
    uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = bars + 3, *v_full = bars + 5, *v_empty = bars + 7;
    uint64_t *s_full = bars + 9, *s_empty = bars + 11, *p_full = bars + 13, *o_full = bars + 15, *o_empty = bars + 17, *q_empty = bars + 19;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 20);
    volatile int *failed = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *xch = reinterpret_cast<float *>(bars + 21);// [2 tiles in flight][2 halves][128 rows]: half-row maxima, then the row sums
    if (smem_u32(smem) & 1023u) {// uniform over the CTA; nothing has been set up yet
        if (threadIdx.x == 0) atomicExch(&s_attn_tc_error, 5);
        return;
    }

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n_items = a.q_tiles * a.n_heads * a.batch;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1), mbar_init(q_empty, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1), mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1), mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1), mbar_init(&s_empty[s], AT_SW);
            mbar_init(&p_full[s], AT_SW), mbar_init(&o_full[s], 1), mbar_init(&o_empty[s], AT_SW);
        }
        *failed = 0;
        fence_mbar_init();
    }
    if (warp == AT_SW + 1) {
        tmem_alloc(tmem_slot, 512);// S x 2, O_tile x 2
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();// q, k and v come from the previous kernels of the stream

    if (warp == AT_SW) {
        if (lane == 0) {
            // t counts key tiles over all items of this CTA: stage t & 1, phase (t >> 1) & 1, whatever the item
            uint32_t t = 0, done = 0;
            for (uint32_t band = 0; band * gridDim.x < n_items && !*failed; ++band) {
                const uint32_t i = at_item_of(band, n_items);
                if (i >= n_items) continue;
                const AtItem w = at_item(a, i);
                // Q is single-buffered: the previous item's last S product must have read it
                if (done && !mbar_wait(q_empty, (done - 1) & 1u)) {
                    *failed = 1;
                    break;
                }
                mbar_arrive_expect_tx(q_full, AT_TILE_BYTES);
                tma_load_4d(sQ, &map_q, 0, w.q0, w.h, w.n, q_full);
                tma_load_4d(sQ + AT_TILE_BYTES / 2, &map_q, 64, w.q0, w.h, w.n, q_full);
                for (uint32_t j = 0; j < w.ntiles; ++j, ++t) {
                    const uint32_t s = t & 1u, ph = (t >> 1) & 1u;
                    if (!mbar_wait(&k_empty[s], ph ^ 1u)) {
                        *failed = 1;
                        break;
                    }
                    mbar_arrive_expect_tx(&k_full[s], AT_TILE_BYTES);
                    tma_load_4d(sK + s * AT_TILE_BYTES, &map_k, 0, j * AT_BN, w.kvh, w.n, &k_full[s]);
                    tma_load_4d(sK + s * AT_TILE_BYTES + AT_TILE_BYTES / 2, &map_k, 64, j * AT_BN, w.kvh, w.n, &k_full[s]);
                    if (!mbar_wait(&v_empty[s], ph ^ 1u)) {
                        *failed = 1;
                        break;
                    }
                    mbar_arrive_expect_tx(&v_full[s], AT_TILE_BYTES);
                    tma_load_4d(sV + s * AT_TILE_BYTES, &map_v, 0, j * AT_BN, w.kvh, w.n, &v_full[s]);
                    tma_load_4d(sV + s * AT_TILE_BYTES + AT_TILE_BYTES / 2, &map_v, 64, j * AT_BN, w.kvh, w.n, &v_full[s]);
                }
                ++done;
            }
        }
    } else if (warp == AT_SW + 1) {
        if (lane == 0) {
            const uint32_t idesc_s = instr_desc(a.is_bf16, AT_BM, AT_BN);
            const uint32_t idesc_o = instr_desc(a.is_bf16, AT_BM, AT_D) | (1u << 16);// B (= V) is MN-major
            const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
            bool ok = true;
            // S of key tile t (counted over all items of this CTA) = Q K^T into accumulator t & 1
            auto issue_s = [&](uint32_t t) {
                const uint32_t s = t & 1u, ph = (t >> 1) & 1u;
                if (!mbar_wait(&k_full[s], ph) || !mbar_wait(&s_empty[s], ph ^ 1u)) return false;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sK + s * AT_TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t off = (kk >> 2) * (AT_TILE_BYTES / 2) + (kk & 3) * 32;
                    tc_mma_f16(tmem_base + s * AT_BN, smem_desc_sw128(q_addr + off), smem_desc_sw128(k_addr + off), idesc_s, kk ? 1u : 0u);
                }
                tc_commit(&k_empty[s]);
                tc_commit(&s_full[s]);
                return true;
            };
            uint32_t t = 0, done = 0;
            for (uint32_t band = 0; ok && band * gridDim.x < n_items; ++band) {
              const uint32_t i = at_item_of(band, n_items);
              if (i >= n_items) continue;
              const uint32_t ntiles = at_item(a, i).ntiles;
              ok = mbar_wait(q_full, done & 1u);
              if (ok) ok = issue_s(t);
              if (ok && ntiles == 1) tc_commit(q_empty);
              for (uint32_t j = 0; ok && j < ntiles; ++j, ++t) {
                if (j + 1 < ntiles) {
                    ok = issue_s(t + 1);
                    if (ok && j + 2 == ntiles) tc_commit(q_empty);// the item's last S: Q may be replaced once it has run
                }
                if (!ok) break;
                const uint32_t s = t & 1u, ph = (t >> 1) & 1u;
                // O_tile[j & 1] = P_j V_j once P_j is in shared memory, V_j has landed and O_tile of tile j - 2 has been read
                if (!mbar_wait(&p_full[s], ph) || !mbar_wait(&v_full[s], ph) || !mbar_wait(&o_empty[s], ph ^ 1u)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(sV + s * AT_TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    // A = P: keys 16 kk .. 16 kk + 15 of the row -> half kk / 4, 32 bytes per step inside the swizzle atom
                    const uint64_t ad = smem_desc_sw128(p_addr + s * AT_TILE_BYTES + (kk >> 2) * (AT_TILE_BYTES / 2) + (kk & 3) * 32);
                    // B = V: 16 keys = 16 lines of 128 bytes further down the [key][64 d] half
                    const uint64_t bd = smem_desc_sw128_ex(v_addr + kk * 2048, a.v_lbo, a.v_sbo);
                    tc_mma_f16(tmem_base + (2 + s) * AT_BN, ad, bd, idesc_o, kk ? 1u : 0u);
                }
                tc_commit(&v_empty[s]);
                tc_commit(&o_full[s]);
              }
              ++done;
            }
            if (!ok) *failed = 2;
        }
    } else {
        // ---- softmax / output warps: lane quarter = warp % 4, column half = warp / 4 ----
        const uint32_t quarter = warp & 3u, half = warp >> 2, row = quarter * 32 + lane;
        const uint32_t lane_addr = (quarter * 32u) << 16, col0 = half * 64u;
        const float c = a.scale_log2e, thr = 8.0f / c;
        float m_used, l_run;
        float acc[64];
        bool ok = true;
        uint32_t t = 0;// key tiles over all items of this CTA: buffers and barrier phases follow it
        // acc += f * (this thread's 64 columns of O_tile buffer b); f carries a rescaling that happened after the tile's
        // probabilities were computed and before the tile is added
        auto add_o_tile = [&](uint32_t b, float f) {
            tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + (2 + b) * AT_BN + lane_addr + col0 + c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) acc[c0 + e] = fmaf(__uint_as_float(r[e]), f, acc[c0 + e]);
            }
            tc_fence_before();
        };
        float pend = 1.f;// factor applied to the accumulators at the previous tile: the product still in flight needs it too
        for (uint32_t band = 0; band * gridDim.x < n_items; ++band) {
        const uint32_t item = at_item_of(band, n_items);
        if (item >= n_items) continue;
        const AtItem w = at_item(a, item);
        const uint32_t ntiles = w.ntiles, q0 = w.q0, qrow = q0 + row;
        m_used = -INFINITY, l_run = 0.f, pend = 1.f;
#pragma unroll
        for (int d = 0; d < 64; ++d) acc[d] = 0.f;
        // A wait that runs out is recorded in `failed`; the two warps of a lane quarter leave the loop together, right after
        // the barrier they share, so neither is left waiting for the other.
        for (uint32_t j = 0; j < ntiles; ++j, ++t) {
            const uint32_t s = t & 1u, ph = (t >> 1) & 1u;
            if (ok && !at_warp_wait(&s_full[s], ph)) ok = false, *failed = 3;
            tc_fence_after();
            const uint32_t s_addr = tmem_base + s * AT_BN + lane_addr + col0, key0 = j * AT_BN + col0;
            // first key this row may NOT see; only the tiles on the diagonal or at the end of the sequence need the mask
            const uint32_t lim = qrow + 1 < a.kv_len ? qrow + 1 : a.kv_len;
            const uint32_t warp_lim = q0 + quarter * 32 + 1 < a.kv_len ? q0 + quarter * 32 + 1 : a.kv_len;// smallest lim in the warp
            const bool masked = key0 + 64 > warp_lim;// warp-uniform
            // pass 1: maximum of this thread's 64 scores, then of the whole row
            float mx = -INFINITY;
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32(s_addr + c0, r);
                tmem_ld_wait();
                if (masked) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) mx = fmaxf(mx, key0 + c0 + e < lim ? __uint_as_float(r[e]) : -INFINITY);
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(r[e]));
                }
            }
            float *xr = xch + s * 256;
            xr[half * 128 + row] = mx;
            if (at_pair_sync_or(1u + quarter, *failed != 0)) break;// the two warps of this lane quarter, leaving together
            mx = fmaxf(mx, xr[(half ^ 1u) * 128 + row]);
            // the product of tile j - 2 (the one before last: tile j - 1's may still be running): its P buffer is free again,
            // its O_tile ready
            if (j > 1) {
                if (!at_warp_wait(&o_full[s], ((t - 2) >> 1) & 1u)) {
                    ok = false, *failed = 3;
                    continue;// the partner learns of it at the next shared barrier (or at the one behind the loop)
                }
                add_o_tile(s, pend);
                __syncwarp();
                if (lane == 0) mbar_arrive(&o_empty[s]);
            }
            // move the reference maximum only when some row of the warp needs it (both warps of a row see the same maxima)
            pend = 1.f;
            if (__any_sync(0xffffffffu, mx > m_used + thr)) {
                const float m_new = fmaxf(m_used, mx);
                const float alpha = (m_used == -INFINITY) ? 0.f : exp2f((m_used - m_new) * c);
#pragma unroll
                for (int d = 0; d < 64; ++d) acc[d] *= alpha;
                l_run *= alpha;
                m_used = m_new;
                pend = alpha;
            }
            // pass 2: p = 2^((s - m) * scale), written as 16-bit into this thread's 128-byte line of P half `half`
            const float mneg = (m_used == -INFINITY) ? 0.f : -m_used * c;
            float lsum = 0.f;
            uint8_t *line = sP + s * AT_TILE_BYTES + half * (AT_TILE_BYTES / 2) + row * 128u;
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32(s_addr + c0, r);
                tmem_ld_wait();
                uint32_t packed[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float p0, p1;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(fmaf(__uint_as_float(r[e]), c, mneg)));
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(fmaf(__uint_as_float(r[e + 1]), c, mneg)));
                    if (masked) {
                        if (key0 + c0 + e >= lim) p0 = 0.f;
                        if (key0 + c0 + e + 1 >= lim) p1 = 0.f;
                    }
                    lsum += p0 + p1;
                    packed[e / 2] = at_pack2<T>(p0, p1);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t chunk = (c0 >> 3) + q;
                    *reinterpret_cast<uint4 *>(line + ((chunk ^ (row & 7u)) << 4)) =
                        make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
            }
            l_run += lsum;
            tc_fence_before();
            fence_proxy_async();// the tensor core reads P through the async proxy
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&s_empty[s]);
                mbar_arrive(&p_full[s]);
            }
        }
        if (*failed) ok = false;
        // the item's last two products (t is now one past its last tile); the buffers go back to the tensor-core thread
        if (ok && ntiles > 1) {
            const uint32_t u = t - 2;
            if (!at_warp_wait(&o_full[u & 1u], (u >> 1) & 1u)) ok = false, *failed = 3;
            if (ok) {
                add_o_tile(u & 1u, pend);
                __syncwarp();
                if (lane == 0) mbar_arrive(&o_empty[u & 1u]);
            }
        }
        if (ok && ntiles) {
            const uint32_t u = t - 1;
            if (!at_warp_wait(&o_full[u & 1u], (u >> 1) & 1u)) ok = false, *failed = 3;
            if (ok) {
                add_o_tile(u & 1u, 1.f);
                __syncwarp();
                if (lane == 0) mbar_arrive(&o_empty[u & 1u]);
            }
        }
        // the row's denominator is the sum of its two threads' partial sums (same reference maximum in both); the slot is the
        // one the tile before last used for its maxima, which both threads have read
        float *xl = xch + (t & 1u) * 256;
        xl[half * 128 + row] = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(1u + quarter) : "memory");
        const float l_tot = l_run + xl[(half ^ 1u) * 128 + row];
        // the next item's first tile writes its maxima into the same slot: both threads must have read the sums first; the two
        // warps also agree here on whether to go on
        const bool stop = at_pair_sync_or(1u + quarter, !ok || *failed != 0);
        if (stop) break;
        // The output goes through shared memory: a thread owns half a row, so stores straight from its registers would touch 32
        // lines per instruction (measured: ~2900 cycles per item, 9 % of the kernel).  Each thread writes its 128 bytes into its line
        // of a P buffer (both are free: the item's last product has been read), swizzled like P; then the two warps of the lane
        // quarter write the quarter's 32 rows, two whole rows per instruction.
        {
            const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
            uint8_t *stage = sP + (t & 1u) * AT_TILE_BYTES;
            uint8_t *line = stage + half * (AT_TILE_BYTES / 2) + row * 128u;
#pragma unroll
            for (int d = 0; d < 64; d += 8) {
                uint4 v;
                v.x = at_pack2<T>(acc[d] * inv, acc[d + 1] * inv), v.y = at_pack2<T>(acc[d + 2] * inv, acc[d + 3] * inv);
                v.z = at_pack2<T>(acc[d + 4] * inv, acc[d + 5] * inv), v.w = at_pack2<T>(acc[d + 6] * inv, acc[d + 7] * inv);
                *reinterpret_cast<uint4 *>(line + (((d >> 3) ^ (row & 7u)) << 4)) = v;
            }
            asm volatile("bar.sync %0, 64;" ::"r"(1u + quarter) : "memory");
            T *base = static_cast<T *>(a.o) + w.n * a.o_sn + w.h * a.o_sh;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t idx = i * 64u + half * 32u + lane, r = quarter * 32u + (idx >> 4), ch = idx & 15u;
                const uint4 v = *reinterpret_cast<const uint4 *>(stage + (ch >> 3) * (AT_TILE_BYTES / 2) + r * 128u + (((ch & 7u) ^ (r & 7u)) << 4));
                if (q0 + r < a.S) *reinterpret_cast<uint4 *>(base + static_cast<int64_t>(q0 + r) * a.o_st + ch * 8u) = v;
            }
            // the next write into this buffer (the next item's first probabilities) comes after a barrier of the same two warps
        }
        }// items
    }
    tc_fence_before();
    __syncthreads();
    if (warp == AT_SW + 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *failed) atomicExch(&s_attn_tc_error, *failed);
}

// ---- Two query tiles per CTA ---------------------------------------------------------------------------------------------------
// With the softmax warps of the kernel above doing nothing at all, a launch still takes 176 of its 215 us: what bounds it is the
// stream of K / V tiles (every 128 query rows pull all the keys below their diagonal through L2: 1.14 GB per launch on
// [4, 32, 2048, 128], 3.2 x the algorithmic bytes from HBM), not the softmax.  Here a CTA owns 256 query rows of one (sequence, head):
// two groups of eight softmax warps (group g = rows 128 g .. 128 g + 127, two threads per row) share every K / V tile, which halves
// that stream, and take turns on the tensor core: S_g = Q_g K^T into the group's 128 score columns of tensor memory, online softmax
// as above, P written 16-bit OVER the scores the writer has read (two keys per 32-bit column), O_g += P V with the A operand taken
// from tensor memory (P never crosses shared memory) and O_g accumulated in tensor memory (columns 256 + 128 g ..), rescaled in
// place only when the group's reference maximum moves.  Per group the chain is serial (S, softmax, P V, next S: the next scores
// overwrite P), the two groups overlap each other.  No exchange between the groups; each thread finishes its own half row.
// Measured on [4, 32, 2048, 128] bf16: 166-172 us = 801-828 TFLOP/s.  With parts of the softmax left out (results wrong, timing only): no
// exponentials 173 us, no maximum pass 164, no exponential pass 139, no softmax at all 135.5: the products and the K / V stream are
// still four fifths of the time.  Per key tile a CTA moves 256 KiB through shared memory (Q and K for two S products, V for two P V
// products, the TMA writes of K and V) = 2048 cycles of its 128 bytes per clock, as long as the four products take at peak rate.
constexpr int AT2_SW = 16, AT2_THREADS = (AT2_SW + 2) * 32;
constexpr uint32_t AT2_STAGE_BYTES = 16384;// per group: 128 rows x 64 d columns of 16-bit output

struct At2Item {
    uint32_t q0, h, n, kvh, ntiles[2], nt;// key tiles group 0 / 1 walk (group 1's rows lie 128 further down); nt = the larger
};
__device__ __forceinline__ At2Item at2_item(const AttnTcArgs &a, uint32_t qp_tiles, uint32_t i) {
    const uint32_t hn = a.n_heads * a.batch, qp = qp_tiles - 1 - i / hn, r = i % hn;
    At2Item it;
    it.q0 = qp * 2 * AT_BM, it.h = r % a.n_heads, it.n = r / a.n_heads;
    it.kvh = it.h / (a.n_heads / a.n_kv);
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const uint32_t first = it.q0 + g * AT_BM;// a group whose rows all lie behind the sequence has nothing to do
        const uint32_t last_key = first + AT_BM < a.kv_len ? first + AT_BM : a.kv_len;
        it.ntiles[g] = first < a.S ? (last_key + AT_BN - 1) / AT_BN : 0u;
    }
    it.nt = it.ntiles[0] > it.ntiles[1] ? it.ntiles[0] : it.ntiles[1];
    return it;
}
// OR over the 256 threads of a group (barrier 10 + g)
__device__ __forceinline__ bool at2_group_sync_or(uint32_t g, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.u32 q, %2, 0;\n"
        "bar.red.or.pred p, %1, 256, q;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(r)
        : "r"(10u + g), "r"(pred ? 1u : 0u)
        : "memory");
    return r != 0;
}

template<class T>
__global__ void __launch_bounds__(AT2_THREADS, 1) attn_prefill_q2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                                                        const __grid_constant__ CUtensorMap map_v, const AttnTcArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sQ = smem;                          // 2 x 32 KiB: group 0's and group 1's query rows
    uint8_t *sK = sQ + 2 * AT_TILE_BYTES;        // 2 x 32 KiB
    uint8_t *sV = sK + 2 * AT_TILE_BYTES;        // 2 x 32 KiB
    uint8_t *sO = sV + 2 * AT_TILE_BYTES;        // 2 x 16 KiB: output staging of group 0 / 1
    uint64_t *bars = reinterpret_cast<uint64_t *>(sO + 2 * AT2_STAGE_BYTES);
    uint64_t *q_full = bars, *q_empty = bars + 1, *k_full = bars + 2, *k_empty = bars + 4, *v_full = bars + 6, *v_empty = bars + 8;
    uint64_t *s_full = bars + 10, *p_full = bars + 12, *o_full = bars + 14, *o_free = bars + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 18);
    volatile int *failed = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *xch = reinterpret_cast<float *>(bars + 19);// [2 groups][2 halves][128 rows]: half-row maxima of the tile in flight, then the sums
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicExch(&s_attn_tc_error, 5);
        return;
    }
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t qp_tiles = (a.S + 2 * AT_BM - 1) / (2 * AT_BM);
    const uint32_t n_items = qp_tiles * a.n_heads * a.batch;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1), mbar_init(q_empty, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1), mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1), mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1), mbar_init(&p_full[s], AT2_SW / 2);
            mbar_init(&o_full[s], 1), mbar_init(&o_free[s], AT2_SW / 2);
        }
        *failed = 0;
        fence_mbar_init();
    }
    if (warp == AT2_SW + 1) {
        tmem_alloc(tmem_slot, 512);// S (and P) of group 0 / 1, O of group 0 / 1
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();

    if (warp == AT2_SW) {
        if (lane == 0) {
            uint32_t t = 0, done = 0;// t: key tiles over all items of this CTA (stage t & 1, phase (t >> 1) & 1)
            for (uint32_t band = 0; band * gridDim.x < n_items && !*failed; ++band) {
                const uint32_t i = at_item_of(band, n_items);
                if (i >= n_items) continue;
                const At2Item w = at2_item(a, qp_tiles, i);
                if (w.nt == 0) continue;
                if (done && !mbar_wait(q_empty, (done - 1) & 1u)) {// the previous item's last S products have read Q
                    *failed = 1;
                    break;
                }
                mbar_arrive_expect_tx(q_full, 2 * AT_TILE_BYTES);
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    tma_load_4d(sQ + g * AT_TILE_BYTES, &map_q, 0, w.q0 + g * AT_BM, w.h, w.n, q_full);
                    tma_load_4d(sQ + g * AT_TILE_BYTES + AT_TILE_BYTES / 2, &map_q, 64, w.q0 + g * AT_BM, w.h, w.n, q_full);
                }
                for (uint32_t j = 0; j < w.nt; ++j, ++t) {
                    const uint32_t s = t & 1u, ph = (t >> 1) & 1u;
                    if (!mbar_wait(&k_empty[s], ph ^ 1u)) {
                        *failed = 1;
                        break;
                    }
                    mbar_arrive_expect_tx(&k_full[s], AT_TILE_BYTES);
                    tma_load_4d(sK + s * AT_TILE_BYTES, &map_k, 0, j * AT_BN, w.kvh, w.n, &k_full[s]);
                    tma_load_4d(sK + s * AT_TILE_BYTES + AT_TILE_BYTES / 2, &map_k, 64, j * AT_BN, w.kvh, w.n, &k_full[s]);
                    if (!mbar_wait(&v_empty[s], ph ^ 1u)) {
                        *failed = 1;
                        break;
                    }
                    mbar_arrive_expect_tx(&v_full[s], AT_TILE_BYTES);
                    tma_load_4d(sV + s * AT_TILE_BYTES, &map_v, 0, j * AT_BN, w.kvh, w.n, &v_full[s]);
                    tma_load_4d(sV + s * AT_TILE_BYTES + AT_TILE_BYTES / 2, &map_v, 64, j * AT_BN, w.kvh, w.n, &v_full[s]);
                }
                ++done;
            }
        }
    } else if (warp == AT2_SW + 1) {
        if (lane == 0) {
            const uint32_t idesc_s = instr_desc(a.is_bf16, AT_BM, AT_BN);
            const uint32_t idesc_o = instr_desc(a.is_bf16, AT_BM, AT_D) | (1u << 16);// B (= V) is MN-major
            bool ok = true;
            uint32_t t = 0, done = 0;
            uint32_t u[2] = {0, 0}; // tiles group 0 / 1 has been given so far: phases of s_full, p_full and o_full follow them
            uint32_t ig[2] = {0, 0};// items in which group 0 / 1 had tiles: phases of o_free
            // S_g = Q_g K^T of the key tile in stage s; the group's score columns are free: it has read them (p_full) and its P V, which
            // took P from them, was issued before
            auto issue_s = [&](uint32_t g, uint32_t s) {
                const uint32_t q_addr = smem_u32(sQ + g * AT_TILE_BYTES), k_addr = smem_u32(sK + s * AT_TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t off = (kk >> 2) * (AT_TILE_BYTES / 2) + (kk & 3) * 32;
                    tc_mma_f16(tmem_base + g * AT_BN, smem_desc_sw128(q_addr + off), smem_desc_sw128(k_addr + off), idesc_s, kk ? 1u : 0u);
                }
                tc_commit(&s_full[g]);
            };
            for (uint32_t band = 0; ok && band * gridDim.x < n_items; ++band) {
                const uint32_t i = at_item_of(band, n_items);
                if (i >= n_items) continue;
                const At2Item w = at2_item(a, qp_tiles, i);
                if (w.nt == 0) continue;
                ok = mbar_wait(q_full, done & 1u) && mbar_wait(&k_full[t & 1u], (t >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                for (uint32_t g = 0; g < 2; ++g)
                    if (w.ntiles[g]) issue_s(g, t & 1u);
                tc_commit(&k_empty[t & 1u]);
                if (w.nt == 1) tc_commit(q_empty);// the item's last S products: Q may be replaced once they have run
                for (uint32_t j = 0; ok && j < w.nt; ++j, ++t) {
                    const uint32_t s = t & 1u, ph = (t >> 1) & 1u;
                    const bool next = j + 1 < w.nt;
                    if (!mbar_wait(&v_full[s], ph) || (next && !mbar_wait(&k_full[s ^ 1u], ((t + 1) >> 1) & 1u))) {
                        ok = false;
                        break;
                    }
                    const uint32_t v_addr = smem_u32(sV + s * AT_TILE_BYTES);
                    // group by group: its P V of this tile, then its scores of the next one, so that one group's softmax runs under the
                    // other group's products
                    for (uint32_t g = 0; ok && g < 2; ++g) {
                        if (j < w.ntiles[g]) {
                            // O_g (+)= P V once the group has written P (and rescaled O where it moved its maximum); the item's first
                            // tile overwrites O_g, which the group must have read out for its previous item
                            if (!mbar_wait(&p_full[g], u[g] & 1u) || (j == 0 && ig[g] && !mbar_wait(&o_free[g], (ig[g] - 1) & 1u))) {
                                ok = false;
                                break;
                            }
                            tc_fence_after();
#pragma unroll
                            for (int kk = 0; kk < 8; ++kk) {
                                // A = P from tensor memory: keys 16 kk .. 16 kk + 15 of every row are 8 columns of 32 bits; keys 0-63 lie
                                // in columns 0-31 of the group's scores, keys 64-127 in columns 64-95 (each over scores its writer has read)
                                const uint64_t bd = smem_desc_sw128_ex(v_addr + kk * 2048, a.v_lbo, a.v_sbo);
                                tc_mma_f16_ts(tmem_base + (2 + g) * AT_BN, tmem_base + g * AT_BN + (kk >> 2) * 64 + (kk & 3) * 8, bd, idesc_o,
                                              (kk || j) ? 1u : 0u);
                            }
                            tc_commit(&o_full[g]);
                            ++u[g];
                            if (j == 0) ++ig[g];
                        }
                        if (next && j + 1 < w.ntiles[g]) issue_s(g, s ^ 1u);
                    }
                    if (!ok) break;
                    tc_commit(&v_empty[s]);
                    if (next) {
                        tc_commit(&k_empty[s ^ 1u]);
                        if (j + 2 == w.nt) tc_commit(q_empty);
                    }
                }
                ++done;
            }
            if (!ok) *failed = 2;
        }
    } else {
        // ---- softmax warps: group g = warp / 8 owns query rows 128 g .. 128 g + 127 of the item; two threads per row: lane quarter =
        // warp % 4, column half = (warp / 4) % 2 (64 key columns of the scores, 64 d columns of O) ----
        const uint32_t g = warp >> 3, quarter = warp & 3u, half = (warp >> 2) & 1u, row = quarter * 32 + lane;
        const uint32_t lane_addr = (quarter * 32u) << 16, col0 = half * 64u;
        const uint32_t s_addr = tmem_base + g * AT_BN + lane_addr + col0, o_addr = tmem_base + (2 + g) * AT_BN + lane_addr + col0;
        const uint32_t pair_bar = 1u + g * 4u + quarter;// the 64 threads that own these 32 rows
        const float c = a.scale_log2e, thr = 8.0f / c;
        float *xr = xch + g * 256;// [2 halves][128 rows]
        uint8_t *stage = sO + g * AT2_STAGE_BYTES;
        bool ok = true;
        uint32_t u = 0;// key tiles this group has worked on, over all items
        for (uint32_t band = 0; band * gridDim.x < n_items; ++band) {
            const uint32_t item = at_item_of(band, n_items);
            if (item >= n_items) continue;
            const At2Item w = at2_item(a, qp_tiles, item);
            const uint32_t ntiles = w.ntiles[g];
            if (ntiles == 0) continue;
            const uint32_t q0 = w.q0 + g * AT_BM, qrow = q0 + row;
            float m_used = -INFINITY, l_run = 0.f;
            bool stop = false;
            const uint32_t lim = qrow + 1 < a.kv_len ? qrow + 1 : a.kv_len;// first key this row may NOT see
            const uint32_t warp_lim = q0 + quarter * 32 + 1 < a.kv_len ? q0 + quarter * 32 + 1 : a.kv_len;// smallest lim in the warp
            for (uint32_t j = 0; j < ntiles; ++j, ++u) {
                const uint32_t key0 = j * AT_BN + col0;
                if (ok && !at_warp_wait(&s_full[g], u & 1u)) ok = false, *failed = 3;
                tc_fence_after();
                const bool masked = key0 + 64 > warp_lim;// warp-uniform: only the diagonal tile and the sequence's last one
                // pass 1: maximum of this thread's 64 scores, then of the row
                float mx = -INFINITY;
#pragma unroll
                for (int c0 = 0; c0 < 64; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(s_addr + c0, r);
                    tmem_ld_wait();
                    if (masked) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) mx = fmaxf(mx, key0 + c0 + e < lim ? __uint_as_float(r[e]) : -INFINITY);
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(r[e]));
                    }
                }
                // The partner read this slot for the previous tile before it arrived on p_full, and these scores exist only because
                // that arrival let the tensor core go on: one slot is enough.
                xr[half * 128 + row] = mx;
                if (at_pair_sync_or(pair_bar, *failed != 0)) {// the two warps of these rows, leaving together
                    stop = true;
                    break;
                }
                mx = fmaxf(mx, xr[(half ^ 1u) * 128 + row]);
                // Move the reference maximum only when some row of the warp needs it (both warps of a row see the same maxima).  O is
                // rescaled where it lies, every thread its 64 columns: the group's previous P V has run (these scores were issued
                // behind it).
                if (__any_sync(0xffffffffu, mx > m_used + thr)) {
                    const float m_new = fmaxf(m_used, mx);
                    const float alpha = (m_used == -INFINITY) ? 0.f : exp2f((m_used - m_new) * c);
                    if (j) {
#pragma unroll 1
                        for (int c0 = 0; c0 < 64; c0 += 32) {
                            uint32_t r[32];
                            tmem_ld_32x32(o_addr + c0, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
                            tmem_st_32x32(o_addr + c0, r);
                        }
                    }
                    l_run *= alpha;
                    m_used = m_new;
                }
                // pass 2: p = 2^((s - m) * scale) as 16-bit, two keys per 32-bit column, over the first 32 columns of this thread's scores
                const float mneg = (m_used == -INFINITY) ? 0.f : -m_used * c;
                float lsum = 0.f;
#pragma unroll
                for (int c0 = 0; c0 < 64; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(s_addr + c0, r);
                    tmem_ld_wait();
                    uint32_t packed[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        float p0, p1;
                        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(fmaf(__uint_as_float(r[e]), c, mneg)));
                        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(fmaf(__uint_as_float(r[e + 1]), c, mneg)));
                        if (masked) {
                            if (key0 + c0 + e >= lim) p0 = 0.f;
                            if (key0 + c0 + e + 1 >= lim) p1 = 0.f;
                        }
                        lsum += p0 + p1;
                        packed[e / 2] = at_pack2<T>(p0, p1);
                    }
                    // columns [c0 / 2, c0 / 2 + 16) of this thread's 64: all inside what it has read so far
                    tmem_st_32x16(s_addr + c0 / 2, packed);
                }
                l_run += lsum;
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[g]);
            }
            // the group's last product of the item
            if (!stop && ok && !at_warp_wait(&o_full[g], (u - 1) & 1u)) ok = false, *failed = 3;
            // the row's denominator is the sum of its two threads' partial sums; the group agrees on whether to go on
            xr[half * 128 + row] = l_run;
            if (at2_group_sync_or(g, stop || !ok || *failed != 0)) break;
            const float l_tot = l_run + xr[(half ^ 1u) * 128 + row];
            const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
            // Output: half by half (d columns 0-63, then 64-127) through the group's staging buffer, whole 128-byte half rows per store.
            // Each thread owns 64 d columns of its row = one 128-byte line of the round its half takes part in.
            tc_fence_after();
            T *base = static_cast<T *>(a.o) + w.n * a.o_sn + w.h * a.o_sh;
            const uint32_t tid_g = (warp & 7u) * 32 + lane;
#pragma unroll 1
            for (uint32_t round = 0; round < 2; ++round) {
                if (half == round) {
#pragma unroll
                    for (int c0 = 0; c0 < 64; c0 += 32) {
                        uint32_t r[32];
                        tmem_ld_32x32(o_addr + c0, r);
                        tmem_ld_wait();
                        uint32_t packed[16];
#pragma unroll
                        for (int e = 0; e < 32; e += 2) packed[e / 2] = at_pack2<T>(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint32_t chunk = (c0 >> 3) + q;
                            *reinterpret_cast<uint4 *>(stage + row * 128u + ((chunk ^ (row & 7u)) << 4)) =
                                make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                        }
                    }
                    tc_fence_before();
                }
                asm volatile("bar.sync %0, 256;" ::"r"(10u + g) : "memory");
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t idx = i * 256u + tid_g, r = idx >> 3, ch = idx & 7u;
                    const uint4 v = *reinterpret_cast<const uint4 *>(stage + r * 128u + ((ch ^ (r & 7u)) << 4));
                    if (q0 + r < a.S) *reinterpret_cast<uint4 *>(base + static_cast<int64_t>(q0 + r) * a.o_st + round * 64 + ch * 8u) = v;
                }
                asm volatile("bar.sync %0, 256;" ::"r"(10u + g) : "memory");
            }
            // O_g has been read out (the barriers above order every thread's loads before this): the next item may overwrite it
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_free[g]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == AT2_SW + 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *failed) atomicExch(&s_attn_tc_error, *failed);
}

int attn_tc_error_word(bool clear) { return error_symbol(s_attn_tc_error, clear); }

// (64 columns of d, tokens, heads, sequences) with the caller's element strides; box = 64 x 128 tokens, 128-byte swizzle
static bool make_map_4d(CUtensorMap *map, const void *base, int is_bf16, uint64_t tokens, uint64_t heads, uint64_t seqs, int64_t st, int64_t sh,
                        int64_t sn) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {128, tokens, heads, seqs};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(st) * 2, static_cast<cuuint64_t>(sh) * 2, static_cast<cuuint64_t>(sn) * 2};
    const cuuint32_t box[4] = {64, 128, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(base), dims, strides, box,
              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// True when the tcgen05 kernel can serve the request: prefill from position 0 (no device-side past), enough rows for a tile,
// strides a tensor map can express.  RG_B200_ATTN_TC=0 keeps every request on the warp-level kernel.
bool attn_prefill_tc_applies(const rg_attn_prefill_params *p, const void *const *in) {
    static const bool on = [] {
        const char *e = std::getenv("RG_B200_ATTN_TC");
        return !(e && e[0] == '0');
    }();
    if (!on || in[3] != nullptr || p->head_dim != AT_D || p->seq_len < 128) return false;
    if (p->dtype != RG_FP16 && p->dtype != RG_BF16) return false;
    for (int i = 0; i < 12; ++i)
        if (p->strides[i] <= 0 || p->strides[i] % 8 != 0) return false;
    return encode_fn() != nullptr;
}

int attn_prefill_tc_launch(const rg_attn_prefill_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    const int64_t *s = p->strides;
    const int is_bf16 = p->dtype == RG_BF16;
    const uint32_t kv_len = p->seq_len < p->kv_capacity ? p->seq_len : p->kv_capacity;
    CUtensorMap mq, mk, mv;
    // rows past kv_len are outside the K / V maps, so they arrive as zeros instead of whatever the cache holds there
    if (!make_map_4d(&mq, in[0], is_bf16, p->seq_len, p->n_heads, p->batch, s[2], s[1], s[0]) ||
        !make_map_4d(&mk, in[1], is_bf16, kv_len, p->n_kv_heads, p->batch, s[5], s[4], s[3]) ||
        !make_map_4d(&mv, in[2], is_bf16, kv_len, p->n_kv_heads, p->batch, s[8], s[7], s[6]))
        return RG_ERR_UNSUPPORTED;
    AttnTcArgs a = {};
    a.o = out[0];
    a.o_sn = s[9], a.o_sh = s[10], a.o_st = s[11];
    a.n_heads = p->n_heads, a.n_kv = p->n_kv_heads, a.S = p->seq_len, a.kv_len = kv_len;
    a.scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(AT_D));
    a.is_bf16 = is_bf16;
    // MN-major operand: the next 64 columns of d are the other half tile (16 KiB further), the next 8 keys 1 KiB further
    static const uint32_t lbo = std::getenv("RG_B200_ATTN_V_LBO") ? static_cast<uint32_t>(atoi(std::getenv("RG_B200_ATTN_V_LBO"))) : AT_TILE_BYTES / 2;
    static const uint32_t sbo = std::getenv("RG_B200_ATTN_V_SBO") ? static_cast<uint32_t>(atoi(std::getenv("RG_B200_ATTN_V_SBO"))) : 1024u;
    a.v_lbo = lbo, a.v_sbo = sbo;
    const size_t smem = 7 * AT_TILE_BYTES + 20 * 8 + 2 * 256 * 4;
    a.q_tiles = (p->seq_len + AT_BM - 1) / AT_BM, a.batch = p->batch;
    const uint32_t sms = static_cast<uint32_t>(sm_count());
    // the kernel with two query tiles per CTA (171.7 us = 801 TFLOP/s on [4, 32, 2048, 128] bf16 against 215 us = 639 for the kernel
    // with one, same box); RG_B200_ATTN_Q2=0 keeps the latter
    static const bool q2 = !(std::getenv("RG_B200_ATTN_Q2") && std::getenv("RG_B200_ATTN_Q2")[0] == '0');
    if (q2 && kv_len > 0) {// (no keys at all: the other kernel writes the zero rows)
        const size_t smem2 = 6 * AT_TILE_BYTES + 2 * AT2_STAGE_BYTES + 20 * 8 + 2048;
        const uint64_t items2 = static_cast<uint64_t>((p->seq_len + 2 * AT_BM - 1) / (2 * AT_BM)) * p->n_heads * p->batch;
        if (items2 > 0xffffffffull) return RG_ERR_SHAPE;
        dim3 grid2(static_cast<unsigned>(items2 < sms ? items2 : sms));
        if (is_bf16) {
            RG_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_q2_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem2)));
            RG_CHECK_CUDA(launch_pdl(attn_prefill_q2_kernel<__nv_bfloat16>, grid2, dim3(AT2_THREADS), smem2, st, mq, mk, mv, a));
        } else {
            RG_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_q2_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem2)));
            RG_CHECK_CUDA(launch_pdl(attn_prefill_q2_kernel<__half>, grid2, dim3(AT2_THREADS), smem2, st, mq, mk, mv, a));
        }
        count_launch();
        return RG_OK;
    }
    // persistent CTAs, one per SM (the shared memory of a CTA fills the SM): the next item's Q, K and V are fetched while the
    // softmax warps finish the current one, and tensor memory and barriers are set up once
    const uint64_t items = static_cast<uint64_t>(a.q_tiles) * p->n_heads * p->batch;
    if (items > 0xffffffffull) return RG_ERR_SHAPE;
    dim3 grid(static_cast<unsigned>(items < sms ? items : sms));
    if (is_bf16) {
        RG_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        RG_CHECK_CUDA(launch_pdl(attn_prefill_tc_kernel<__nv_bfloat16>, grid, dim3(AT_THREADS), smem, st, mq, mk, mv, a));
    } else {
        RG_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        RG_CHECK_CUDA(launch_pdl(attn_prefill_tc_kernel<__half>, grid, dim3(AT_THREADS), smem, st, mq, mk, mv, a));
    }
    count_launch();
    return RG_OK;
}

}// namespace rg
