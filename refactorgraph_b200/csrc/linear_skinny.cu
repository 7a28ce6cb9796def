// Weight-streaming linear layer for 5..32 rows of X (batched decode, one rank of a tensor-parallel step):
//   Y = epilogue(X * W^T),  W[n,k] row-major 16-bit, fp32 accumulation.
// Such a product is HBM-bound (every weight byte is used for at most 32 multiply-adds), so the kernel is built like
// the m <= 4 streaming kernel — persistent grid, weights pulled through a shared-memory ring by bulk copies that do not
// wait for the previous kernel — and only the arithmetic differs: the 16 (or 32) activation rows are the M side of
// mma.sync.m16n8k16, eight weight rows its N side.
//
//  * k is cut into `ksplit` parts so that a warp's share of X fits in registers as A fragments (64 registers): the eight
//    consumer warps take the eight 16-column steps of every 128-column block, a part has at most 16 blocks (8 for 32 rows).
//  * a unit = (block of R = 8 or 16 weight rows, part) = 32 KiB.  W is described to the TMA unit as a 3-D tensor
//    (64 columns, rows, k / 64 column blocks), so ONE tiled copy brings a unit's box [column block][row][128 bytes] (two copies
//    when the epilogue pairs rows from two places); per-row bulk copies of 2-4 KiB ran into the copy unit's request rate
//    (~9 M requests/s per SM) long before HBM.  The 128-byte swizzle puts the eight rows a B-fragment load touches on
//    eight different bank groups.
//  * per unit every warp holds a 16 x 8 (x MT x NT) partial tile, which it parks in a ring of shared-memory buffers and
//    moves on — the consumer warps never meet at a barrier; four epilogue warps sum the eight tiles of a unit in warp
//    order and finish it: with ksplit > 1 the tile goes to a scratch area and the last part to arrive sums all parts in part order
//    (self-resetting counters), then the epilogue runs: plain store, alpha/beta with a C operand, SiLU gate on paired
//    gate / up rows, or QKV split + rotary embedding + KV-cache append on paired (i, i + D/2) rows.
//  * every wait is bounded; a wait that runs out is recorded and all threads leave through the same barriers.
// Summation order is fixed (k steps, then warps, then parts), so results do not depend on timing.
//
// Where it is used.  On B200 the warp-level mma.sync path runs at about an eighth of the tcgen05 rate, and with 16 rows of X
// this kernel needs ~60 % of that for the multiply-adds alone: cycle counters in the consumer warps show ~870 cycles per 32 KiB
// unit inside the mma loop and ~120 waiting for data, i.e. the tensor path, not HBM, bounds it (3.8-4.4 TB/s on 134 MB of
// weights, where the tcgen05 kernel streams 5.0).  It wins where the tcgen05 kernel's 128-row tiles are too few to fill the
// GPU without a deep split (1280 x 8192 weights, one rank's QKV projection at tensor-parallel 8: 13.0 us against 18.3 us) and
// it carries the RoPE / cache-append and SiLU epilogues for 5..32 rows, so the dispatch (mat_mul.cu, host fusion pass) sends
// it the products with few rows of W and a long k, and leaves the rest on tcgen05.  Also measured and dropped: per-row 1-D
// bulk copies instead of the tiled box (same speed), a CTA-wide barrier per unit for the cross-warp sum (same speed),
// an L2 prefetch cursor eight units ahead of the ring (8-15 % slower), five instead of six stages (same speed).
#include "gemm_dispatch.cuh"
#include <cuda.h>
#include <cstdlib>

namespace rg {

bool tma_encode_rows_by_blocks(void *map, const void *base, int is_bf16, uint64_t rows, uint64_t k, uint32_t box_rows, uint32_t box_blocks);// gemm_tc.cu

constexpr int SK_NW = 8;                              // consumer warps
constexpr int SK_EW = 4;                              // epilogue warps
constexpr int SK_THREADS = (SK_NW + SK_EW + 1) * 32;  // + producer warp
constexpr int SK_STAGES = 6;
constexpr uint32_t SK_STAGE_BYTES = 33 * 1024;        // a 32 KiB box, or two 16 KiB boxes the second of which starts 512 bytes later (see sk_sub_offset)

static __device__ int s_skinny_error;      // a bounded wait ran out
static __device__ int s_skinny_index_error;// a cache-append position or block-table entry was out of range (store skipped)

struct SkinnyArgs {
    const void *W, *X, *C;
    const int64_t *pos;
    const int32_t *table;
    void *Y, *kc, *vc;
    float *part;
    unsigned *cnt;
    uint32_t m, n, k;
    int epilogue;// 0 store, 1 alpha * acc + beta * C, 2 SiLU gate, 3 QKV split + RoPE + cache append
    float alpha, beta;
    uint32_t c_row_stride, c_col_stride, y_row_stride;
    uint32_t n_heads;
    float log2_theta;
    rg_kv_layout kv;
    uint32_t tokens_per_seq;
    uint32_t ksplit, kblocks, nrb, units;
    int w_static;
};

// 3-D tiled copy (128-byte swizzle) into this CTA's shared memory with an L2 eviction hint, completion counted on `bar`
__device__ __forceinline__ void sk_tma_load(void *dst, const CUtensorMap *map, uint32_t row, uint32_t block, uint64_t *bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(0u), "r"(row), "r"(block), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
// Where the 128-byte swizzle puts a byte whose unswizzled offset from a 1024-byte aligned base is `off`: bits 4-6 ^= bits 7-9.
__device__ __forceinline__ uint32_t sk_swz(uint32_t off) { return off ^ ((off >> 3) & 0x70u); }
// Stage offset of the second half of a paired unit.  With 4-row halves both halves' rows would fall on the same four swizzle
// phases; starting the second box 512 bytes (four 128-byte lines) later shifts its phases by four.
template<int R> __device__ __forceinline__ constexpr uint32_t sk_sub_offset() { return 16384u + (R == 8 ? 512u : 0u); }

// global row of W behind row j of row block rb, or 0xffffffff when the block has no such row
template<int R>
__device__ __forceinline__ uint32_t sk_unit_row(const SkinnyArgs &a, uint32_t rb, uint32_t j) {
    constexpr uint32_t half = R / 2;
    if (a.epilogue == 2) {// rows past the gate (up) half are never stored: the copy may fetch whatever lies there
        const uint32_t F = a.n / 2, r = rb * half + (j % half);
        return j < half ? r : F + r;
    }
    if (a.epilogue == 3) {
        const uint32_t D = a.kv.head_dim, per_head = (D / 2) / half;
        return (rb / per_head) * D + (j < half ? 0u : D / 2) + (rb % per_head) * half + (j % half);
    }
    const uint32_t r = rb * R + j;
    return r < a.n ? r : 0xffffffffu;
}

template<class T> __device__ __forceinline__ uint32_t sk_pack2(float lo, float hi);
template<> __device__ __forceinline__ uint32_t sk_pack2<__half>(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}
template<> __device__ __forceinline__ uint32_t sk_pack2<__nv_bfloat16>(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// Stores y[tok, col] and y[tok, col + 1] (the two values a lane holds next to each other), as one 32-bit word when possible.
template<class T>
__device__ __forceinline__ void sk_store2(T *base, uint64_t off, float v0, float v1, bool two, bool aligned) {
    if (two && aligned) {
        *reinterpret_cast<uint32_t *>(base + off) = sk_pack2<T>(v0, v1);
    } else {
        base[off] = Num<T>::from_f(v0);
        if (two) base[off + 1] = Num<T>::from_f(v1);
    }
}

template<class T, int MT, int NT>
__global__ void __launch_bounds__(SK_THREADS, 1) linear_skinny_kernel(const __grid_constant__ CUtensorMap map_full,
                                                                      const __grid_constant__ CUtensorMap map_half, const SkinnyArgs a) {
    constexpr int R = 8 * NT;                 // weight rows per unit
    constexpr int BMAX = 16 / MT;             // 128-column blocks per part
    constexpr int TILE = MT * NT * 128;       // floats of a unit's output tile, in C-fragment order
    constexpr int NBUF = MT * NT >= 4 ? 1 : 4; // partial-tile buffers in flight (16 KiB of shared memory either way)
    constexpr int EWU = NBUF < SK_EW ? NBUF : SK_EW;// epilogue warps in use: a buffer always belongs to the same warp
    static_assert(2 * BMAX * R * 128 == 32768, "a unit is a 32 KiB box");
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *ring = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);// the swizzle is a function of address bits 7-9
    float *pbuf = reinterpret_cast<float *>(ring + SK_STAGES * SK_STAGE_BYTES);// [NBUF][SK_NW][TILE]
    uint64_t *full = reinterpret_cast<uint64_t *>(pbuf + NBUF * SK_NW * TILE);
    uint64_t *empty = full + SK_STAGES;
    uint64_t *slot_full = empty + SK_STAGES;  // [NBUF] all eight warps have parked their tile of the unit
    uint64_t *slot_empty = slot_full + 8;     // [NBUF] the epilogue warp has taken the tiles
    volatile int *failed = reinterpret_cast<volatile int *>(slot_empty + 8);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3u;
    const uint32_t u0 = static_cast<uint32_t>(static_cast<uint64_t>(a.units) * blockIdx.x / gridDim.x);
    const uint32_t u1 = static_cast<uint32_t>(static_cast<uint64_t>(a.units) * (blockIdx.x + 1) / gridDim.x);
    const uint32_t nu = u1 - u0;

    if (tid == 0) {
        for (int s = 0; s < SK_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], SK_NW);
        }
        for (int s = 0; s < NBUF; ++s) {
            mbar_init(&slot_full[s], SK_NW);
            mbar_init(&slot_empty[s], 1);
        }
        *failed = 0;
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == SK_NW + SK_EW) {
        // ---------------- producer: one thread, one or two tiled copies per unit ----------------
        if (lane == 0) {
            if (!a.w_static) pdl_wait();
            const uint64_t policy = l2_policy_evict_first();
            const bool paired = a.epilogue >= 2;
            uint32_t p = u0 / a.nrb, rb = u0 % a.nrb;
            for (uint32_t i = 0; i < nu; ++i) {
                const uint32_t s = i % SK_STAGES, ph = (i / SK_STAGES) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u)) {
                    atomicExch(&s_skinny_error, 2);
                    break;
                }
                const uint32_t kb0 = a.kblocks * p / a.ksplit;
                uint8_t *st = ring + s * SK_STAGE_BYTES;
                mbar_arrive_expect_tx(&full[s], 32768u);// the box is always complete: rows or column blocks outside W arrive as zeros
                if (!paired) {
                    sk_tma_load(st, &map_full, rb * R, 2 * kb0, &full[s], policy);
                } else {
                    sk_tma_load(st, &map_half, sk_unit_row<R>(a, rb, 0) & 0x7fffffffu, 2 * kb0, &full[s], policy);
                    sk_tma_load(st + sk_sub_offset<R>(), &map_half, sk_unit_row<R>(a, rb, R / 2) & 0x7fffffffu, 2 * kb0, &full[s], policy);
                }
                if (++rb == a.nrb) rb = 0, ++p;
            }
        }
        return;
    }

    if (warp >= SK_NW) {
        // ---------------- epilogue warps: warp e finishes the units i = e, e + 4, ... ----------------
        pdl_wait();
        const uint32_t e = warp - SK_NW;
        if (e >= EWU) return;
        T *Y = static_cast<T *>(a.Y);
        const T *C = static_cast<const T *>(a.C);
        for (uint32_t i = e; i < nu; i += EWU) {
            const uint32_t sl = i % NBUF;
            if (!mbar_wait(&slot_full[sl], (i / NBUF) & 1u)) {
                atomicExch(&s_skinny_error, 3);
                return;
            }
            if (*failed) return;
            // the eight warps' tiles, summed in warp order
            float4 v[MT * NT];
#pragma unroll
            for (int q = 0; q < MT * NT; ++q) {
                const float *src = pbuf + static_cast<size_t>(sl) * SK_NW * TILE + q * 128 + lane * 4;
                float4 sum = *reinterpret_cast<const float4 *>(src);
#pragma unroll
                for (int w = 1; w < SK_NW; ++w) {
                    const float4 x4 = *reinterpret_cast<const float4 *>(src + w * TILE);
                    sum.x += x4.x, sum.y += x4.y, sum.z += x4.z, sum.w += x4.w;
                }
                v[q] = sum;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&slot_empty[sl]);
            const uint32_t u = u0 + i, p = u / a.nrb, rb = u % a.nrb;
            if (a.ksplit > 1) {
                float *mine = a.part + (static_cast<size_t>(rb) * a.ksplit + p) * TILE;
#pragma unroll
                for (int q = 0; q < MT * NT; ++q) __stcg(reinterpret_cast<float4 *>(mine + q * 128 + lane * 4), v[q]);
                __threadfence();
                __syncwarp();
                unsigned old = 0;
                if (lane == 0) old = atomicAdd(&a.cnt[rb], 1u);
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old != a.ksplit - 1) continue;// another part finishes this row block
                __threadfence();
#pragma unroll
                for (int q = 0; q < MT * NT; ++q) v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (uint32_t pp = 0; pp < a.ksplit; ++pp) {
                    const float *src = a.part + (static_cast<size_t>(rb) * a.ksplit + pp) * TILE;
#pragma unroll
                    for (int q = 0; q < MT * NT; ++q) {
                        const float4 w = __ldcg(reinterpret_cast<const float4 *>(src + q * 128 + lane * 4));
                        v[q].x += w.x, v[q].y += w.y, v[q].z += w.z, v[q].w += w.w;
                    }
                }
                if (lane == 0) a.cnt[rb] = 0u;// ready for the next launch that uses this workspace
            }
            // ---- epilogue on the finished tile: lane (g, t) holds tokens g, g + 8 (+16 mt), columns 2t, 2t + 1 (+8 nt) ----
            if (a.epilogue <= 1) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const float4 c = v[mt * NT + nt];
                        const uint32_t col = rb * R + nt * 8 + 2 * t;
                        if (col >= a.n) continue;
                        const bool two = col + 1 < a.n, al = ((a.y_row_stride | col) & 1u) == 0;
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const uint32_t tok = mt * 16 + g + 8 * hh;
                            if (tok >= a.m) continue;
                            float y0 = a.alpha * (hh ? c.z : c.x), y1 = a.alpha * (hh ? c.w : c.y);
                            if (a.epilogue == 1) {
                                const uint64_t co = static_cast<uint64_t>(tok) * a.c_row_stride + static_cast<uint64_t>(col) * a.c_col_stride;
                                y0 += a.beta * Num<T>::to_f(C[co]);
                                if (two) y1 += a.beta * Num<T>::to_f(C[co + a.c_col_stride]);
                            }
                            sk_store2<T>(Y, static_cast<uint64_t>(tok) * a.y_row_stride + col, y0, y1, two, al);
                        }
                    }
                continue;
            }
            // paired rows: lo = first half of the unit's rows, hi = second half; value index j = position inside the half
            constexpr uint32_t half = R / 2;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                float4 lo4, hi4;
                bool mine;
                if constexpr (NT == 2) {
                    lo4 = v[mt * 2], hi4 = v[mt * 2 + 1], mine = true;// tile 0 holds the lo rows, tile 1 the hi rows
                } else {
                    const float4 own = v[mt];
                    float4 oth;
                    oth.x = __shfl_xor_sync(0xffffffffu, own.x, 2), oth.y = __shfl_xor_sync(0xffffffffu, own.y, 2);
                    oth.z = __shfl_xor_sync(0xffffffffu, own.z, 2), oth.w = __shfl_xor_sync(0xffffffffu, own.w, 2);
                    lo4 = own, hi4 = oth, mine = t < 2;// columns 0..3 are lo rows, 4..7 hi rows: lanes t < 2 own the lo side
                }
                if (!mine) continue;
                const uint32_t j = 2 * (NT == 2 ? t : (t & 1u));
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const uint32_t tok = mt * 16 + g + 8 * hh;
                    if (tok >= a.m) continue;
                    const float l0 = a.alpha * (hh ? lo4.z : lo4.x), l1 = a.alpha * (hh ? lo4.w : lo4.y);
                    const float h0 = a.alpha * (hh ? hi4.z : hi4.x), h1 = a.alpha * (hh ? hi4.w : hi4.y);
                    if (a.epilogue == 2) {
                        const uint32_t F = a.n / 2, col = rb * half + j;
                        if (col >= F) continue;
                        const float y0 = l0 / (1.f + expf(-l0)) * h0, y1 = l1 / (1.f + expf(-l1)) * h1;
                        sk_store2<T>(Y, static_cast<uint64_t>(tok) * a.y_row_stride + col, y0, y1, col + 1 < F, ((a.y_row_stride | col) & 1u) == 0);
                        continue;
                    }
                    // QKV: head h, pair (i, i + D/2) for i = i0 + j, j + 1
                    const uint32_t D = a.kv.head_dim, per_head = (D / 2) / half, nq = a.n_heads, nkv = a.kv.n_kv_heads;
                    const uint32_t h = rb / per_head, i0 = (rb % per_head) * half + j;
                    const int64_t ps = a.pos[tok];
                    float lo[2] = {l0, l1}, hi[2] = {h0, h1};
                    if (h < nq + nkv) {
#pragma unroll
                        for (int x = 0; x < 2; ++x) {
                            const float inv_freq = exp2f(-a.log2_theta * (2.0f * static_cast<float>(i0 + x) / static_cast<float>(D)));
                            float sn, cs;
                            sincosf(static_cast<float>(ps) * inv_freq, &sn, &cs);
                            const float r0 = lo[x] * cs - hi[x] * sn, r1 = hi[x] * cs + lo[x] * sn;
                            lo[x] = r0, hi[x] = r1;
                        }
                    }
                    T *dst;
                    if (h < nq) {
                        dst = Y + (static_cast<uint64_t>(tok) * nq + h) * D;
                    } else {
                        const bool is_k = h < nq + nkv;
                        const uint32_t kvh = is_k ? h - nq : h - nq - nkv;
                        const uint32_t seq = a.tokens_per_seq > 1 ? tok / a.tokens_per_seq : tok;
                        if (!kv_pos_ok(ps, a.kv, a.table != nullptr)) {
                            s_skinny_index_error = 1;
                            continue;
                        }
                        uint64_t base;
                        if (a.table) {
                            const uint32_t page = a.kv.page_size;
                            const int32_t blk = a.table[static_cast<uint64_t>(seq) * a.kv.max_blocks_per_seq + static_cast<uint32_t>(ps) / page];
                            if (!kv_block_ok(blk, a.kv)) {
                                s_skinny_index_error = 1;
                                continue;
                            }
                            base = ((static_cast<uint64_t>(blk) * nkv + kvh) * page + static_cast<uint32_t>(ps) % page) * D;
                        } else {
                            base = ((static_cast<uint64_t>(seq) * nkv + kvh) * a.kv.max_seq + static_cast<uint64_t>(ps)) * D;
                        }
                        dst = static_cast<T *>(is_k ? a.kc : a.vc) + base;
                    }
                    *reinterpret_cast<uint32_t *>(dst + i0) = sk_pack2<T>(lo[0], lo[1]);          // i0 is even, rows are 16-byte aligned
                    *reinterpret_cast<uint32_t *>(dst + i0 + D / 2) = sk_pack2<T>(hi[0], hi[1]);
                }
            }
        }
        return;
    }

    // ---------------- consumers: warp w owns the 16-column step w of every 128-column block ----------------
    pdl_wait();// X comes from the previous kernel
    const uint32_t *Xw = static_cast<const uint32_t *>(a.X);
    uint32_t xf[BMAX][MT][4];
    uint32_t cur_part = 0xffffffffu, nb = 0;
    uint32_t p = u0 / a.nrb, rbc = u0 % a.nrb;
    for (uint32_t i = 0; i < nu; ++i) {
        if (i && ++rbc == a.nrb) rbc = 0, ++p;
        if (p != cur_part) {
            cur_part = p;
            const uint32_t kb0 = a.kblocks * p / a.ksplit;
            nb = a.kblocks * (p + 1) / a.ksplit - kb0;
#pragma unroll
            for (int b = 0; b < BMAX; ++b)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint32_t k0 = (kb0 + b) * 128u + warp * 16u + 2u * t;
                    const uint32_t r0 = mt * 16 + g, r1 = r0 + 8;
                    const bool lb = static_cast<uint32_t>(b) < nb;
                    // A fragment of m16n8k16: (row g, k 2t), (row g + 8, k 2t), (row g, k 2t + 8), (row g + 8, k 2t + 8)
                    xf[b][mt][0] = (lb && r0 < a.m) ? __ldcg(Xw + (static_cast<uint64_t>(r0) * a.k + k0) / 2) : 0u;
                    xf[b][mt][1] = (lb && r1 < a.m) ? __ldcg(Xw + (static_cast<uint64_t>(r1) * a.k + k0) / 2) : 0u;
                    xf[b][mt][2] = (lb && r0 < a.m) ? __ldcg(Xw + (static_cast<uint64_t>(r0) * a.k + k0 + 8) / 2) : 0u;
                    xf[b][mt][3] = (lb && r1 < a.m) ? __ldcg(Xw + (static_cast<uint64_t>(r1) * a.k + k0 + 8) / 2) : 0u;
                }
        }
        const uint32_t s = i % SK_STAGES, ph = (i / SK_STAGES) & 1u;
        const bool got = __all_sync(0xffffffffu, mbar_wait(&full[s], ph) ? 1 : 0) != 0;// uniform for the warp
        if (!got) *failed = 1;
        // CH independent accumulator chains per output tile (k blocks b, b + CH, ...): a chain of dependent mma.sync instructions
        // runs at the instruction's latency, not at its issue rate
        constexpr int CH = MT * NT >= 4 ? 1 : 4;
        float accc[CH][MT][NT][4];
#pragma unroll
        for (int c = 0; c < CH; ++c)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int r = 0; r < 4; ++r) accc[c][mt][nt][r] = 0.f;
        if (got) {
            // row g of n-tile nt, columns b * 128 + warp * 16 + 2t (+8): column block 2b + warp / 4, byte (warp % 4) * 32 + 4t (+16)
            // of its 128-byte line; a box holds [column block][row][128 bytes], swizzled
            const uint8_t *st = ring + s * SK_STAGE_BYTES;
            const bool paired = a.epilogue >= 2;
            uint32_t rowoff[NT], rows_in_box[NT];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t j = nt * 8 + g;
                if (!paired) rowoff[nt] = j * 128u, rows_in_box[nt] = R;
                else
                    rowoff[nt] = (j >= R / 2 ? sk_sub_offset<R>() : 0u) + (j % (R / 2)) * 128u, rows_in_box[nt] = R / 2;
            }
            const uint32_t inline_off = (warp & 3u) * 32u + t * 4u;
            // all B fragments of the unit are loaded before the first mma, so that the shared-memory latency is paid once per
            // unit and not once per k block; a full part takes the branch-free path
            uint32_t bf[BMAX][NT][2];
            if (nb == BMAX) {
#pragma unroll
                for (int b = 0; b < BMAX; ++b)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const uint32_t off = rowoff[nt] + (2u * b + (warp >> 2)) * rows_in_box[nt] * 128u + inline_off;
                        bf[b][nt][0] = *reinterpret_cast<const uint32_t *>(st + sk_swz(off));
                        bf[b][nt][1] = *reinterpret_cast<const uint32_t *>(st + sk_swz(off + 16u));
                    }
#pragma unroll
                for (int b = 0; b < BMAX; ++b)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) mma16816<T>(accc[b % CH][mt][nt], xf[b][mt], bf[b][nt][0], bf[b][nt][1]);
            } else {
#pragma unroll
                for (int b = 0; b < BMAX; ++b) {
                    if (static_cast<uint32_t>(b) < nb) {
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const uint32_t off = rowoff[nt] + (2u * b + (warp >> 2)) * rows_in_box[nt] * 128u + inline_off;
                            const uint32_t b0 = *reinterpret_cast<const uint32_t *>(st + sk_swz(off));
                            const uint32_t b1 = *reinterpret_cast<const uint32_t *>(st + sk_swz(off + 16u));
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) mma16816<T>(accc[b % CH][mt][nt], xf[b][mt], b0, b1);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        float acc[MT][NT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float v = accc[0][mt][nt][r];
#pragma unroll
                    for (int c = 1; c < CH; ++c) v += accc[c][mt][nt][r];
                    acc[mt][nt][r] = v;
                }
        if (!got) break;// this warp gives up; the others run into their own bounded waits
        // park this warp's partial tile in the unit's buffer and move on
        const uint32_t sl = i % NBUF;
        int oks = 1;
        if (lane == 0) oks = mbar_wait(&slot_empty[sl], ((i / NBUF) & 1u) ^ 1u) ? 1 : 0;
        if (!__shfl_sync(0xffffffffu, oks, 0)) {
            *failed = 1;
            break;
        }
        float *pb = pbuf + (static_cast<size_t>(sl) * SK_NW + warp) * TILE;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                *reinterpret_cast<float4 *>(pb + (mt * NT + nt) * 128 + lane * 4) = make_float4(acc[mt][nt][0], acc[mt][nt][1], acc[mt][nt][2], acc[mt][nt][3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&slot_full[sl]);
    }
    if (*failed && lane == 0) atomicExch(&s_skinny_error, 1);
}

int skinny_error_word(bool clear) { return error_symbol(s_skinny_error, clear); }
int skinny_index_error_word(bool clear) { return error_symbol(s_skinny_index_error, clear); }

// ---- host ---------------------------------------------------------------------------------------
struct SkinnyPlan {
    uint32_t mt, nt, R, ksplit, kblocks, nrb, units, tile;
    size_t cnt_bytes, part_bytes, smem;
};

static int skinny_plan(int dtype, uint32_t m, uint32_t n, uint32_t k, int epilogue, const rg_kv_layout *kv, uint32_t n_heads, SkinnyPlan &pl) {
    if (dtype != RG_FP16 && dtype != RG_BF16) return RG_ERR_DTYPE;
    if (m == 0 || m > 32 || n == 0 || k == 0 || k % 128 != 0) return RG_ERR_SHAPE;
    if (epilogue < 0 || epilogue > 3) return RG_ERR_UNSUPPORTED;
    pl.mt = m <= 16 ? 1 : 2, pl.nt = pl.mt;
    pl.R = 8 * pl.nt;
    const uint32_t bmax = 16 / pl.mt, half = pl.R / 2;
    pl.kblocks = k / 128;
    pl.ksplit = (pl.kblocks + bmax - 1) / bmax;
    if (epilogue == 2) {
        if (n % 2 != 0) return RG_ERR_SHAPE;
        pl.nrb = (n / 2 + half - 1) / half;
    } else if (epilogue == 3) {
        if (!kv) return RG_ERR_NULL;
        const uint32_t D = kv->head_dim;
        if (D == 0 || (D / 2) % half != 0 || n != (n_heads + 2 * kv->n_kv_heads) * D) return RG_ERR_SHAPE;
        pl.nrb = n / pl.R;
    } else {
        pl.nrb = (n + pl.R - 1) / pl.R;
    }
    const uint64_t units = static_cast<uint64_t>(pl.nrb) * pl.ksplit;
    if (units > 0xffffffffull) return RG_ERR_SHAPE;
    pl.units = static_cast<uint32_t>(units);
    pl.tile = pl.mt * pl.nt * 128;
    pl.cnt_bytes = pl.ksplit > 1 ? (static_cast<size_t>(pl.nrb) * 4 + 255) / 256 * 256 : 0;
    pl.part_bytes = pl.ksplit > 1 ? static_cast<size_t>(pl.nrb) * pl.ksplit * pl.tile * 4 : 0;
    pl.smem = SK_STAGES * SK_STAGE_BYTES + 4 * SK_NW * 128 * 4 + (2 * SK_STAGES + 16) * 8 + 16 + 1024;// + room to align the ring to 1 KiB
    return RG_OK;
}

bool linear_skinny_shape(int dtype, uint32_t m, uint32_t n, uint32_t k) {
    SkinnyPlan pl;
    return m > 4 && skinny_plan(dtype, m, n, k, 0, nullptr, 0, pl) == RG_OK;
}
size_t linear_skinny_workspace(int dtype, uint32_t m, uint32_t n, uint32_t k, int epilogue, const rg_kv_layout *kv, uint32_t n_heads) {
    SkinnyPlan pl;
    if (skinny_plan(dtype, m, n, k, epilogue, kv, n_heads, pl) != RG_OK) return 0;
    return pl.cnt_bytes + pl.part_bytes;
}

template<class T>
static int skinny_launch(const SkinnyArgs &a, const SkinnyPlan &pl, int is_bf16, cudaStream_t st) {
    // one unit = box of R rows (or two boxes of R / 2 rows) x 32 / MT column blocks of 64
    CUtensorMap full, half;
    const uint32_t blocks = 32 / pl.mt;
    if (!tma_encode_rows_by_blocks(&full, a.W, is_bf16, a.n, a.k, pl.R, blocks) ||
        !tma_encode_rows_by_blocks(&half, a.W, is_bf16, a.n, a.k, pl.R / 2, blocks))
        return RG_ERR_UNSUPPORTED;
    void (*kern)(const CUtensorMap, const CUtensorMap, const SkinnyArgs) = pl.mt == 1 ? linear_skinny_kernel<T, 1, 1> : linear_skinny_kernel<T, 2, 2>;
    RG_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pl.smem)));
    unsigned grid = static_cast<unsigned>(sm_count());
    if (grid > pl.units) grid = pl.units;
    RG_CHECK_CUDA(launch_pdl(kern, dim3(grid), dim3(SK_THREADS), pl.smem, st, full, half, a));
    count_launch();
    return RG_OK;
}

// in = {X, W, C or NULL, positions or NULL, block_table or NULL}; out = {Y, k_cache or NULL, v_cache or NULL}
int linear_skinny(const SkinnyCall &c, void *ws, const void *const *in, void *const *out, cudaStream_t st) {
    SkinnyPlan pl;
    const int rc = skinny_plan(c.dtype, c.m, c.n, c.k, c.epilogue, &c.kv, c.n_heads, pl);
    if (rc != RG_OK) return rc;
    SkinnyArgs a = {};
    a.X = in[0], a.W = in[1], a.C = in[2];
    a.pos = static_cast<const int64_t *>(in[3]);
    a.table = static_cast<const int32_t *>(in[4]);
    a.Y = out[0], a.kc = out[1], a.vc = out[2];
    if (!a.X || !a.W || !a.Y) return RG_ERR_NULL;
    if (c.epilogue == 1 && !a.C) return RG_ERR_NULL;
    if (c.epilogue == 3 && (!a.pos || !a.kc || !a.vc)) return RG_ERR_NULL;
    if (c.epilogue == 3 && a.table && c.kv.page_size == 0) return RG_ERR_SHAPE;
    if (!aligned16(a.X) || !aligned16(a.W) || !aligned16(a.Y) || (a.kc && !aligned16(a.kc)) || (a.vc && !aligned16(a.vc))) return RG_ERR_ALIGN;
    if (pl.ksplit > 1 && !ws) return RG_ERR_NULL;
    a.cnt = static_cast<unsigned *>(ws);
    a.part = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + pl.cnt_bytes);
    a.m = c.m, a.n = c.n, a.k = c.k, a.epilogue = c.epilogue;
    a.alpha = c.alpha, a.beta = c.beta;
    a.c_row_stride = c.c_row_stride, a.c_col_stride = c.c_col_stride, a.y_row_stride = c.y_row_stride;
    a.n_heads = c.n_heads, a.log2_theta = c.epilogue == 3 ? log2f(c.theta) : 0.f;
    a.kv = c.kv, a.tokens_per_seq = c.tokens_per_seq;
    a.ksplit = pl.ksplit, a.kblocks = pl.kblocks, a.nrb = pl.nrb, a.units = pl.units;
    a.w_static = c.w_static;
    return c.dtype == RG_FP16 ? skinny_launch<__half>(a, pl, 0, st) : skinny_launch<__nv_bfloat16>(a, pl, 1, st);
}

}// namespace rg
