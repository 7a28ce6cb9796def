// Tensor-core GEMM for sm_100a:  Y[m,n] = alpha * A[m,k] * B[n,k]^T (+ beta * C),  fp16 / bf16 operands (both
// K-major: activations [tokens, k] and weights [out, in], the reference MatMul with transB = 1), fp32 accumulation
// in tensor memory.  Replaces the cublasGemmEx call of MatMulCublas
// (src/04kernel/src/kernels/mat_mul/cublas_kernel.cu:48-55) for prefill-sized products.
//
// Persistent CTAs (one per SM) walk 128 x BN output tiles (BN = 256 or 128; 64 / 32 with the operands swapped so that a
// skinny activation matrix becomes the N side of the instruction) in an L2-friendly grouped order:
//   warp 4  (one thread): TMA producer — cp.async.bulk.tensor.2d loads of the A tile [128 x 64] and B tile [BN x 64]
//                         with the 128-byte swizzle into a STAGES-deep shared-memory ring (full[] mbarriers).
//   warp 5  (one thread): MMA issuer — per stage four tcgen05.mma.cta_group::1.kind::f16 (M 128, N BN, K 16) whose
//                         shared-memory descriptors advance 32 bytes along K inside the swizzle atom; tcgen05.commit
//                         releases the stage (empty[]) and finally signals the accumulator (acc_full).
//   warps 0-3:            epilogue — tcgen05.ld of each warp's 32 TMEM lanes, alpha/beta/bias, conversion, stores.
// The accumulator is double-buffered in tensor memory (2 x BN columns, acc_full[] / acc_empty[] mbarriers), so a tile's
// epilogue overlaps the next tile's main loop.  Warp 5 also allocates and frees the TMEM columns.  Every mbarrier wait is bounded; on expiry the CTA records
// an error word, still frees its tensor memory and exits.
// Products of 512 rows and more run on CTA pairs (template flag PAIR, tcgen05 ... cta_group::2): see the comment above the kernel.
#include "gemm_dispatch.cuh"
#include "tcgen05.cuh"
#include "ar_slots.cuh"
#include <cstdlib>
#include <type_traits>
#include <cuda.h>

namespace rg {

static __device__ int s_tc_error;
static __device__ int s_tc_index_error;// a cache-append position or block-table entry was out of range (store skipped)

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;// 64 x 2 B = one 128-byte swizzle row
constexpr int TC_THREADS = 192;

struct TcArgs {
    void *Y;
    const void *C;
    uint32_t m, n, k;// problem as the kernel sees it: D[m,n] = A[m,k] B[n,k]^T
    float alpha, beta;
    uint32_t c_row_stride, c_col_stride;
    uint64_t y_row_stride, y_col_stride;// element strides of Y over the kernel's (row, col) = lets swapped runs write Y^T
    int is_bf16;
    uint32_t splits;   // partial slots per output tile: the k-splits (1 = none), or with streamk the most CTAs a tile can span
    uint32_t streamk;  // != 0: CTA c owns the contiguous run [U c / G, U (c+1) / G) of the U = tiles * kblocks (tile, k-block) units
    float *partial;    // [tiles][splits][128][BN] fp32, used when splits > 1
    unsigned *counter; // [tiles] arrival counters, zero before the first call and left at zero
    uint32_t group_m;  // row tiles per group of the tile order
    uint32_t early;    // operand that no earlier kernel of the stream writes (a weight): 1 = A, 2 = B, 0 = neither
    // QKV epilogue (rope != 0): columns are [q heads | k heads | v heads] of head_dim 128, rows are tokens; q is rotated into
    // q_out[token, nq * 128], k rotated and v copied into the caches at pos[token] of sequence token / tokens_per_seq
    uint32_t swiglu;   // != 0: B tile = 128 gate rows + the matching 128 up rows (swiglu rows further down B); Y[m, n / 2] = silu(g) * u
    uint32_t rope, nq, tokens_per_seq;
    float log2_theta;
    const int64_t *pos;
    const int32_t *table;
    void *q_out, *kc, *vc;
    rg_kv_layout kv;
    // push != 0 (weights on the M side only): the finished 16-bit values do not go to Y; paired with the flag of the all-reduce
    // call in flight they are stored into this rank's input slot in the allocation of every rank (1, one-shot) or of the rank
    // that owns the run of chunks (2, two-shot), over NVLink with ordinary 8-byte stores — the row-parallel product and the send
    // half of the all-reduce are one kernel
    uint32_t push;
    ArPeers ar;
};

// Row `feat` of the kernel's output (an output feature; a.m of them) for token `tok`: even lanes take the value of the next
// lane (feature feat + 1: both lie in one 16-byte chunk of the token's row) and store {two 16-bit values, flag}.  Called by all
// 32 lanes of a warp; `live` = this lane's row exists.
template<class T>
__device__ __forceinline__ void tc_push_value(const TcArgs &a, uint32_t flag, unsigned q, uint32_t feat, uint32_t tok, float v, bool live, uint32_t lane) {
    const float vn = __shfl_down_sync(0xffffffffu, v, 1);
    if ((lane & 1u) || !live) return;
    const T lo = Num<T>::from_f(v), hi = Num<T>::from_f(vn);
    const uint32_t data = static_cast<uint32_t>(*reinterpret_cast<const uint16_t *>(&lo)) | (static_cast<uint32_t>(*reinterpret_cast<const uint16_t *>(&hi)) << 16);
    const uint64_t e = static_cast<uint64_t>(tok) * a.m + feat, chunk = e >> 3;
    const size_t off = ar_slot_offset(a.ar.capacity, a.ar.world, q, a.ar.rank) + chunk * 32 + ((e & 7u) >> 1) * 8;
    if (a.push == 2) {
        const int owner = static_cast<int>((chunk / 32) % static_cast<uint64_t>(a.ar.world));
        asm volatile("st.global.cg.v2.u32 [%0], {%1, %2};" ::"l"(a.ar.peer[owner] + off), "r"(data), "r"(flag) : "memory");
    } else {
#pragma unroll
        for (int r = 0; r < AR_MAX_RANKS; ++r)
            if (r < a.ar.world) asm volatile("st.global.cg.v2.u32 [%0], {%1, %2};" ::"l"(a.ar.peer[r] + off), "r"(data), "r"(flag) : "memory");
    }
}

// Tile order: groups of TC_GROUP_M row tiles are walked column by column, so the CTAs running at the same time share
// a few A row-panels and B column-panels in L2 instead of streaming all of B once per row tile.
constexpr uint32_t TC_GROUP_M = 16;
__device__ __forceinline__ void tile_coords(uint32_t t, uint32_t m_tiles, uint32_t n_tiles, uint32_t &mt, uint32_t &nt, uint32_t group_m = TC_GROUP_M) {
    const uint32_t per_group = group_m * n_tiles;
    const uint32_t grp = t / per_group, first = grp * group_m;
    const uint32_t rows = m_tiles - first < group_m ? m_tiles - first : group_m;
    const uint32_t r = t - grp * per_group;
    mt = first + r % rows;
    nt = r / rows;
}

// One CTA's work, as (tile, k-block range) segments.  Split mode: items c, c + G, ... of tiles * splits, item = (tile, split).
// Stream-K mode: a contiguous run of (tile, k-block) units, so every CTA streams the same number of bytes whatever the tile
// count; a tile that spans several CTAs is summed by the last of them to arrive (ord = this CTA's place among them).
struct TcSeg {
    uint32_t tile, kb0, kb1, ord, ncontrib;
};
struct TcWalk {
    uint32_t streamk, splits, kblocks, items, item, G;
    uint64_t U, u, u1;
    // unit = what walks the tiles: a CTA, or a pair of CTAs (pair mode: unit index and count are halved)
    __device__ __forceinline__ void init(const TcArgs &a, uint32_t tiles, uint32_t kblocks_, uint32_t unit = blockIdx.x, uint32_t units = gridDim.x) {
        streamk = a.streamk, splits = a.splits, kblocks = kblocks_, G = units;
        items = tiles * a.splits, item = unit;
        U = static_cast<uint64_t>(tiles) * kblocks_;
        u = U * unit / G, u1 = U * (unit + 1) / G;
    }
    // CTA that owns unit x: the largest c with floor(U c / G) <= x
    __device__ __forceinline__ uint32_t owner(uint64_t x) const { return static_cast<uint32_t>(((x + 1) * G + U - 1) / U - 1); }
    __device__ __forceinline__ bool next(TcSeg &s) {
        if (!streamk) {
            if (item >= items) return false;
            const uint32_t ks = item % splits;
            s.tile = item / splits, s.kb0 = kblocks * ks / splits, s.kb1 = kblocks * (ks + 1) / splits;
            s.ord = ks, s.ncontrib = splits;
            item += G;
            return true;
        }
        if (u >= u1) return false;
        s.tile = static_cast<uint32_t>(u / kblocks), s.kb0 = static_cast<uint32_t>(u % kblocks);
        const uint64_t left = u1 - u;
        s.kb1 = left < kblocks - s.kb0 ? s.kb0 + static_cast<uint32_t>(left) : kblocks;
        u += s.kb1 - s.kb0;
        if (s.kb0 == 0 && s.kb1 == kblocks) {
            s.ord = 0, s.ncontrib = 1;
        } else {
            const uint64_t x0 = static_cast<uint64_t>(s.tile) * kblocks;
            const uint32_t cf = owner(x0), cl = owner(x0 + kblocks - 1);
            s.ord = blockIdx.x - cf, s.ncontrib = cl - cf + 1;
        }
        return true;
    }
};

// Persistent: CTA c computes tiles c, c + gridDim.x, ...  The accumulator is double-buffered in tensor memory (2 x BN
// columns), so the epilogue of one tile (tcgen05.ld, conversion, stores) overlaps the MMA main loop of the next.
// PAIR: two CTAs (a cluster of two on neighbouring SMs) compute one 256 x BN tile with tcgen05 ... cta_group::2: each CTA loads its
// 128 rows of A and HALF of the B tile, the even CTA issues the products for both, each CTA's tensor memory receives its 128 rows of
// the accumulator and its epilogue warps store them.  Per SM and k-block that is 32 KiB from L2 instead of 48 for the same 128 x 256
// outputs: the single-CTA kernel is bound by requests to L2 (ncu: 68 % of request cycles, tensor pipe 80 %; an extra L2 prefetch
// per box made it 22 % slower).  No load is multicast.
template<class T, int BN, int STAGES, bool PUSH = false, bool PAIR = false>// PUSH: the epilogue that stores into the all-reduce slots is compiled in
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                              const __grid_constant__ CUtensorMap tmap_b, const TcArgs a) {
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = (PAIR ? BN / 2 : BN) * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t ROWS = PAIR ? 2 * TC_BM : TC_BM;// rows of a tile
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;// 0 = the CTA that issues the products
    const uint32_t unit = PAIR ? blockIdx.x >> 1 : blockIdx.x, units = PAIR ? gridDim.x >> 1 : gridDim.x;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // the swizzled tiles need 1024-byte alignment
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);
    uint64_t *empty = full + STAGES;
    uint64_t *acc_full = empty + STAGES; // [2]
    uint64_t *acc_empty = acc_full + 2;  // [2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    int *failed = reinterpret_cast<int *>(tmem_slot + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m_tiles = (a.m + ROWS - 1) / ROWS, n_tiles = (a.n + BN - 1) / BN, tiles = m_tiles * n_tiles;
    const uint32_t kblocks = (a.k + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], PAIR ? 8 : 4);// one arrival per epilogue warp (pair mode: of both CTAs, on the even CTA's barrier)
        }
        *failed = 0;
        fence_mbar_init();
    }
    if (warp == 5) {
        if constexpr (PAIR) {
            tmem_alloc_pair(tmem_slot, 2 * BN);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, 2 * BN);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync();// the partner's barriers are initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: everything up to here, and the first stages of a weight operand, overlap the previous
    // kernel of the stream; each role waits for that kernel right before it first touches memory the kernel may write.
    pdl_launch_dependents();

    if (warp == 4) {
        if (lane == 0) {
            uint32_t it = 0, pre = 0;
            // B tile of column tile nt: BN consecutive rows of B, or (SiLU-gate form) 128 gate rows and their 128 up rows
            auto load_b = [&](uint8_t *dst, uint32_t kb, uint32_t nt, uint64_t *bar) {
                if (BN == 256 && a.swiglu) {
                    tma_load_2d(dst, &tmap_b, kb * TC_BK, nt * 128, bar);
                    tma_load_2d(dst + 128 * TC_BK * 2, &tmap_b, kb * TC_BK, a.swiglu + nt * 128, bar);
                } else {
                    tma_load_2d(dst, &tmap_b, kb * TC_BK, nt * BN, bar);
                }
            };
            // A tile of row tile mt: 128 consecutive rows of A, or (SiLU-gate form with the weights on the A side) 64 gate rows
            // and their 64 up rows: two boxes of a 64-row tensor map, one behind the other
            auto load_a = [&](uint8_t *dst, uint32_t kb, uint32_t mt, uint64_t *bar) {
                if (BN <= 64 && a.swiglu) {
                    tma_load_2d(dst, &tmap_a, kb * TC_BK, mt * 64, bar);
                    tma_load_2d(dst + 64 * TC_BK * 2, &tmap_a, kb * TC_BK, a.swiglu + mt * 64, bar);
                } else {
                    tma_load_2d(dst, &tmap_a, kb * TC_BK, mt * TC_BM, bar);
                }
            };
            TcWalk walk;
            walk.init(a, tiles, kblocks, unit, units);
            TcSeg sg;
            if (!PAIR && a.early) {
                // weight tiles of this CTA's first segment go in flight before the wait; their partner tiles follow after it
                TcWalk peek = walk;
                if (peek.next(sg)) {
                    uint32_t mt, nt;
                    tile_coords(sg.tile, m_tiles, n_tiles, mt, nt, a.group_m);
                    for (uint32_t kb = sg.kb0; kb < sg.kb1 && pre < STAGES; ++kb, ++pre) {
                        mbar_arrive_expect_tx(&full[pre], STAGE_BYTES);
                        uint8_t *st = smem + pre * STAGE_BYTES;
                        if (a.early == 1) load_a(st, kb, mt, &full[pre]);
                        else
                            load_b(st + A_BYTES, kb, nt, &full[pre]);
                    }
                }
            }
            pdl_wait();
            bool good = true;
            while (good && walk.next(sg)) {
                uint32_t mt, nt;
                tile_coords(sg.tile, m_tiles, n_tiles, mt, nt, a.group_m);
                for (uint32_t kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    uint8_t *st = smem + s * STAGE_BYTES;
                    if (it < pre) {// stage armed and half filled above
                        if (a.early == 1) load_b(st + A_BYTES, kb, nt, &full[s]);
                        else
                            load_a(st, kb, mt, &full[s]);
                        continue;
                    }
                    if (!mbar_wait(&empty[s], ph ^ 1u)) {
                        *failed = 1;
                        good = false;
                        break;
                    }
                    if constexpr (PAIR) {
                        // both CTAs' bytes are counted on the even CTA's barrier, which its producer arms for the two of them
                        const uint32_t bar = cluster_map(&full[s], 0);
                        if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * STAGE_BYTES);
                        tma_load_2d_pair(st, &tmap_a, kb * TC_BK, (mt * 2 + rank) * TC_BM, bar);
                        const uint32_t brow = a.swiglu ? (rank ? a.swiglu + nt * 128 : nt * 128) : nt * BN + rank * (BN / 2);
                        tma_load_2d_pair(st + A_BYTES, &tmap_b, kb * TC_BK, brow, bar);
                        continue;
                    }
                    mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
                    load_a(st, kb, mt, &full[s]);
                    load_b(st + A_BYTES, kb, nt, &full[s]);
                }
            }
        }
    } else if (warp == 5) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = instr_desc(a.is_bf16, ROWS, BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            TcWalk walk;
            walk.init(a, tiles, kblocks, unit, units);
            TcSeg sg;
            for (; ok && walk.next(sg); ++local) {
                const uint32_t buf = local & 1u, kb0 = sg.kb0, kb1 = sg.kb1;
                if (!mbar_wait(&acc_empty[buf], ((local >> 1) & 1u) ^ 1u)) {
                    *failed = 4;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    if (!mbar_wait(&full[s], ph)) {
                        *failed = 2;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; ++kk) {
                        const uint64_t ad = smem_desc_sw128(a_addr + kk * 32), bd = smem_desc_sw128(b_addr + kk * 32);
                        if constexpr (PAIR) tc_mma_f16_pair(d_tmem, ad, bd, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
                        else
                            tc_mma_f16(d_tmem, ad, bd, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
                    }
                    // frees the stage once these MMAs have read it (pair mode: in both CTAs)
                    if constexpr (PAIR) tc_commit_pair(&empty[s], 3);
                    else
                        tc_commit(&empty[s]);
                }
                // this tile's accumulator is complete when it arrives
                if constexpr (PAIR) tc_commit_pair(&acc_full[buf], 3);
                else
                    tc_commit(&acc_full[buf]);
            }
        }
    } else {
        // ---- epilogue warps 0..3: TMEM lanes [32*warp, 32*warp + 32) = tile rows ----
        pdl_wait();// C, Y and the split-K workspace may still be in use by the previous kernel
        T *Y = static_cast<T *>(a.Y);
        const T *C = static_cast<const T *>(a.C);
        const bool c_rowmajor = C && a.c_col_stride == 1 && (a.c_row_stride % 8) == 0;
        __shared__ int s_last;
        // the all-reduce call this product feeds: its number stays put until the receiving kernel behind this one has run
        uint32_t ar_flag_v = 0;
        unsigned ar_q = 0;
        if constexpr (PUSH) {
            const unsigned long long seq = *reinterpret_cast<const volatile unsigned long long *>(a.ar.mine);
            ar_flag_v = ar_flag(seq), ar_q = static_cast<unsigned>(seq & 1ull);
        }
        // SiLU gate with the weights on the A side: tile rows [0, 64) are gate rows, [64, 128) their up rows; the up half hands
        // its values to the gate half through this buffer
        constexpr int UPW = BN <= 64 ? BN : 1;
        __shared__ float s_up[BN <= 64 ? 64 : 1][UPW + 1];
        // v[0..W) = this thread's row, columns c_first ..; every one of the 128 epilogue threads calls it
        auto swiglu_rows = [&](const float *v, auto width, uint32_t mt, uint32_t c_first) {
            constexpr int W = decltype(width)::value;
            const uint32_t trow = warp * 32 + lane, f = a.swiglu;
            if (trow >= 64) {
#pragma unroll
                for (int j = 0; j < W; ++j) s_up[trow - 64][j] = v[j];
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (trow < 64) {
                const uint32_t feat = mt * 64 + trow;
#pragma unroll
                for (int j = 0; j < W; ++j) {
                    const uint32_t tok = c_first + j;
                    if (feat < f && tok < a.n) {
                        const float g = a.alpha * v[j], u = a.alpha * s_up[trow][j];
                        Y[static_cast<uint64_t>(tok) * f + feat] = Num<T>::from_f(g / (1.f + expf(-g)) * u);
                    }
                }
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
        };
        // QKV split + rotation + cache append with the weights on the A side: a tile of 128 rows is one head (head_dim 128), tile
        // rows i and i + 64 are a rotation pair.  The upper half hands its values to the lower half, which rotates the pair with
        // the token's angle and stores both results: into the q buffer, or into the K / V cache row of the token's position
        // (checked against the layout; a bad position or block id skips the store and raises the index error).
        auto rope_rows = [&](const float *v, auto width, uint32_t mt, uint32_t c_first) {
            constexpr int W = decltype(width)::value;
            const uint32_t trow = warp * 32 + lane, nkv = a.kv.n_kv_heads;
            if (trow >= 64) {
#pragma unroll
                for (int j = 0; j < W; ++j) s_up[trow - 64][j] = v[j];
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (trow < 64 && mt < a.nq + 2 * nkv) {
                const uint32_t gh = mt;
                const bool is_q = gh < a.nq, rotate = gh < a.nq + nkv;
                const uint32_t kvh = is_q ? 0u : (rotate ? gh - a.nq : gh - a.nq - nkv);
                const float inv_freq = exp2f(-a.log2_theta * (2.0f * static_cast<float>(trow) / 128.0f));
#pragma unroll 1
                for (int j = 0; j < W; ++j) {
                    const uint32_t tok = c_first + j;
                    if (tok >= a.n) break;
                    float lo = a.alpha * v[j], hi = a.alpha * s_up[trow][j];
                    const int64_t p = a.pos[tok];
                    if (rotate) {
                        float sn, cs;
                        sincosf(static_cast<float>(p) * inv_freq, &sn, &cs);
                        const float r0 = lo * cs - hi * sn, r1 = hi * cs + lo * sn;
                        lo = r0, hi = r1;
                    }
                    T *dst;
                    if (is_q) {
                        dst = static_cast<T *>(a.q_out) + (static_cast<uint64_t>(tok) * a.nq + gh) * 128u;
                    } else {
                        if (!kv_pos_ok(p, a.kv, a.table != nullptr)) {
                            s_tc_index_error = 1;
                            continue;
                        }
                        const uint32_t seq = a.tokens_per_seq > 1 ? tok / a.tokens_per_seq : tok;
                        uint64_t cache_row;
                        uint32_t head_pitch;
                        if (a.table) {
                            const uint32_t page = a.kv.page_size;
                            const int32_t blk = a.table[static_cast<uint64_t>(seq) * a.kv.max_blocks_per_seq + static_cast<uint32_t>(p) / page];
                            if (!kv_block_ok(blk, a.kv)) {
                                s_tc_index_error = 1;
                                continue;
                            }
                            cache_row = (static_cast<uint64_t>(blk) * nkv * page + static_cast<uint32_t>(p) % page) * 128u;
                            head_pitch = page * 128u;
                        } else {
                            cache_row = (static_cast<uint64_t>(seq) * nkv * a.kv.max_seq + static_cast<uint64_t>(p)) * 128u;
                            head_pitch = a.kv.max_seq * 128u;
                        }
                        dst = static_cast<T *>(rotate ? a.kc : a.vc) + cache_row + static_cast<uint64_t>(kvh) * head_pitch;
                    }
                    dst[trow] = Num<T>::from_f(lo);
                    dst[trow + 64] = Num<T>::from_f(hi);
                }
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
        };
        uint32_t local = 0;
        TcWalk walk;
        walk.init(a, tiles, kblocks, unit, units);
        TcSeg sg;
        // hands an accumulator buffer back to the thread that issues the products (pair mode: in the even CTA)
        auto release_acc = [&](uint32_t buf) {
            if constexpr (PAIR) mbar_arrive_cluster(cluster_map(&acc_empty[buf], 0));
            else
                mbar_arrive(&acc_empty[buf]);
        };
        for (; walk.next(sg); ++local) {
            uint32_t mt, nt;
            const uint32_t tile = sg.tile, ks = sg.ord;
            tile_coords(tile, m_tiles, n_tiles, mt, nt, a.group_m);
            const uint32_t buf = local & 1u, m0 = PAIR ? (mt * 2 + rank) * TC_BM : mt * TC_BM, n0 = nt * BN;
            if (!mbar_wait(&acc_full[buf], (local >> 1) & 1u)) {
                *failed = 3;
                break;
            }
            tc_fence_after();
            if (sg.ncontrib > 1) {
                // split-K: park this split's fp32 tile; the last split to arrive sums all of them in split order
                const uint32_t trow = warp * 32 + lane;
                float *mine = a.partial + (static_cast<size_t>(tile) * a.splits + ks) * (TC_BM * BN) + static_cast<size_t>(trow) * BN;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + buf * BN + ((warp * 32u) << 16) + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<uint4 *>(mine + c0 + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) release_acc(buf);
                // the barrier orders the 128 threads' stores before thread 0's release-increment (cumulative at gpu scope)
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (threadIdx.x == 0) {
                    unsigned old;
                    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(a.counter + tile) : "memory");
                    s_last = old == sg.ncontrib - 1 ? 1 : 0;
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (!s_last) continue;
                const uint32_t row = m0 + trow;
                const float *base = a.partial + static_cast<size_t>(tile) * a.splits * (TC_BM * BN) + static_cast<size_t>(trow) * BN;
                if constexpr (BN <= 64) {// split-K is only planned for the skinny (swapped) shapes
                    if (a.swiglu) {
                        float acc[BN];
#pragma unroll
                        for (int c = 0; c < BN; ++c) acc[c] = 0.f;
#pragma unroll 2
                        for (uint32_t sidx = 0; sidx < sg.ncontrib; ++sidx) {
                            const float4 *src = reinterpret_cast<const float4 *>(base + static_cast<size_t>(sidx) * (TC_BM * BN));
                            float4 v[BN / 4];
#pragma unroll
                            for (int c = 0; c < BN / 4; ++c) v[c] = __ldcg(src + c);
#pragma unroll
                            for (int c = 0; c < BN / 4; ++c) acc[4 * c] += v[c].x, acc[4 * c + 1] += v[c].y, acc[4 * c + 2] += v[c].z, acc[4 * c + 3] += v[c].w;
                        }
                        swiglu_rows(acc, std::integral_constant<int, BN>{}, mt, n0);
                    } else if (a.rope) {
                        float acc[BN];
#pragma unroll
                        for (int c = 0; c < BN; ++c) acc[c] = 0.f;
#pragma unroll 2
                        for (uint32_t sidx = 0; sidx < sg.ncontrib; ++sidx) {
                            const float4 *src = reinterpret_cast<const float4 *>(base + static_cast<size_t>(sidx) * (TC_BM * BN));
                            float4 v[BN / 4];
#pragma unroll
                            for (int c = 0; c < BN / 4; ++c) v[c] = __ldcg(src + c);
#pragma unroll
                            for (int c = 0; c < BN / 4; ++c) acc[4 * c] += v[c].x, acc[4 * c + 1] += v[c].y, acc[4 * c + 2] += v[c].z, acc[4 * c + 3] += v[c].w;
                        }
                        rope_rows(acc, std::integral_constant<int, BN>{}, mt, n0);
                    } else if (PUSH) {
                        float acc[BN];
#pragma unroll
                        for (int c = 0; c < BN; ++c) acc[c] = 0.f;
                        if (row < a.m) {
#pragma unroll 2
                            for (uint32_t sidx = 0; sidx < sg.ncontrib; ++sidx) {
                                const float4 *src = reinterpret_cast<const float4 *>(base + static_cast<size_t>(sidx) * (TC_BM * BN));
                                float4 v[BN / 4];
#pragma unroll
                                for (int c = 0; c < BN / 4; ++c) v[c] = __ldcg(src + c);
#pragma unroll
                                for (int c = 0; c < BN / 4; ++c) acc[4 * c] += v[c].x, acc[4 * c + 1] += v[c].y, acc[4 * c + 2] += v[c].z, acc[4 * c + 3] += v[c].w;
                            }
                        }
#pragma unroll
                        for (int c = 0; c < BN; ++c)
                            if (n0 + c < a.n) tc_push_value<T>(a, ar_flag_v, ar_q, row, n0 + c, a.alpha * acc[c], row < a.m, lane);
                    } else if (row < a.m) {
                        // this thread's row of every split: the BN/4 loads of one split are independent, so the sum
                        // costs one L2 round trip per split (fixed split order => deterministic)
                        float4 acc[BN / 4];
#pragma unroll
                        for (int c = 0; c < BN / 4; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
                        for (uint32_t sidx = 0; sidx < sg.ncontrib; ++sidx) {
                            const float4 *src = reinterpret_cast<const float4 *>(base + static_cast<size_t>(sidx) * (TC_BM * BN));
                            float4 v[BN / 4];
#pragma unroll
                            for (int c = 0; c < BN / 4; ++c) v[c] = __ldcg(src + c);
#pragma unroll
                            for (int c = 0; c < BN / 4; ++c) acc[c].x += v[c].x, acc[c].y += v[c].y, acc[c].z += v[c].z, acc[c].w += v[c].w;
                        }
#pragma unroll
                        for (int c = 0; c < BN / 4; ++c) {
                            const float vals[4] = {acc[c].x, acc[c].y, acc[c].z, acc[c].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint32_t col = n0 + c * 4 + j;
                                if (col < a.n) {
                                    float v = a.alpha * vals[j];
                                    if (C) v += a.beta * Num<T>::to_f(C[static_cast<uint64_t>(row) * a.c_row_stride + static_cast<uint64_t>(col) * a.c_col_stride]);
                                    Y[static_cast<uint64_t>(row) * a.y_row_stride + static_cast<uint64_t>(col) * a.y_col_stride] = Num<T>::from_f(v);
                                }
                            }
                        }
                    }
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (threadIdx.x == 0) a.counter[tile] = 0u;
                continue;
            }
            const uint32_t row = m0 + warp * 32 + lane;
            if constexpr (BN <= 64) {
                if constexpr (PUSH) {
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 32) {
                        uint32_t r[32];
                        tmem_ld_32x32(tmem_base + buf * BN + ((warp * 32u) << 16) + c0, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + c0 + j < a.n) tc_push_value<T>(a, ar_flag_v, ar_q, row, n0 + c0 + j, a.alpha * __uint_as_float(r[j]), row < a.m, lane);
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) release_acc(buf);
                    continue;
                }
                if (a.swiglu || a.rope) {
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 32) {
                        uint32_t r[32];
                        tmem_ld_32x32(tmem_base + buf * BN + ((warp * 32u) << 16) + c0, r);
                        tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                        if (a.swiglu) swiglu_rows(v, std::integral_constant<int, 32>{}, mt, n0 + c0);
                        else
                            rope_rows(v, std::integral_constant<int, 32>{}, mt, n0 + c0);
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) release_acc(buf);
                    continue;
                }
            }
            if constexpr (BN == 256) {
                if (a.swiglu) {
                    // accumulator columns [0, 128) = gate, [128, 256) = up of output columns n0/2 .. n0/2 + 127
                    const uint32_t j0 = (n0 / 256) * 128, f = a.n / 2;
#pragma unroll 1
                    for (int c0 = 0; c0 < 128; c0 += 32) {
                        uint32_t gt[32], up[32];
                        const uint32_t taddr = tmem_base + buf * BN + ((warp * 32u) << 16) + c0;
                        tmem_ld_32x32(taddr, gt);
                        tmem_ld_32x32(taddr + 128, up);
                        tmem_ld_wait();
                        if (row < a.m && j0 + c0 < f) {
                            T *dst = Y + static_cast<uint64_t>(row) * f + j0 + c0;
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                float o[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    const float g = a.alpha * __uint_as_float(gt[j + e]), u = a.alpha * __uint_as_float(up[j + e]);
                                    o[e] = g / (1.f + expf(-g)) * u;
                                }
                                Vec16<T> v;
                                v.pack(o);
                                v.store(dst + j);
                            }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) release_acc(buf);
                    continue;
                }
            }
            if constexpr (BN >= 128) {
                if (a.rope) {
                    // this thread's token: rotate the pairs (i, i + 64) of every q and k head of the tile, copy v heads, and
                    // write each head straight to its destination (q buffer or KV cache, contiguous or paged)
                    const bool live = row < a.m;
                    const int64_t p = live ? a.pos[row] : 0;
                    const uint32_t seq = a.tokens_per_seq > 1 ? row / a.tokens_per_seq : row, nkv = a.kv.n_kv_heads;
                    uint64_t cache_row = 0;// element offset of (seq, kv head 0, p) in a cache, without the head term
                    uint32_t head_pitch = 0;
                    bool cache_ok = live;// false: this token's k / v heads are not stored
                    if (live && !kv_pos_ok(p, a.kv, a.table != nullptr)) {
                        s_tc_index_error = 1;
                        cache_ok = false;
                    }
                    if (cache_ok) {
                        if (a.table) {
                            const uint32_t page = a.kv.page_size;
                            const int32_t blk = a.table[static_cast<uint64_t>(seq) * a.kv.max_blocks_per_seq + static_cast<uint32_t>(p) / page];
                            if (!kv_block_ok(blk, a.kv)) {
                                s_tc_index_error = 1;
                                cache_ok = false;
                            }
                            cache_row = (static_cast<uint64_t>(cache_ok ? blk : 0) * nkv * page + static_cast<uint32_t>(p) % page) * 128u;
                            head_pitch = page * 128u;
                        } else {
                            cache_row = (static_cast<uint64_t>(seq) * nkv * a.kv.max_seq + static_cast<uint64_t>(p)) * 128u;
                            head_pitch = a.kv.max_seq * 128u;
                        }
                    }
#pragma unroll 1
                    for (int pc = 0; pc < 2; ++pc) {
                        float cs[32], sn[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float inv_freq = exp2f(-a.log2_theta * (2.0f * static_cast<float>(pc * 32 + j) / 128.0f));
                            sincosf(static_cast<float>(p) * inv_freq, &sn[j], &cs[j]);
                        }
#pragma unroll 1
                        for (int hh = 0; hh < BN / 128; ++hh) {
                            const uint32_t col0 = n0 + hh * 128;
                            if (col0 >= a.n) break;
                            uint32_t lo[32], hi[32];
                            const uint32_t taddr = tmem_base + buf * BN + ((warp * 32u) << 16) + hh * 128 + pc * 32;
                            tmem_ld_32x32(taddr, lo);
                            tmem_ld_32x32(taddr + 64, hi);
                            tmem_ld_wait();
                            if (!live) continue;
                            const uint32_t gh = col0 / 128;
                            T *dst;
                            if (gh < a.nq) {
                                dst = static_cast<T *>(a.q_out) + (static_cast<uint64_t>(row) * a.nq + gh) * 128u;
                            } else {
                                if (!cache_ok) continue;
                                const bool is_k = gh < a.nq + nkv;
                                const uint32_t kvh = is_k ? gh - a.nq : gh - a.nq - nkv;
                                dst = static_cast<T *>(is_k ? a.kc : a.vc) + cache_row + static_cast<uint64_t>(kvh) * head_pitch;
                            }
                            const bool rotate = gh < a.nq + nkv;
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                float fl[8], fh[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    const float x0 = a.alpha * __uint_as_float(lo[j + e]), x1 = a.alpha * __uint_as_float(hi[j + e]);
                                    fl[e] = rotate ? x0 * cs[j + e] - x1 * sn[j + e] : x0;
                                    fh[e] = rotate ? x1 * cs[j + e] + x0 * sn[j + e] : x1;
                                }
                                Vec16<T> vl, vh;
                                vl.pack(fl), vh.pack(fh);
                                vl.store(dst + pc * 32 + j);
                                vh.store(dst + 64 + pc * 32 + j);
                            }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) release_acc(buf);
                    continue;
                }
            }
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + buf * BN + ((warp * 32u) << 16) + c0, r);
                tmem_ld_wait();
                if (row < a.m) {
                    if (a.y_col_stride == 1 && n0 + c0 + 32 <= a.n && (a.y_row_stride % 8) == 0 && (!C || c_rowmajor)) {
                        // contiguous 64-byte run of this thread's row: four 16-byte stores (and loads of C)
                        T *dst = Y + static_cast<uint64_t>(row) * a.y_row_stride + n0 + c0;
                        const T *csrc = C ? C + static_cast<uint64_t>(row) * a.c_row_stride + n0 + c0 : nullptr;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            float f[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) f[e] = a.alpha * __uint_as_float(r[j + e]);
                            if (csrc) {
                                Vec16<T> cv;
                                float cf[8];
                                cv.load(csrc + j);
                                cv.unpack(cf);
#pragma unroll
                                for (int e = 0; e < 8; ++e) f[e] += a.beta * cf[e];
                            }
                            Vec16<T> v;
                            v.pack(f);
                            v.store(dst + j);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t col = n0 + c0 + j;
                            if (col < a.n) {
                                float v = a.alpha * __uint_as_float(r[j]);
                                if (C) v += a.beta * Num<T>::to_f(C[static_cast<uint64_t>(row) * a.c_row_stride + static_cast<uint64_t>(col) * a.c_col_stride]);
                                Y[static_cast<uint64_t>(row) * a.y_row_stride + static_cast<uint64_t>(col) * a.y_col_stride] = Num<T>::from_f(v);
                            }
                        }
                    }
                }
            }
            // hand the accumulator buffer back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) release_acc(buf);
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync();// the partner has read its accumulators and received every arrival meant for it
    if (warp == 5) {
        tc_fence_after();
        if constexpr (PAIR) tmem_dealloc_pair(tmem_base, 2 * BN);
        else
            tmem_dealloc(tmem_base, 2 * BN);
    }
    if (threadIdx.x == 0 && *failed) atomicExch(&s_tc_error, *failed);
}

// ---- host -----------------------------------------------------------------------------------------------------
// rows x k matrix, K-major (row stride = ld elements); box = 64 (k) x box_rows, 128-byte swizzle
static bool make_map(CUtensorMap *map, const void *base, int is_bf16, uint64_t rows, uint64_t k, uint64_t ld, uint32_t box_rows) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {TC_BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims,
              strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A K-major matrix W[rows, k] seen as (64 columns, rows, k / 64 column blocks): one request then loads a box of box_rows rows
// x box_blocks column blocks, stored [block][row][128 bytes] with the 128-byte swizzle (the streaming skinny kernel's unit).
bool tma_encode_rows_by_blocks(void *map, const void *base, int is_bf16, uint64_t rows, uint64_t k, uint32_t box_rows, uint32_t box_blocks) {
    EncodeFn fn = encode_fn();
    if (!fn || k % 64 != 0) return false;
    const cuuint64_t dims[3] = {64, rows, k / 64};
    const cuuint64_t strides[2] = {k * 2, 128};
    const cuuint32_t box[3] = {64, box_rows, box_blocks};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(static_cast<CUtensorMap *>(map), is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
              const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool gemm_tc_supported(const rg_mat_mul_params *p, const void *const *in, void *const *out) {
    if (p->dtype != RG_FP16 && p->dtype != RG_BF16) return false;
    if (p->trans_a || !p->trans_b) return false;
    if (p->k % 8 != 0 || p->k < 64) return false;
    if (!aligned16(in[0]) || !aligned16(in[1]) || !aligned16(out[0])) return false;
    if (p->batch > 1 && ((p->stride_a % 8) || (p->stride_b % 8) || (p->stride_y % 8))) return false;
    // worth a tensor-core launch only when there is a tile's worth of work
    if (static_cast<uint64_t>(p->m) * p->n < 64ull * 64ull) return false;
    return encode_fn() != nullptr;
}

// k-splits for a skinny product.  Stamps inside the kernel (16 tokens, 8192 x 1024 ... 7168 x 8192 weights) show where the time
// goes: one CTA streams its operands at ~60 GB/s (its ring of stages in flight / the memory latency), and a split product pays
// ~3 us more (partial tile to L2, release/acquire counter, the last arriver's sum) plus ~0.5 us per split summed.  The split
// count minimises that estimate; products with more tiles than half the SMs only get a 2-way split when it repairs a mostly
// empty last wave (22016 x 4096 at m = 16: 52.6 us unsplit, 46.6 / 52.8 / 88.9 us with 2 / 3 / 6 splits).
static uint32_t tc_splits(uint32_t tiles, uint32_t kblocks) {
    const uint32_t sms = static_cast<uint32_t>(sm_count());
    const uint32_t cap = kblocks / 8 ? kblocks / 8 : 1;
    if (tiles * 2 > sms) {
        auto busy = [&](uint32_t items) { return static_cast<float>(items) / static_cast<float>((items + sms - 1) / sms * sms); };
        // 96 tiles (12288 x 4096 at 32 tokens) leave a third of the SMs idle and two splits fill one wave and a third of the
        // next; three fill two waves (batch-32 decode step 11.65 -> 11.55 ms)
        if (cap >= 3 && tiles < sms && busy(3 * tiles) > busy(tiles) + 0.25f && busy(3 * tiles) > busy(2 * tiles) + 0.15f) return 3;
        return (cap >= 2 && tiles < 2 * sms && busy(2 * tiles) > busy(tiles) + 0.15f) ? 2 : 1;
    }
    uint32_t smax = sms / tiles;
    if (smax > cap) smax = cap;
    if (smax > 16) smax = 16;
    const float tile_us = static_cast<float>(kblocks) * (TC_BM * TC_BK * 2) / 60000.f;// one CTA streaming a whole tile's k range
    uint32_t best = 1;
    float best_us = tile_us;
    for (uint32_t s = 2; s <= smax; ++s) {
        const float us = tile_us / static_cast<float>(s) + 3.0f + 0.5f * static_cast<float>(s);
        if (us < best_us) best_us = us, best = s;
    }
    return best;
}
struct TcPlan {
    bool swap;
    uint32_t bn, tiles, splits;
    uint32_t streamk_grid;// != 0: stream-K over this many CTAs; `splits` is then the partial slots per tile
    size_t counter_bytes, partial_bytes;
};
static TcPlan tc_plan(const rg_mat_mul_params *p) {
    TcPlan pl;
    pl.swap = p->m <= 64 && p->n >= 128;
    const uint32_t km = pl.swap ? p->n : p->m, kn = pl.swap ? p->m : p->n;
    pl.bn = pl.swap ? (p->m <= 32 ? 32 : 64) : (p->n >= 256 ? 256 : 128);
    pl.tiles = ((km + TC_BM - 1) / TC_BM) * ((kn + pl.bn - 1) / pl.bn);
    const uint32_t kblocks = (p->k + TC_BK - 1) / TC_BK;
    pl.splits = pl.swap ? tc_splits(pl.tiles, kblocks) : 1;
    pl.streamk_grid = 0;
    if (pl.swap) {// tuning knobs: RG_B200_TC_SPLITS=<n> forces the split count of skinny products, RG_B200_TC_STREAMK=0/1 the mode
        static const char *force = std::getenv("RG_B200_TC_SPLITS");
        static const char *sk = std::getenv("RG_B200_TC_STREAMK");
        const uint32_t sms = static_cast<uint32_t>(sm_count());
        const uint64_t units = static_cast<uint64_t>(pl.tiles) * kblocks;
        // stream-K when every SM gets a run of at least 64 k-blocks (1 MiB of weights): below that the partial-tile round
        // trips of up to two boundary tiles per CTA cost more than the imbalance they remove (measured at 16 / 32 tokens:
        // 22016 x 4096, 74 k-blocks per SM: 44.5 -> 41.6 us; 8192 x 3584, 24 per SM: 17.8 -> 20.0 us; 7168 x 8192, 48: equal)
        bool streamk = units / sms >= 64;
        if (sk && sk[0]) streamk = sk[0] != '0' && units >= sms;
        if (force && force[0]) {
            const uint32_t f = static_cast<uint32_t>(std::atoi(force));
            if (f >= 1) pl.splits = f > kblocks ? kblocks : f, streamk = false;
        }
        if (streamk) {
            const uint32_t per = static_cast<uint32_t>(units / sms);// the shortest run
            const uint32_t slots = (kblocks + per - 1) / per + 1;   // the most CTAs one tile can span
            if (slots <= 8) pl.streamk_grid = sms, pl.splits = slots;// deeper tiles keep the uniform split (cheaper sums)
        }
    }
    pl.counter_bytes = pl.splits > 1 ? (static_cast<size_t>(pl.tiles) * 4 + 255) / 256 * 256 : 0;
    pl.partial_bytes = pl.splits > 1 ? static_cast<size_t>(pl.tiles) * pl.splits * TC_BM * pl.bn * 4 : 0;
    return pl;
}
size_t gemm_tc_workspace(const rg_mat_mul_params *p) {
    const TcPlan pl = tc_plan(p);
    return pl.counter_bytes + pl.partial_bytes;
}

// Measured on one rank's share of a tensor-parallel-8 decode step (16 tokens, 80 layers, one GPU, no exchange; 9.55 ms):
// 5 stages for the up-to-32-token products, so that a CTA of the next kernel fits beside one of this kernel and fetches its
// first weight tiles early: 10.55 ms; 10 stages: 9.57 ms; asking L2 for 16 / 48 further weight tiles of the CTA's run before the
// dependency wait (cp.async.bulk.prefetch.tensor): 9.62 / 9.69 ms.  None is kept.
// Also measured and not kept, on the 32-token x 22016 x 4096 product (41.3 us = 4.4 TB/s; a TMA-only stream of the same tiles
// from 148 CTAs with 192 KiB in flight reaches 5.8 TB/s): 10 stages (42.1 us); the four k-steps of a k-block into four separate
// accumulators added in the epilogue, so that consecutive instructions do not depend on one another (41.0 us).  Cycle counters:
// the issuing thread spends ~340 cycles per k-block (4 instructions + commit) and waits for data 41 % of the time, the producer
// waits for a free stage 41 % of the time.  Leaving the activation-tile loads out altogether (timing only): 41.3 us.  What is
// left is the fill and drain of the memory pipeline around the dependency on the previous kernel (~10 us per launch): the
// TMA-only stream has no such dependency, so its launches overlap.
template<class T, int BN, int STAGES, bool PUSH = false>
static int tc_launch(const CUtensorMap &ma, const CUtensorMap &mb, const TcArgs &a_in, cudaStream_t st) {
    TcArgs a = a_in;
    a.group_m = TC_GROUP_M;
    constexpr size_t smem = STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
    auto kern = gemm_tc_kernel<T, BN, STAGES, PUSH>;
    RG_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    // the whole shared-memory carve-out, so that a CTA of the next kernel can sit beside one of this kernel when both fit
    RG_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, static_cast<int>(cudaSharedmemCarveoutMaxShared)));
    const uint32_t items = ((a.n + BN - 1) / BN) * ((a.m + TC_BM - 1) / TC_BM) * a.splits;
    const uint32_t sms = static_cast<uint32_t>(sm_count());
    const uint32_t grid = a.streamk ? a.streamk : (items < sms ? items : sms);
    RG_CHECK_CUDA(launch_pdl(kern, dim3(grid), dim3(TC_THREADS), smem, st, ma, mb, a));
    count_launch();
    return launch_status();
}

// Pair mode: clusters of two CTAs, one 256 x BN tile per pair (B's tensor map has boxes of BN / 2 rows).  RG_B200_GEMM_PAIR=0 keeps
// the single-CTA kernel.
static bool tc_pair_enabled() {
    static const bool on = !(std::getenv("RG_B200_GEMM_PAIR") && std::getenv("RG_B200_GEMM_PAIR")[0] == '0');
    return on;
}
template<class T>
static int tc_launch_pair(const CUtensorMap &ma, const CUtensorMap &mb, const TcArgs &a_in, cudaStream_t st) {
    constexpr int BN = 256, STAGES = 6;
    TcArgs a = a_in;
    a.group_m = TC_GROUP_M;// of 256-row tiles; measured on 8192 x 12288 x 4096: 4 / 8 / 16 / 32 row tiles per group 577 / 557 / 550 / 605 us
    constexpr size_t smem = STAGES * (TC_BM * TC_BK * 2 + (BN / 2) * TC_BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
    auto kern = gemm_tc_kernel<T, BN, STAGES, false, true>;
    RG_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    const uint32_t items = ((a.n + BN - 1) / BN) * ((a.m + 2 * TC_BM - 1) / (2 * TC_BM));
    // as many pairs as the device can hold at once (asked once per device; half the SM count where the question fails)
    static int resident[64] = {};
    int dev = 0;
    RG_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && resident[dev] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(sm_count()) & ~1u), cfg.blockDim = dim3(TC_THREADS), cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr, cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = sm_count() / 2;
        }
        resident[dev] = n;
    }
    const uint32_t pairs = static_cast<uint32_t>(dev >= 0 && dev < 64 ? resident[dev] : sm_count() / 2);
    const uint32_t grid = 2 * (items < pairs ? items : pairs);
    RG_CHECK_CUDA(launch_pdl_cluster(kern, dim3(grid), dim3(TC_THREADS), smem, st, 2u, ma, mb, a));
    count_launch();
    return launch_status();
}

int gemm_tc(const rg_mat_mul_params *p, void *ws, const void *const *in, void *const *out, cudaStream_t st) {
    const int is_bf16 = p->dtype == RG_BF16;
    const size_t es = 2;
    const TcPlan pl = tc_plan(p);
    if (pl.splits > 1 && !ws) return RG_ERR_NULL;
    for (uint32_t b = 0; b < p->batch; ++b) {
        const uint8_t *A = static_cast<const uint8_t *>(in[0]) + b * p->stride_a * es;
        const uint8_t *B = static_cast<const uint8_t *>(in[1]) + b * p->stride_b * es;
        uint8_t *Y = static_cast<uint8_t *>(out[0]) + b * p->stride_y * es;
        const uint8_t *C = p->has_bias ? static_cast<const uint8_t *>(in[2]) + b * p->stride_c * es : nullptr;
        TcArgs a = {};
        a.alpha = p->alpha, a.beta = p->beta, a.is_bf16 = is_bf16, a.k = p->k;
        a.splits = pl.splits, a.streamk = pl.streamk_grid;
        a.counter = static_cast<unsigned *>(ws);
        a.partial = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + pl.counter_bytes);
        CUtensorMap ma, mb;
        // a skinny activation matrix (m <= 64) goes on the N side of the instruction: D^T[n, m] = W[n,k] X[m,k]^T
        const bool swap = pl.swap;
        uint32_t bn;
        if (!swap) {
            bn = p->n >= 256 ? 256 : 128;
            a.m = p->m, a.n = p->n;
            a.early = (p->flags & RG_MM_B_STATIC) ? 2u : 0u;
            a.Y = Y, a.y_row_stride = p->n, a.y_col_stride = 1;
            a.C = C, a.c_row_stride = p->bias_row_stride, a.c_col_stride = p->bias_col_stride;
            if (bn == 256 && pl.splits == 1 && !pl.streamk_grid && p->m >= 512 && tc_pair_enabled()) {
                if (!make_map(&ma, A, is_bf16, p->m, p->k, p->k, TC_BM) || !make_map(&mb, B, is_bf16, p->n, p->k, p->k, 128)) return RG_ERR_CUDA;
                const int rc = is_bf16 ? tc_launch_pair<__nv_bfloat16>(ma, mb, a, st) : tc_launch_pair<__half>(ma, mb, a, st);
                if (rc != RG_OK) return rc;
                continue;
            }
            if (!make_map(&ma, A, is_bf16, p->m, p->k, p->k, TC_BM) || !make_map(&mb, B, is_bf16, p->n, p->k, p->k, bn)) return RG_ERR_CUDA;
        } else {
            bn = p->m <= 32 ? 32 : 64;
            a.m = p->n, a.n = p->m;
            a.early = (p->flags & RG_MM_B_STATIC) ? 1u : 0u;
            a.Y = Y, a.y_row_stride = 1, a.y_col_stride = p->n;
            a.C = C, a.c_row_stride = p->bias_col_stride, a.c_col_stride = p->bias_row_stride;
            if (!make_map(&ma, B, is_bf16, p->n, p->k, p->k, TC_BM) || !make_map(&mb, A, is_bf16, p->m, p->k, p->k, bn)) return RG_ERR_CUDA;
        }
        int rc;
#define RG_TC(T)                                                                        \
    (bn == 256 ? tc_launch<T, 256, 4>(ma, mb, a, st) : bn == 128 ? tc_launch<T, 128, 6>(ma, mb, a, st) \
     : bn == 64 ? tc_launch<T, 64, 8>(ma, mb, a, st) : tc_launch<T, 32, 8>(ma, mb, a, st))
        rc = is_bf16 ? RG_TC(__nv_bfloat16) : RG_TC(__half);
#undef RG_TC
        if (rc != RG_OK) return rc;
    }
    return RG_OK;
}

// Y = X W^T with the QKV split, rotation and cache append in the epilogue (rg_b200_linear, epilogue 3, more than 64 tokens).
int gemm_tc_qkv_rope(const rg_linear_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    if (p->dtype != RG_FP16 && p->dtype != RG_BF16) return RG_ERR_DTYPE;
    const uint32_t nq = p->n_heads, nkv = p->kv.n_kv_heads;
    if (p->kv.head_dim != 128 || nkv == 0 || nq == 0 || p->n != (nq + 2 * nkv) * 128u || p->m <= 64) return RG_ERR_SHAPE;
    if (p->prologue != 0 || p->k % 8 != 0 || p->k < 64 || !(p->theta > 0.f)) return RG_ERR_UNSUPPORTED;
    if (!in[0] || !in[1] || !in[4] || !out[0] || !out[1] || !out[2]) return RG_ERR_NULL;
    if (in[5] && p->kv.page_size == 0) return RG_ERR_SHAPE;
    if (!aligned16(in[0]) || !aligned16(in[1]) || !aligned16(out[0]) || !aligned16(out[1]) || !aligned16(out[2])) return RG_ERR_ALIGN;
    if (!encode_fn()) return RG_ERR_UNSUPPORTED;
    const int is_bf16 = p->dtype == RG_BF16;
    TcArgs a = {};
    a.alpha = 1.f, a.beta = 0.f, a.is_bf16 = is_bf16, a.k = p->k, a.m = p->m, a.n = p->n;
    a.splits = 1, a.early = 2;
    a.Y = out[0], a.y_row_stride = p->n, a.y_col_stride = 1;
    a.rope = 1, a.nq = nq, a.tokens_per_seq = p->tokens_per_seq, a.log2_theta = log2f(p->theta);
    a.pos = static_cast<const int64_t *>(in[4]), a.table = static_cast<const int32_t *>(in[5]);
    a.q_out = out[0], a.kc = out[1], a.vc = out[2], a.kv = p->kv;
    CUtensorMap ma, mb;
    const bool pair = p->m >= 512 && tc_pair_enabled();// a pair of CTAs per 256-token tile: each loads half of the B tile
    if (!make_map(&ma, in[0], is_bf16, p->m, p->k, p->k, TC_BM) || !make_map(&mb, in[1], is_bf16, p->n, p->k, p->k, pair ? 128 : 256)) return RG_ERR_CUDA;
    if (pair) return is_bf16 ? tc_launch_pair<__nv_bfloat16>(ma, mb, a, st) : tc_launch_pair<__half>(ma, mb, a, st);
    return is_bf16 ? tc_launch<__nv_bfloat16, 256, 4>(ma, mb, a, st) : tc_launch<__half, 256, 4>(ma, mb, a, st);
}

// Y[m, n/2] = silu(X Wg^T) * (X Wu^T), W = [gate rows ; up rows] (rg_b200_linear, epilogue 2, more than 64 tokens): one B tile
// pairs 128 gate rows with their 128 up rows, so both halves of an output column meet in one accumulator.
// Up to 64 tokens: the weights go on the instruction's M side (a tile = 64 gate rows + their 64 up rows), the tokens on its N
// side, with the k-split / stream-K plan of the plain skinny product; the up half of a tile hands its sums to the gate half.
static rg_mat_mul_params swiglu_small_as_mat_mul(const rg_linear_params *p) {
    rg_mat_mul_params mp = {};
    mp.dtype = p->dtype, mp.m = p->m, mp.n = p->n, mp.k = p->k, mp.batch = 1;
    mp.trans_b = 1, mp.alpha = 1.f, mp.flags = RG_MM_B_STATIC;
    return mp;
}
bool gemm_tc_swiglu_small_shape(const rg_linear_params *p) {
    return (p->dtype == RG_FP16 || p->dtype == RG_BF16) && p->epilogue == 2 && p->prologue == 0 && p->m > 4 && p->m <= 64 &&
           p->n % 128 == 0 && p->n >= 128 && p->k % 8 == 0 && p->k >= 64 && encode_fn() != nullptr;
}
size_t gemm_tc_swiglu_small_workspace(const rg_linear_params *p) {
    const rg_mat_mul_params mp = swiglu_small_as_mat_mul(p);
    return gemm_tc_workspace(&mp);
}
int gemm_tc_swiglu_small(const rg_linear_params *p, void *ws, const void *const *in, void *const *out, cudaStream_t st) {
    if (!gemm_tc_swiglu_small_shape(p)) return RG_ERR_SHAPE;
    if (!in[0] || !in[1] || !out[0]) return RG_ERR_NULL;
    if (!aligned16(in[0]) || !aligned16(in[1]) || !aligned16(out[0])) return RG_ERR_ALIGN;
    const rg_mat_mul_params mp = swiglu_small_as_mat_mul(p);
    const TcPlan pl = tc_plan(&mp);
    if (!pl.swap) return RG_ERR_SHAPE;
    if (pl.splits > 1 && !ws) return RG_ERR_NULL;
    const int is_bf16 = p->dtype == RG_BF16;
    TcArgs a = {};
    a.alpha = 1.f, a.beta = 0.f, a.is_bf16 = is_bf16, a.k = p->k;
    a.m = p->n, a.n = p->m;// kernel rows = weight rows (gate and up interleaved by tile), kernel columns = tokens
    a.splits = pl.splits, a.streamk = pl.streamk_grid;
    a.counter = static_cast<unsigned *>(ws);
    a.partial = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + pl.counter_bytes);
    a.early = 1, a.swiglu = p->n / 2;
    a.Y = out[0], a.y_row_stride = 1, a.y_col_stride = p->n / 2;
    CUtensorMap ma, mb;
    if (!make_map(&ma, in[1], is_bf16, p->n, p->k, p->k, 64) || !make_map(&mb, in[0], is_bf16, p->m, p->k, p->k, pl.bn)) return RG_ERR_CUDA;
    if (pl.bn == 32) return is_bf16 ? tc_launch<__nv_bfloat16, 32, 8>(ma, mb, a, st) : tc_launch<__half, 32, 8>(ma, mb, a, st);
    return is_bf16 ? tc_launch<__nv_bfloat16, 64, 8>(ma, mb, a, st) : tc_launch<__half, 64, 8>(ma, mb, a, st);
}

// Row-parallel product feeding an all-reduce: the plain skinny product (weights on the M side) whose epilogue stores into the
// communicator's slots.  m <= 64 tokens, n a multiple of 8, no C operand.
int gemm_tc_push(const rg_mat_mul_params *p, void *ws, const void *const *in, const ArPeers &peers, cudaStream_t st) {
    if (p->dtype != RG_FP16 && p->dtype != RG_BF16) return RG_ERR_UNSUPPORTED;
    if (p->trans_a || !p->trans_b || p->batch != 1 || p->has_bias || p->m == 0 || p->m > 64 || p->n < 128 || p->n % 8 != 0 || p->k % 8 != 0 || p->k < 64)
        return RG_ERR_UNSUPPORTED;
    if (!aligned16(in[0]) || !aligned16(in[1]) || !encode_fn()) return RG_ERR_UNSUPPORTED;
    const TcPlan pl = tc_plan(p);
    if (!pl.swap) return RG_ERR_UNSUPPORTED;
    if (pl.splits > 1 && !ws) return RG_ERR_NULL;
    const int is_bf16 = p->dtype == RG_BF16;
    TcArgs a = {};
    a.alpha = p->alpha, a.beta = 0.f, a.is_bf16 = is_bf16, a.k = p->k;
    a.m = p->n, a.n = p->m;// kernel rows = output features, kernel columns = tokens
    a.splits = pl.splits, a.streamk = pl.streamk_grid;
    a.counter = static_cast<unsigned *>(ws);
    a.partial = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + pl.counter_bytes);
    a.early = (p->flags & RG_MM_B_STATIC) ? 1u : 0u;
    a.push = peers.two_shot ? 2u : 1u, a.ar = peers;
    CUtensorMap ma, mb;
    if (!make_map(&ma, in[1], is_bf16, p->n, p->k, p->k, TC_BM) || !make_map(&mb, in[0], is_bf16, p->m, p->k, p->k, pl.bn)) return RG_ERR_CUDA;
    if (pl.bn == 32) return is_bf16 ? tc_launch<__nv_bfloat16, 32, 8, true>(ma, mb, a, st) : tc_launch<__half, 32, 8, true>(ma, mb, a, st);
    return is_bf16 ? tc_launch<__nv_bfloat16, 64, 8, true>(ma, mb, a, st) : tc_launch<__half, 64, 8, true>(ma, mb, a, st);
}

// The same for the QKV projection with its split / rotation / cache-append epilogue on 5..64 tokens (a 128-row tile = one head).
static rg_mat_mul_params qkv_small_as_mat_mul(const rg_linear_params *p) { return swiglu_small_as_mat_mul(p); }
bool gemm_tc_qkv_rope_small_shape(const rg_linear_params *p) {
    const uint32_t nq = p->n_heads, nkv = p->kv.n_kv_heads;
    return (p->dtype == RG_FP16 || p->dtype == RG_BF16) && p->epilogue == 3 && p->prologue == 0 && p->m > 4 && p->m <= 64 && p->kv.head_dim == 128 &&
           nq > 0 && nkv > 0 && p->n == (nq + 2 * nkv) * 128u && p->k % 8 == 0 && p->k >= 64 && p->theta > 0.f && encode_fn() != nullptr;
}
size_t gemm_tc_qkv_rope_small_workspace(const rg_linear_params *p) {
    const rg_mat_mul_params mp = qkv_small_as_mat_mul(p);
    return gemm_tc_workspace(&mp);
}
int gemm_tc_qkv_rope_small(const rg_linear_params *p, void *ws, const void *const *in, void *const *out, cudaStream_t st) {
    if (!gemm_tc_qkv_rope_small_shape(p)) return RG_ERR_SHAPE;
    if (!in[0] || !in[1] || !in[4] || !out[0] || !out[1] || !out[2]) return RG_ERR_NULL;
    if (in[5] && p->kv.page_size == 0) return RG_ERR_SHAPE;
    if (!aligned16(in[0]) || !aligned16(in[1])) return RG_ERR_ALIGN;
    const rg_mat_mul_params mp = qkv_small_as_mat_mul(p);
    const TcPlan pl = tc_plan(&mp);
    if (!pl.swap) return RG_ERR_SHAPE;
    if (pl.splits > 1 && !ws) return RG_ERR_NULL;
    const int is_bf16 = p->dtype == RG_BF16;
    TcArgs a = {};
    a.alpha = 1.f, a.beta = 0.f, a.is_bf16 = is_bf16, a.k = p->k;
    a.m = p->n, a.n = p->m;// kernel rows = output features (a tile = a head), kernel columns = tokens
    a.splits = pl.splits, a.streamk = pl.streamk_grid;
    a.counter = static_cast<unsigned *>(ws);
    a.partial = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + pl.counter_bytes);
    a.early = 1;
    a.rope = 1, a.nq = p->n_heads, a.tokens_per_seq = p->tokens_per_seq, a.log2_theta = log2f(p->theta);
    a.pos = static_cast<const int64_t *>(in[4]), a.table = static_cast<const int32_t *>(in[5]);
    a.q_out = out[0], a.kc = out[1], a.vc = out[2], a.kv = p->kv;
    CUtensorMap ma, mb;
    if (!make_map(&ma, in[1], is_bf16, p->n, p->k, p->k, TC_BM) || !make_map(&mb, in[0], is_bf16, p->m, p->k, p->k, pl.bn)) return RG_ERR_CUDA;
    if (pl.bn == 32) return is_bf16 ? tc_launch<__nv_bfloat16, 32, 8>(ma, mb, a, st) : tc_launch<__half, 32, 8>(ma, mb, a, st);
    return is_bf16 ? tc_launch<__nv_bfloat16, 64, 8>(ma, mb, a, st) : tc_launch<__half, 64, 8>(ma, mb, a, st);
}

int gemm_tc_swiglu(const rg_linear_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    if (p->dtype != RG_FP16 && p->dtype != RG_BF16) return RG_ERR_DTYPE;
    const uint32_t f = p->n / 2;
    if (p->m <= 64 || p->n % 2 != 0 || f % 128 != 0) return RG_ERR_SHAPE;
    if (p->prologue != 0 || p->k % 8 != 0 || p->k < 64) return RG_ERR_UNSUPPORTED;
    if (!in[0] || !in[1] || !out[0]) return RG_ERR_NULL;
    if (!aligned16(in[0]) || !aligned16(in[1]) || !aligned16(out[0])) return RG_ERR_ALIGN;
    if (!encode_fn()) return RG_ERR_UNSUPPORTED;
    const int is_bf16 = p->dtype == RG_BF16;
    TcArgs a = {};
    a.alpha = 1.f, a.beta = 0.f, a.is_bf16 = is_bf16, a.k = p->k, a.m = p->m, a.n = p->n;
    a.splits = 1, a.early = 2, a.swiglu = f;
    a.Y = out[0], a.y_row_stride = f, a.y_col_stride = 1;
    CUtensorMap ma, mb;
    if (!make_map(&ma, in[0], is_bf16, p->m, p->k, p->k, TC_BM) || !make_map(&mb, in[1], is_bf16, p->n, p->k, p->k, 128)) return RG_ERR_CUDA;
    // pair mode: the even CTA of a pair loads the tile's gate rows, the odd one its up rows
    if (p->m >= 512 && tc_pair_enabled()) return is_bf16 ? tc_launch_pair<__nv_bfloat16>(ma, mb, a, st) : tc_launch_pair<__half>(ma, mb, a, st);
    return is_bf16 ? tc_launch<__nv_bfloat16, 256, 4>(ma, mb, a, st) : tc_launch<__half, 256, 4>(ma, mb, a, st);
}

int gemm_tc_error_word(bool clear) { return error_symbol(s_tc_error, clear); }
int gemm_tc_index_error_word(bool clear) { return error_symbol(s_tc_index_error, clear); }

}// namespace rg
