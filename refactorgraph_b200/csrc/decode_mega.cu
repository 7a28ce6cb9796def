// One decode step of a Llama-style decoder (batch 1) as ONE persistent cooperative kernel.
//
// Why: at batch 1 a step is ~13 GB of weights streamed through ~165 small kernels; every kernel boundary drains
// the memory pipeline (tail, launch, prologue) although the NEXT kernel's weights never depend on the previous
// one.  Here one CTA per SM runs the whole step:
//   * warp 8 (one thread) is a producer that walks the step's entire schedule — for every layer the QKV, KV-cache,
//     O, gate/up and down phases, then the LM head — and streams each CTA's share of the weights (and of the old
//     KV tiles) into a 6 x 32 KiB shared-memory ring with cp.async.bulk + mbarriers.  It is throttled only by ring
//     space, never by a phase boundary, so HBM stays busy while the consumers synchronise.
//   * warps 0-7 consume: per phase they (re)load the activation vector into registers (RMSNorm, or the merge of the
//     attention partials), reduce their units, run the phase epilogue (RoPE + cache append, residual add, SiLU*up,
//     logits + running arg-max) and meet the other CTAs at a grid barrier (monotonic counter, bounded spin).
//   * attention over the cached tokens [0, pos) is split over (head, 64-token tile) units; the token produced in
//     this step is folded in when the partial records are merged, so its K/V rows never have to be prefetched.
// Measured and not kept: replacing three of a layer's five grid barriers (after O, gate/up and down) by readiness carried
// in the data — every element of h, u and x a 32-bit word {value, 16-bit tag}, the next phase's consumers polling the words
// they need (with a 150 ns back-off) instead of barrier + load.  Correct (all parity tests green), but 3.08-3.09 ms per step
// against 3.01: the per-phase stamps show the wait moves from the barrier into the activation load (what a barrier costs is
// mostly the arrival skew of the CTAs, which a poll has to sit out just the same), the two remaining barriers absorb the
// accumulated skew, and 38 000 polling threads slow the attention and down phases' streams.
// Semantics equal the multi-kernel graph: Gather, [Linear(norm,QKV,RoPE,append), AttentionDecode, Linear(O,+res),
// Linear(norm,gate/up,SiLU), Linear(down,+res)] x L, Linear(norm, LM head), TopK(k=1, softmax), state updates.
#include "gemm_dispatch.cuh"
#include <algorithm>

namespace rg {

constexpr int MG_NW = 8;
constexpr int MG_CONSUMERS = MG_NW * 32;
constexpr int MG_THREADS = MG_CONSUMERS + 32;
constexpr int MG_STAGES = 6;   // 192 KiB of weights in flight per SM: enough to ride through a grid barrier
constexpr uint32_t MG_STAGE_BYTES = 32768;
constexpr int MG_KCH = 6;          // k <= 6 * 256 * 8 = 12288
constexpr int MG_MAX_LAYERS = 96;
constexpr int MG_TILE = 64;        // tokens per attention unit
constexpr int MG_PART_UNITS = 128; // max units of one phase per CTA (checked on the host for every phase of the shape)
constexpr int MG_MAX_REC = 8;
// Measured and removed: asking L2 to fetch further ahead than the ring (cp.async.bulk.prefetch.L2 by the producer, 8 or 14
// units ahead: step +45 %; prefetch.global.L2 by a consumer warp while a grid barrier completes, 2..16 units: +6..50 %).
// Every extra request in flight queues in front of the barrier's atomics and polls and lengthens the barrier.  Limiting the
// producer to 2..4 copies in flight instead of 6 changed neither the barrier time nor the step time.  P.V with the mixed-precision
// FMA (fma.rn.f32.f16 on the raw cache values, no conversions) left the attention loop at 6.4 us per layer.

static __device__ int s_mega_error;
static __device__ int s_mega_index_error;// the step's position or token id did not fit the cache / vocabulary: the step did nothing

struct MegaLayer {
    const void *norm1, *wqkv, *wo, *norm2, *wgu, *wd;
    void *kc, *vc;
};
struct MegaArgs {
    MegaLayer layer[MG_MAX_LAYERS];
    const void *embed, *norm_f, *lm_head;
    int64_t *token, *pos;
    int64_t *next;
    float *prob;
    void *logits;
    uint8_t *ws;
    uint32_t layers, H, nH, nKV, D, F, V, max_seq;
    float eps, log2_theta, scale;
};
struct MegaHeader {
    unsigned long long bar;  // monotonic arrival counter
    unsigned long long epoch;// value of bar at the start of the launch in flight
    unsigned long long best; // arg-max composite (key << 32 | ~index)
    int abort;
};
// workspace layout (bytes): header 256 | lse[G] float2 | x[H] | h[H] | q[nH*D] | u[F] (16-bit) | rec[G][MG_MAX_REC][D+2] float
struct MegaWs {
    MegaHeader *hdr;
    float2 *lse;
    void *x, *h, *q, *u;
    float *rec;
    unsigned long long *timeline;// [phases + 1][4] %globaltimer of CTA 0: phase entered, activations ready, units consumed, epilogue done
};
__host__ __device__ inline size_t mg_align(size_t v) { return (v + 255) / 256 * 256; }
__host__ __device__ inline size_t mega_ws_bytes(uint32_t G, uint32_t H, uint32_t nH, uint32_t D, uint32_t F) {
    return 256 + mg_align(G * 8) + 2 * mg_align(H * 2) + mg_align(static_cast<size_t>(nH) * D * 2) + mg_align(F * 2) +
           mg_align(static_cast<size_t>(G) * MG_MAX_REC * (D + 2) * 4) + mg_align((MG_MAX_LAYERS * 5 + 2) * 4 * 8);
}
__device__ inline MegaWs mega_ws(uint8_t *p, uint32_t G, uint32_t H, uint32_t nH, uint32_t D, uint32_t F) {
    MegaWs w;
    w.hdr = reinterpret_cast<MegaHeader *>(p);
    p += 256;
    w.lse = reinterpret_cast<float2 *>(p);
    p += mg_align(G * 8);
    w.x = p;
    p += mg_align(H * 2);
    w.h = p;
    p += mg_align(H * 2);
    w.q = p;
    p += mg_align(static_cast<size_t>(nH) * D * 2);
    w.u = p;
    p += mg_align(F * 2);
    w.rec = reinterpret_cast<float *>(p);
    p += mg_align(static_cast<size_t>(G) * MG_MAX_REC * (D + 2) * 4);
    w.timeline = reinterpret_cast<unsigned long long *>(p);
    return w;
}

enum : int { PH_QKV = 0, PH_ATT = 1, PH_O = 2, PH_GU = 3, PH_DOWN = 4, PH_LM = 5 };

struct Phase {
    int type;
    const uint8_t *W;  // weights (linear phases)
    uint32_t n, k;     // rows, columns of W
    uint32_t g, segs;  // rows per segment, segments per unit
    uint32_t units;
    uint32_t layer;
};

__host__ __device__ inline uint32_t pow2_floor_d(uint32_t v) {
    uint32_t p = 0;
    for (uint32_t b = 1; b && b <= v; b <<= 1) p = b;
    return p;
}
// Rows per segment (g) and units of a linear phase with `n` rows of `k` columns; one definition for the kernel's schedule and
// for the host-side check that no CTA gets more units of a phase than its shared-memory partial-sum table holds.
__host__ __device__ inline uint32_t mega_phase_units(int type, uint32_t n, uint32_t k, uint32_t segs, uint32_t D, uint32_t F, uint32_t &g_out) {
    uint32_t g = pow2_floor_d(MG_STAGE_BYTES / (k * 2u * segs));
    if (g * segs > 4) g = 4 / segs;
    uint32_t units;
    if (type == 0 /* PH_QKV */) {
        while (g > 1 && (D / 2) % g != 0) g >>= 1;
        units = n / (2 * g);
    } else if (type == 3 /* PH_GU */) {
        units = (F + g - 1) / g;
    } else {
        units = (n + g - 1) / g;
    }
    g_out = g;
    return units;
}
// Phase p of the step: 5 per layer, then the LM head.  `T` = attention tiles over the cached tokens [0, pos).
__device__ inline Phase phase_of(const MegaArgs &a, uint32_t p, uint32_t T) {
    Phase ph;
    ph.layer = p / 5;
    ph.type = ph.layer < a.layers ? static_cast<int>(p % 5) : PH_LM;
    ph.W = nullptr;
    ph.n = ph.k = ph.g = ph.segs = ph.units = 0;
    if (ph.type == PH_ATT) return ph;// attention units are assigned by att_range, not by unit_range
    const MegaLayer &L = a.layer[ph.layer < a.layers ? ph.layer : 0];
    switch (ph.type) {
        case PH_QKV: ph.W = static_cast<const uint8_t *>(L.wqkv), ph.n = (a.nH + 2 * a.nKV) * a.D, ph.k = a.H, ph.segs = 2; break;
        case PH_O: ph.W = static_cast<const uint8_t *>(L.wo), ph.n = a.H, ph.k = a.nH * a.D, ph.segs = 1; break;
        case PH_GU: ph.W = static_cast<const uint8_t *>(L.wgu), ph.n = 2 * a.F, ph.k = a.H, ph.segs = 2; break;
        case PH_DOWN: ph.W = static_cast<const uint8_t *>(L.wd), ph.n = a.H, ph.k = a.F, ph.segs = 1; break;
        default: ph.W = static_cast<const uint8_t *>(a.lm_head), ph.n = a.V, ph.k = a.H, ph.segs = 1; break;
    }
    ph.units = mega_phase_units(ph.type, ph.n, ph.k, ph.segs, a.D, a.F, ph.g);
    return ph;
}
// first row of segment s of unit u and how many of its g rows exist
__device__ __forceinline__ uint32_t mega_unit_row(const MegaArgs &a, const Phase &ph, uint32_t u, uint32_t s, uint32_t &rows) {
    if (ph.type == PH_QKV) {
        const uint32_t half = a.D / 2, per_head = half / ph.g;
        rows = ph.g;
        return (u / per_head) * a.D + s * half + (u % per_head) * ph.g;
    }
    const uint32_t span = ph.type == PH_GU ? a.F : ph.n;
    const uint32_t r0 = u * ph.g;
    rows = span - r0 < ph.g ? span - r0 : ph.g;
    return s * span + r0;
}
__device__ __forceinline__ void unit_range(uint32_t units, uint32_t &u0, uint32_t &u1) {
    u0 = static_cast<uint32_t>(static_cast<uint64_t>(units) * blockIdx.x / gridDim.x);
    u1 = static_cast<uint32_t>(static_cast<uint64_t>(units) * (blockIdx.x + 1) / gridDim.x);
}
// Attention work split: SPLITS = G / nH CTAs per head (the remaining CTAs idle in this phase); CTA c handles head
// c / SPLITS and the tiles [NT*j/SPLITS, NT*(j+1)/SPLITS) with j = c % SPLITS.  One partial record per CTA.
__host__ __device__ inline uint32_t att_splits(uint32_t G, uint32_t nH) {
    const uint32_t s = G / nH;
    return s > 8 ? 8 : s;
}
__device__ __forceinline__ bool att_range(const MegaArgs &a, uint32_t NT, uint32_t cta, uint32_t G, uint32_t &head, uint32_t &t0, uint32_t &t1) {
    const uint32_t splits = att_splits(G, a.nH);
    head = cta / splits;
    if (head >= a.nH) return false;
    const uint32_t j = cta % splits;
    t0 = NT * j / splits, t1 = NT * (j + 1) / splits;
    return t1 > t0;
}
// Position in a CTA's share of the step's schedule: phase p, unit u of [.., u1) (attention: tiles of `head`).
struct MegaCursor {
    uint32_t p, u, u1, head;
    Phase ph;
    bool done;
};
// Moves to the first phase >= c.p in which this CTA has units.
__device__ inline void mega_cursor_seek(const MegaArgs &a, MegaCursor &c, uint32_t nphases, uint32_t NT) {
    for (; c.p < nphases; ++c.p) {
        c.ph = phase_of(a, c.p, NT);
        uint32_t u0;
        c.head = 0;
        if (c.ph.type == PH_ATT) {
            if (!att_range(a, NT, blockIdx.x, gridDim.x, c.head, u0, c.u1)) u0 = c.u1 = 0;
        } else {
            unit_range(c.ph.units, u0, c.u1);
        }
        c.u = u0;
        if (c.u < c.u1) return;
    }
    c.done = true;
}
__device__ __forceinline__ void mega_cursor_advance(const MegaArgs &a, MegaCursor &c, uint32_t nphases, uint32_t NT) {
    if (++c.u >= c.u1) {
        ++c.p;
        mega_cursor_seek(a, c, nphases, NT);
    }
}
// The (up to two) contiguous pieces of the cursor's unit: returns the piece count, fills source, bytes and ring offset.
__device__ __forceinline__ uint32_t mega_pieces(const MegaArgs &a, const MegaCursor &c, uint32_t pos, const uint8_t *(&src)[2],
                                               uint32_t (&bytes)[2], uint32_t (&dst)[2]) {
    if (c.ph.type == PH_ATT) {
        const uint32_t kvh = c.head / (a.nH / a.nKV);
        const uint32_t tok0 = c.u * MG_TILE, ntok = pos - tok0 < MG_TILE ? pos - tok0 : MG_TILE;
        const size_t off = (static_cast<size_t>(kvh) * a.max_seq + tok0) * a.D * 2u;
        src[0] = static_cast<const uint8_t *>(a.layer[c.ph.layer].kc) + off;
        src[1] = static_cast<const uint8_t *>(a.layer[c.ph.layer].vc) + off;
        bytes[0] = bytes[1] = ntok * a.D * 2u;
        dst[0] = 0, dst[1] = MG_STAGE_BYTES / 2;
        return 2;
    }
    const uint32_t row_bytes = c.ph.k * 2u;
    for (uint32_t sg = 0; sg < c.ph.segs; ++sg) {
        uint32_t rows;
        const uint32_t row = mega_unit_row(a, c.ph, c.u, sg, rows);
        src[sg] = c.ph.W + static_cast<uint64_t>(row) * row_bytes;
        bytes[sg] = rows * row_bytes;
        dst[sg] = sg * c.ph.g * row_bytes;
    }
    return c.ph.segs;
}
__device__ __forceinline__ void mg_consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(MG_CONSUMERS) : "memory"); }

__device__ __forceinline__ unsigned long long ld_acquire_gpu(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_volatile_int(const int *p) { return *reinterpret_cast<const volatile int *>(p); }

template<int V> __device__ __forceinline__ void mg_reduce_halving(float (&vals)[V], int lane) {
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

// Consumes `nu` units of a linear phase from the ring: R rows per unit, KC live 16-byte chunks per thread along k.
// part[(i*4 + row) * MG_NW + warp] receives each warp's partial row sums of local unit i.
template<class T, int R, int KC>
__device__ __forceinline__ bool mega_linear_units(const uint8_t *smem, uint64_t *full, uint64_t *empty, float *part,
                                                  const float (&x)[MG_KCH][8], uint32_t nu, uint32_t &it, uint32_t k,
                                                  uint32_t tid, uint32_t warp, uint32_t lane) {
    const uint32_t kchunks = k / 8, row_bytes = k * 2u;
    for (uint32_t i = 0; i < nu; ++i, ++it) {
        const uint32_t s = it % MG_STAGES, par = (it / MG_STAGES) & 1u;
        if (!mbar_wait(&full[s], par)) return false;
        const uint8_t *st = smem + s * MG_STAGE_BYTES;
        uint4 raw[R][KC];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                const uint32_t ci = tid + c * MG_CONSUMERS;
                raw[r][c] = ci < kchunks ? *reinterpret_cast<const uint4 *>(st + static_cast<size_t>(r) * row_bytes + ci * 16) : make_uint4(0, 0, 0, 0);
            }
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                float w[8];
                unpack8<T>(raw[r][c], w);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[r] = fmaf(w[j], x[c][j], acc[r]);
            }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        mg_reduce_halving<4>(acc, static_cast<int>(lane));
        if ((lane & 7u) == 0) part[(i * 4 + (lane >> 3)) * MG_NW + warp] = acc[0];
    }
    return true;
}

template<class T>
__global__ void __launch_bounds__(MG_THREADS, 1) decode_mega_kernel(const __grid_constant__ MegaArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + MG_STAGES * MG_STAGE_BYTES);
    uint64_t *empty = full + MG_STAGES;
    float *red = reinterpret_cast<float *>(empty + MG_STAGES);// 32 floats
    float *qs = red + 32;                                      // [D] query of the current head (fp32)
    float *sc = qs + 256;                                      // [64] scores / probabilities, then [nH] new-token scores
    float *part = sc + 128;                                    // [MG_PART_UNITS * 4][MG_NW]; reused as [16][D] in attention
    int *s_fail = reinterpret_cast<int *>(part + MG_PART_UNITS * 4 * MG_NW);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, G = gridDim.x;
    const MegaWs ws = mega_ws(a.ws, G, a.H, a.nH, a.D, a.F);
    MegaHeader *hdr = ws.hdr;
    const int64_t pos64 = *a.pos, token = *a.token;
    // Both are device state a generation loop advances by itself.  Every CTA reads the same two words before any CTA can
    // reach the end of the step (where they are rewritten), so the decision is uniform: a step whose new token would not
    // fit the cache, or whose token id is outside the vocabulary, touches nothing and returns before the first barrier.
    if (pos64 < 0 || pos64 >= static_cast<int64_t>(a.max_seq) || token < 0 || token >= static_cast<int64_t>(a.V)) {
        if (blockIdx.x == 0 && threadIdx.x == 0) s_mega_index_error = 1;
        return;
    }
    const uint32_t pos = static_cast<uint32_t>(pos64);            // tokens already cached; the new token sits at pos
    const uint32_t NT = (pos + MG_TILE - 1) / MG_TILE;              // attention tiles over [0, pos)
    const uint32_t nphases = a.layers * 5 + 1;
    const unsigned long long epoch = *reinterpret_cast<volatile unsigned long long *>(&hdr->epoch);

    if (tid == 0) {
        for (int s = 0; s < MG_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], MG_NW);
        }
        *s_fail = 0;
        fence_mbar_init();
    }
    __syncthreads();

    if (warp == MG_NW) {
        // ================= producer: the whole step's stream for this CTA =================
        if (lane == 0) {
            const uint64_t policy = l2_policy_evict_first();
            MegaCursor ld{0, 0, 0, 0, {}, false};
            mega_cursor_seek(a, ld, nphases, NT);
            for (uint32_t it = 0; !ld.done; ++it) {
                const uint32_t s = it % MG_STAGES, par = (it / MG_STAGES) & 1u;
                if (!mbar_wait(&empty[s], par ^ 1u)) {
                    atomicExch(&hdr->abort, 1);
                    break;
                }
                uint8_t *st = smem + s * MG_STAGE_BYTES;
                const uint8_t *src[2];
                uint32_t bytes[2], dst[2];
                const uint32_t n = mega_pieces(a, ld, pos, src, bytes, dst);
                mbar_arrive_expect_tx(&full[s], n == 2 ? bytes[0] + bytes[1] : bytes[0]);
                for (uint32_t i = 0; i < n; ++i) {
                    if (ld.ph.type == PH_ATT) bulk_g2s(st + dst[i], src[i], bytes[i], &full[s]);
                    else
                        bulk_g2s_hint(st + dst[i], src[i], bytes[i], &full[s], policy);
                }
                mega_cursor_advance(a, ld, nphases, NT);
            }
        }
        return;
    }

    // ================= consumers =================
    uint32_t it = 0;        // units consumed so far (ring position)
    uint32_t nbar = 0;      // grid barriers passed
    bool ok = true;
    // running arg-max / log-sum-exp of the LM head rows owned by this thread
    unsigned long long best = 0ull;
    float lse_m = -INFINITY, lse_s = 0.f;

    // Values of the NEXT phase that do not depend on the phase being finished are fetched between the arrival at a
    // grid barrier and the wait for it: the RMSNorm weights of a norm-prologue phase, or (before the O projection) the
    // new token's V row and its score against every head's query (q, K and V of the new token were published by the
    // barrier before the attention phase).
    uint4 pre[MG_KCH];
    auto prework = [&](uint32_t pn) {
        const uint32_t layer = pn / 5;
        const int type = layer < a.layers ? static_cast<int>(pn % 5) : PH_LM;
        if (type == PH_QKV || type == PH_GU || type == PH_LM) {
            const T *gamma = static_cast<const T *>(type == PH_LM ? a.norm_f : type == PH_QKV ? a.layer[layer].norm1 : a.layer[layer].norm2);
#pragma unroll
            for (int c = 0; c < MG_KCH; ++c) {
                const uint32_t ci = tid + c * MG_CONSUMERS;
                pre[c] = ci < a.H / 8 ? __ldg(reinterpret_cast<const uint4 *>(gamma + ci * 8)) : make_uint4(0, 0, 0, 0);
            }
        } else if (type == PH_O) {
            const T *qbuf = static_cast<const T *>(ws.q);
            const uint32_t kvrep = a.nH / a.nKV;
#pragma unroll
            for (int c = 0; c < MG_KCH; ++c) {
                const uint32_t ci = tid + c * MG_CONSUMERS;
                pre[c] = make_uint4(0, 0, 0, 0);
                if (ci < a.nH * a.D / 8) {
                    const uint32_t h = ci * 8 / a.D, d0 = ci * 8 % a.D;
                    pre[c] = __ldcg(reinterpret_cast<const uint4 *>(static_cast<const T *>(a.layer[layer].vc) + (static_cast<size_t>(h / kvrep) * a.max_seq + pos) * a.D + d0));
                }
            }
            // score of the new token for every head: 8 threads per head
            for (uint32_t hb = 0; hb < a.nH; hb += MG_CONSUMERS / 8) {
                const uint32_t h = hb + tid / 8, pt = tid % 8;
                float d = 0.f;
                if (h < a.nH) {
                    const T *kn = static_cast<const T *>(a.layer[layer].kc) + (static_cast<size_t>(h / kvrep) * a.max_seq + pos) * a.D;
                    // D/8 chunks of 8 elements, 8 threads per head: chunks pt, pt + 8 (both loads in flight together)
                    uint4 qa = make_uint4(0, 0, 0, 0), ka = qa, qb = qa, kb = qa;
                    qa = __ldcg(reinterpret_cast<const uint4 *>(qbuf + h * a.D + pt * 8));
                    ka = __ldcg(reinterpret_cast<const uint4 *>(kn + pt * 8));
                    if (a.D > 64) {
                        qb = __ldcg(reinterpret_cast<const uint4 *>(qbuf + h * a.D + 64 + pt * 8));
                        kb = __ldcg(reinterpret_cast<const uint4 *>(kn + 64 + pt * 8));
                    }
                    float qf[8], kf[8];
                    unpack8<T>(qa, qf), unpack8<T>(ka, kf);
#pragma unroll
                    for (int e = 0; e < 8; ++e) d = fmaf(qf[e], kf[e], d);
                    unpack8<T>(qb, qf), unpack8<T>(kb, kf);
#pragma unroll
                    for (int e = 0; e < 8; ++e) d = fmaf(qf[e], kf[e], d);
                }
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                if (h < a.nH && pt == 0) sc[h] = d * a.scale;
            }
        }
    };
    auto grid_barrier = [&](uint32_t pnext) {
        // consumers of this CTA first (bar.sync orders their global writes before thread 0's release), then all CTAs
        mg_consumer_bar();
        ++nbar;
        if (tid == 0) asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(&hdr->bar), "l"(1ull) : "memory");
        if (pnext < nphases) prework(pnext);
        if (tid == 0) {
            const unsigned long long target = epoch + static_cast<unsigned long long>(nbar) * G;
            const uint64_t t0 = global_timer_ns();
            for (;;) {
                if (ld_acquire_gpu(&hdr->bar) >= target) break;
                if (ld_volatile_int(&hdr->abort) || global_timer_ns() - t0 > 2000000000ull) {
                    atomicExch(&hdr->abort, 1);
                    *s_fail = 1;
                    break;
                }
            }
        }
        mg_consumer_bar();// also publishes the scores prework wrote to shared memory
        if (*s_fail) ok = false;
        if (blockIdx.x == 0 && tid == 0) ws.timeline[nbar * 4] = global_timer_ns();
    };
    auto stamp = [&](uint32_t p, uint32_t k) {
        if (blockIdx.x == 0 && tid == 0) ws.timeline[p * 4 + k] = global_timer_ns();
    };
    stamp(0, 0);
    prework(0);

    for (uint32_t p = 0; p < nphases && ok; ++p) {
        const Phase ph = phase_of(a, p, NT);
        uint32_t u0, u1, att_head = 0;
        if (ph.type == PH_ATT) {
            if (!att_range(a, NT, blockIdx.x, G, att_head, u0, u1)) u0 = u1 = 0;
        } else {
            unit_range(ph.units, u0, u1);
        }
        const uint32_t nu = u1 - u0;

        if (ph.type == PH_ATT) {
            // ---------------- attention over cached tokens: this CTA = one head, a run of 64-token tiles ----------
            // Tiles are taken from the ring two at a time.  Each warp owns 8 tokens of either tile = the 16 rows of one
            // mma.sync.m16n8k16 whose B operand is the query: row r reads its 32-byte k-chunks in the order s ^ (r % 8)
            // (no bank conflicts although the rows lie 2*D bytes apart) and column n of B holds the query permuted the
            // same way, so C[r][r % 8] is the score of row r.  Each warp keeps its own online-softmax state, so a tile
            // needs no CTA-wide barrier; P.V runs on the FMA pipe, every lane accumulating its D/32 output dims.
            const T *qbuf = static_cast<const T *>(ws.q);
            const uint32_t D = a.D, DV = D / 32, NCH = D / 16, gq = lane >> 2, kq = lane & 3u, pg = gq % NCH;
            const bool own = kq == (gq >> 1);// this lane's c[gq & 1] / c[2 + (gq & 1)] are the scores of rows gq / gq + 8
            uint32_t qb[8][2];
            float m_w = -INFINITY, l_w = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
            if (nu) {
#pragma unroll
                for (int st = 0; st < 8; ++st) {
                    qb[st][0] = qb[st][1] = 0u;
                    if (st < static_cast<int>(NCH)) {
                        const uint32_t ch = static_cast<uint32_t>(st) ^ pg, hs = (NCH == 8 ? ch >> 2 : gq >> 2) & 1u;
                        const T *qp = qbuf + att_head * D + (ch * 16 + 2 * kq);
                        qb[st][0] = __ldcg(reinterpret_cast<const uint32_t *>(qp + (hs ? 8 : 0)));
                        qb[st][1] = __ldcg(reinterpret_cast<const uint32_t *>(qp + (hs ? 0 : 8)));
                    }
                }
            }
            for (uint32_t t = u0; t < u1 && ok;) {
                const uint32_t nb = u1 - t >= 2 ? 2u : 1u;
                const uint32_t sA = it % MG_STAGES, sB = (it + 1) % MG_STAGES;
                if (!mbar_wait(&full[sA], (it / MG_STAGES) & 1u) || (nb == 2 && !mbar_wait(&full[sB], ((it + 1) / MG_STAGES) & 1u))) {
                    ok = false;
                    break;
                }
                if (t == u0) stamp(p, 1);// first tiles have landed
                const uint32_t tokA = t * MG_TILE, ntA = pos - tokA < MG_TILE ? pos - tokA : MG_TILE;
                const uint32_t tokB = tokA + MG_TILE, ntB = nb == 2 ? (pos - tokB < MG_TILE ? pos - tokB : MG_TILE) : 0u;
                const uint8_t *ksA = smem + sA * MG_STAGE_BYTES, *ksB = smem + sB * MG_STAGE_BYTES;
                const uint32_t tk = warp * 8 + gq;// this lane's row in either tile
                const bool vA = tk < ntA, vB = tk < ntB;
                float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};// two chains: mma latency, not issue, bounds this
#pragma unroll
                for (int st = 0; st < 8; ++st) {
                    if (st < static_cast<int>(NCH)) {
                        // the two 16-byte halves of a chunk swap roles (in A and in B alike) where that keeps the 32 lanes of
                        // one load on 32 different banks
                        const uint32_t ch = static_cast<uint32_t>(st) ^ pg, hs = (NCH == 8 ? ch >> 2 : gq >> 2) & 1u;
                        const uint32_t off = tk * (D * 2) + ch * 32 + kq * 4, o0 = off + (hs ? 16u : 0u), o1 = off + (hs ? 0u : 16u);
                        uint32_t af[4];
                        af[0] = vA ? *reinterpret_cast<const uint32_t *>(ksA + o0) : 0u;
                        af[2] = vA ? *reinterpret_cast<const uint32_t *>(ksA + o1) : 0u;
                        af[1] = vB ? *reinterpret_cast<const uint32_t *>(ksB + o0) : 0u;
                        af[3] = vB ? *reinterpret_cast<const uint32_t *>(ksB + o1) : 0u;
                        if (st & 1) mma16816<T>(c2, af, qb[st][0], qb[st][1]);
                        else
                            mma16816<T>(c, af, qb[st][0], qb[st][1]);
                    }
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) c[e] += c2[e];
                const float sa = (own && vA) ? ((gq & 1u) ? c[1] : c[0]) * a.scale : -INFINITY;
                const float sb = (own && vB) ? ((gq & 1u) ? c[3] : c[2]) * a.scale : -INFINITY;
                const float m_new = fmaxf(m_w, warp_max(fmaxf(sa, sb)));
                const float pa = (sa == -INFINITY) ? 0.f : __expf(sa - m_new);
                const float pb = (sb == -INFINITY) ? 0.f : __expf(sb - m_new);
                const float corr = (m_w == -INFINITY) ? 0.f : __expf(m_w - m_new);
                l_w = l_w * corr + warp_sum(pa + pb);
                m_w = m_new;
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] *= corr;
                // P.V: all 16 loads of the warp's rows first (rows past the end of the sequence read as zero: no branch
                // separates the loads), then the multiply-adds
                uint2 vraw[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint8_t *vs = (j < 8 ? ksA : ksB) + MG_STAGE_BYTES / 2;
                    const uint32_t tok = warp * 8 + (j & 7);
                    const bool live = tok < (j < 8 ? ntA : ntB);
                    vraw[j] = make_uint2(0u, 0u);
                    if (DV == 4) {
                        if (live) vraw[j] = *reinterpret_cast<const uint2 *>(vs + tok * (D * 2) + lane * 8);
                    } else {
                        if (live) vraw[j].x = *reinterpret_cast<const uint32_t *>(vs + tok * (D * 2) + lane * 4);
                    }
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
                if (lane == 0) {
                    mbar_arrive(&empty[sA]);
                    if (nb == 2) mbar_arrive(&empty[sB]);
                }
                t += nb, it += nb;
            }
            stamp(p, 2);
            if (ok && nu) {
                // merge the eight warps' states and write this CTA's record [m, l, -, -, acc[D]]
                float *wst = part + warp * (D + 2);
                if (lane == 0) wst[0] = m_w, wst[1] = l_w;
                for (uint32_t e = 0; e < DV; ++e) wst[2 + lane * DV + e] = acc[e];
                mg_consumer_bar();
                float *rec = ws.rec + static_cast<size_t>(blockIdx.x) * (D + 4);
                float M = -INFINITY;
                for (int w = 0; w < MG_NW; ++w) M = fmaxf(M, part[w * (D + 2)]);
                if (tid < D) {
                    float o = 0.f;
                    for (int w = 0; w < MG_NW; ++w) {
                        const float mw = part[w * (D + 2)];
                        if (mw != -INFINITY) o += part[w * (D + 2) + 2 + tid] * expf(mw - M);
                    }
                    rec[4 + tid] = o;
                }
                if (tid == 0) {
                    float L = 0.f;
                    for (int w = 0; w < MG_NW; ++w) {
                        const float mw = part[w * (D + 2)];
                        if (mw != -INFINITY) L += part[w * (D + 2) + 1] * expf(mw - M);
                    }
                    rec[0] = M, rec[1] = L;
                }
            }
            if (!ok) {
                atomicExch(&hdr->abort, 1);
                *s_fail = 1;
            }
            stamp(p, 3);
            grid_barrier(p + 1);
            continue;
        }

        // ---------------- linear phases ----------------
        const uint32_t kchunks = ph.k / 8;
        float x[MG_KCH][8];
        {
            // activation vector of this phase, in registers
            const T *src = nullptr, *gamma = nullptr;
            if (ph.type == PH_QKV) {
                src = ph.layer == 0 ? static_cast<const T *>(a.embed) + static_cast<size_t>(token) * a.H : static_cast<const T *>(ws.x);
                gamma = static_cast<const T *>(a.layer[ph.layer].norm1);
            } else if (ph.type == PH_GU) {
                src = static_cast<const T *>(ws.h), gamma = static_cast<const T *>(a.layer[ph.layer].norm2);
            } else if (ph.type == PH_DOWN) {
                src = static_cast<const T *>(ws.u);
            } else if (ph.type == PH_LM) {
                src = a.layers ? static_cast<const T *>(ws.x) : static_cast<const T *>(a.embed) + static_cast<size_t>(token) * a.H;
                gamma = static_cast<const T *>(a.norm_f);
            }
            if (ph.type == PH_O) {
                // x = attention output = merge of the partial records + the token produced in this step (its V row is in
                // pre[], its scores in sc[]: see prework)
                const uint32_t kvrep = a.nH / a.nKV;
                (void) kvrep;
                const uint32_t splits = att_splits(G, a.nH);
#pragma unroll
                for (int c = 0; c < MG_KCH; ++c) {
                    const uint32_t ci = tid + c * MG_CONSUMERS;
#pragma unroll
                    for (int j = 0; j < 8; ++j) x[c][j] = 0.f;
                    if (ci < kchunks) {
                        const uint32_t h = ci * 8 / a.D, d0 = ci * 8 % a.D;
                        // start from the token produced in this step, then fold in the records of head h (CTAs
                        // h*splits + j whose tile range is not empty) four at a time, rescaling to the running maximum
                        float vnf[8];
                        unpack8<T>(pre[c], vnf);
                        float mx = sc[h], den = 1.f;
#pragma unroll
                        for (int j = 0; j < 8; ++j) x[c][j] = vnf[j];
                        for (uint32_t j0 = 0; j0 < splits; j0 += 4) {
                            float2 ml[4];
                            float4 r0[4], r1[4];
                            uint32_t live = 0;
#pragma unroll
                            for (uint32_t jj = 0; jj < 4; ++jj) {
                                const uint32_t j = j0 + jj;
                                if (j < splits && NT * (j + 1) / splits > NT * j / splits) {
                                    const float *rec = ws.rec + static_cast<size_t>(h * splits + j) * (a.D + 4);
                                    ml[jj] = __ldcg(reinterpret_cast<const float2 *>(rec));
                                    r0[jj] = __ldcg(reinterpret_cast<const float4 *>(rec + 4 + d0));
                                    r1[jj] = __ldcg(reinterpret_cast<const float4 *>(rec + 4 + d0 + 4));
                                    live |= 1u << jj;
                                }
                            }
                            float nm = mx;
#pragma unroll
                            for (uint32_t jj = 0; jj < 4; ++jj)
                                if (live >> jj & 1u) nm = fmaxf(nm, ml[jj].x);
                            const float f = expf(mx - nm);
                            den *= f;
#pragma unroll
                            for (int j = 0; j < 8; ++j) x[c][j] *= f;
                            mx = nm;
#pragma unroll
                            for (uint32_t jj = 0; jj < 4; ++jj) {
                                if (live >> jj & 1u) {
                                    const float w = expf(ml[jj].x - mx);
                                    den += ml[jj].y * w;
                                    x[c][0] += r0[jj].x * w, x[c][1] += r0[jj].y * w, x[c][2] += r0[jj].z * w, x[c][3] += r0[jj].w * w;
                                    x[c][4] += r1[jj].x * w, x[c][5] += r1[jj].y * w, x[c][6] += r1[jj].z * w, x[c][7] += r1[jj].w * w;
                                }
                            }
                        }
                        const float inv = 1.f / den;
                        // the multi-kernel path stores the attention output in 16 bits before the projection
#pragma unroll
                        for (int j = 0; j < 8; ++j) x[c][j] = Num<T>::to_f(Num<T>::from_f(x[c][j] * inv));
                    }
                }
            } else {
                float ss = 0.f;
#pragma unroll
                for (int c = 0; c < MG_KCH; ++c) {
                    const uint32_t ci = tid + c * MG_CONSUMERS;
                    if (ci < kchunks) {
                        unpack8<T>(__ldcg(reinterpret_cast<const uint4 *>(src + ci * 8)), x[c]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) x[c][j] = 0.f;
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) ss += x[c][j] * x[c][j];
                }
                if (gamma) {
                    float v = warp_sum(ss);
                    if (lane == 0) red[warp] = v;
                    mg_consumer_bar();
                    float tot = 0.f;
#pragma unroll
                    for (int w = 0; w < MG_NW; ++w) tot += red[w];
                    mg_consumer_bar();
                    const float rstd = rsqrtf(tot / static_cast<float>(ph.k) + a.eps);
#pragma unroll
                    for (int c = 0; c < MG_KCH; ++c) {
                        const uint32_t ci = tid + c * MG_CONSUMERS;
                        if (ci < kchunks) {
                            float gw[8];
                            unpack8<T>(pre[c], gw);
#pragma unroll
                            for (int j = 0; j < 8; ++j) x[c][j] *= rstd * gw[j];
                        }
                    }
                }
            }
        }

        stamp(p, 1);
        const uint32_t R = ph.g * ph.segs;
        // the row count per unit (1, 2 or 4) and the number of live k-chunks per thread (2, 4 or 6) are fixed for a
        // phase: dispatch once to a fully unrolled loop so that all shared-memory loads of a unit are in flight together
        const uint32_t kc_live = (kchunks + MG_CONSUMERS - 1) / MG_CONSUMERS;
#define RG_MG_RUN(R_, KC_) ok = mega_linear_units<T, R_, KC_>(smem, full, empty, part, x, nu, it, ph.k, tid, warp, lane)
        if (R == 4) {
            if (kc_live <= 2) RG_MG_RUN(4, 2);
            else if (kc_live <= 4) RG_MG_RUN(4, 4);
            else RG_MG_RUN(4, 6);
        } else if (R == 2) {
            if (kc_live <= 2) RG_MG_RUN(2, 2);
            else if (kc_live <= 4) RG_MG_RUN(2, 4);
            else RG_MG_RUN(2, 6);
        } else {
            if (kc_live <= 2) RG_MG_RUN(1, 2);
            else if (kc_live <= 4) RG_MG_RUN(1, 4);
            else RG_MG_RUN(1, 6);
        }
#undef RG_MG_RUN
        if (!ok) {
            atomicExch(&hdr->abort, 1);
            *s_fail = 1;
        }
        mg_consumer_bar();
        if (*s_fail) ok = false;
        stamp(p, 2);

        // ---------------- epilogue: one item = (local unit, row r within g) ----------------
        if (ok) {
            const uint32_t g = ph.g;
            for (uint32_t e = tid; e < nu * g; e += MG_CONSUMERS) {
                const uint32_t r = e % g, lu = e / g, u = u0 + lu;
                float val[2] = {0.f, 0.f};
                for (uint32_t sg = 0; sg < ph.segs; ++sg) {
                    const float *pp = part + ((lu * 4) + (sg * g + r)) * MG_NW;
                    float t = 0.f;
#pragma unroll
                    for (int w = 0; w < MG_NW; ++w) t += pp[w];
                    val[sg] = t;
                }
                uint32_t rows;
                const uint32_t row0 = mega_unit_row(a, ph, u, 0, rows);
                if (r >= rows) continue;
                if (ph.type == PH_QKV) {
                    const uint32_t D = a.D, half = D / 2, nq = a.nH, nkv = a.nKV;
                    const uint32_t h = row0 / D, i = row0 % D + r;
                    float lo = val[0], hi = val[1];
                    if (h < nq + nkv) {
                        const float inv_freq = exp2f(-a.log2_theta * (2.0f * static_cast<float>(i) / static_cast<float>(D)));
                        float sn, cs;
                        sincosf(static_cast<float>(pos) * inv_freq, &sn, &cs);
                        const float a0 = lo * cs - hi * sn, b0 = hi * cs + lo * sn;
                        lo = a0, hi = b0;
                    }
                    if (h < nq) {
                        T *q = static_cast<T *>(ws.q) + h * D;
                        q[i] = Num<T>::from_f(lo);
                        q[i + half] = Num<T>::from_f(hi);
                    } else {
                        const bool is_k = h < nq + nkv;
                        const uint32_t kvh = is_k ? h - nq : h - nq - nkv;
                        T *cache = static_cast<T *>(is_k ? a.layer[ph.layer].kc : a.layer[ph.layer].vc);
                        const size_t base = (static_cast<size_t>(kvh) * a.max_seq + pos) * D;
                        cache[base + i] = Num<T>::from_f(lo);
                        cache[base + i + half] = Num<T>::from_f(hi);
                    }
                } else if (ph.type == PH_O) {
                    const T *resid = ph.layer == 0 ? static_cast<const T *>(a.embed) + static_cast<size_t>(token) * a.H : static_cast<const T *>(ws.x);
                    static_cast<T *>(ws.h)[row0 + r] = Num<T>::from_f(val[0] + Num<T>::to_f(__ldcg(resid + row0 + r)));
                } else if (ph.type == PH_GU) {
                    const float gt = val[0];
                    static_cast<T *>(ws.u)[row0 + r] = Num<T>::from_f(gt / (1.f + expf(-gt)) * val[1]);
                } else if (ph.type == PH_DOWN) {
                    static_cast<T *>(ws.x)[row0 + r] = Num<T>::from_f(val[0] + Num<T>::to_f(__ldcg(static_cast<const T *>(ws.h) + row0 + r)));
                } else {
                    const T lg = Num<T>::from_f(val[0]);
                    static_cast<T *>(a.logits)[row0 + r] = lg;
                    const float f = Num<T>::to_f(lg);
                    uint32_t key = 0u;
                    if (f == f) {
                        const uint32_t b = __float_as_uint(f);
                        key = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
                        if (f > lse_m) {
                            lse_s = lse_s * (lse_m == -INFINITY ? 0.f : expf(lse_m - f)) + 1.f;
                            lse_m = f;
                        } else {
                            lse_s += expf(f - lse_m);
                        }
                    }
                    const unsigned long long comp = (static_cast<unsigned long long>(key) << 32) | static_cast<unsigned long long>(~(row0 + r));
                    best = comp > best ? comp : best;
                }
            }
        }
        if (ph.type == PH_LM && ok) {
            // CTA-level arg-max and log-sum-exp of this CTA's logits
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long ob = __shfl_xor_sync(0xffffffffu, best, o);
                best = ob > best ? ob : best;
                const float om = __shfl_xor_sync(0xffffffffu, lse_m, o), os = __shfl_xor_sync(0xffffffffu, lse_s, o);
                const float mm = fmaxf(lse_m, om);
                const float s1 = lse_m == -INFINITY ? 0.f : lse_s * expf(lse_m - mm), s2 = om == -INFINITY ? 0.f : os * expf(om - mm);
                lse_m = mm, lse_s = s1 + s2;
            }
            if (lane == 0) {
                atomicMax(&hdr->best, best);
                red[warp] = lse_m;
                red[8 + warp] = lse_s;
            }
            mg_consumer_bar();
            if (tid == 0) {
                float mm = -INFINITY, ssum = 0.f;
                for (int w = 0; w < MG_NW; ++w) mm = fmaxf(mm, red[w]);
                for (int w = 0; w < MG_NW; ++w) ssum += red[w] == -INFINITY ? 0.f : red[8 + w] * expf(red[w] - mm);
                ws.lse[blockIdx.x] = make_float2(mm, ssum);
            }
        }
        stamp(p, 3);
        grid_barrier(p + 1);
    }

    // ================= finish: next token, probability, state =================
    if (ok && blockIdx.x == 0 && warp == 0) {
        float mm = -INFINITY, ssum = 0.f;
        for (uint32_t c = lane; c < G; c += 32) mm = fmaxf(mm, __ldcg(&ws.lse[c].x));
        mm = warp_max(mm);
        for (uint32_t c = lane; c < G; c += 32) {
            const float2 v = __ldcg(&ws.lse[c]);
            ssum += v.x == -INFINITY ? 0.f : v.y * expf(v.x - mm);
        }
        ssum = warp_sum(ssum);
        if (lane == 0) {
            const unsigned long long b = ld_acquire_gpu(&hdr->best);
            const uint32_t idx = ~static_cast<uint32_t>(b & 0xffffffffull);
            *a.next = static_cast<int64_t>(idx);
            *a.prob = 1.0f / ssum;     // exp(max - max) / sum
            *a.token = static_cast<int64_t>(idx);
            *a.pos = static_cast<int64_t>(pos) + 1;
            hdr->best = 0ull;
            *reinterpret_cast<volatile unsigned long long *>(&hdr->epoch) = epoch + static_cast<unsigned long long>(nbar) * G;
        }
    }
    if (!ok && tid == 0) atomicExch(&s_mega_error, 1);
}

int mega_error_word(bool clear) { return error_symbol(s_mega_error, clear); }
int mega_index_error_word(bool clear) { return error_symbol(s_mega_index_error, clear); }

}// namespace rg

using namespace rg;

static size_t mega_smem_bytes() {
    return MG_STAGES * MG_STAGE_BYTES + 2 * MG_STAGES * 8 + (32 + 256 + 128) * 4 + MG_PART_UNITS * 4 * MG_NW * 4 + 16;
}

static int mega_validate(const rg_decode_step_params *p) {
    if (p->dtype != RG_FP16 && p->dtype != RG_BF16) return RG_ERR_DTYPE;
    if (p->layers > MG_MAX_LAYERS || p->hidden == 0 || p->n_heads == 0 || p->n_kv_heads == 0 || p->n_heads % p->n_kv_heads) return RG_ERR_SHAPE;
    if (p->head_dim != 128 && p->head_dim != 64) return RG_ERR_SHAPE;
    const uint32_t qd = p->n_heads * p->head_dim;
    if (p->hidden % 8 || p->ffn % 8 || qd % 8) return RG_ERR_SHAPE;
    if (p->hidden > MG_KCH * 256 * 8 || p->ffn > MG_KCH * 256 * 8 || qd > MG_KCH * 256 * 8) return RG_ERR_SHAPE;
    if (p->hidden * 4u > MG_STAGE_BYTES || p->ffn * 2u > MG_STAGE_BYTES || qd * 2u > MG_STAGE_BYTES) return RG_ERR_SHAPE;
    if (p->n_heads > 128 || MG_TILE * p->head_dim * 2u * 2u > MG_STAGE_BYTES) return RG_ERR_SHAPE;
    return RG_OK;
}

extern "C" {

// Diagnostics: copies the per-phase timestamps (ns, %globaltimer of CTA 0) of the last call out of the workspace: four
// entries per phase (entered, activations ready, units consumed, epilogue done; phases are, per layer, QKV, attention,
// O, gate/up, down, then the LM head) and one more group whose first entry is the end of the last grid barrier.
// Synchronises the device.  Returns the number of entries written.
size_t rg_b200_decode_step_timeline(const rg_decode_step_params *p, const void *ws, uint64_t *out, size_t capacity) {
    if (!p || !ws || !out) return 0;
    const uint32_t G = static_cast<uint32_t>(sm_count());
    const size_t off = mega_ws_bytes(G, p->hidden, p->n_heads, p->head_dim, p->ffn) - mg_align((MG_MAX_LAYERS * 5 + 2) * 4 * 8);
    size_t n = (static_cast<size_t>(p->layers) * 5 + 2) * 4;
    if (n > capacity) n = capacity;
    if (cudaDeviceSynchronize() != cudaSuccess) return 0;
    if (cudaMemcpy(out, static_cast<const uint8_t *>(ws) + off, n * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
    return n;
}

size_t rg_b200_decode_step_workspace(const rg_decode_step_params *p) {
    if (!p) return 0;
    return mega_ws_bytes(static_cast<uint32_t>(sm_count()), p->hidden, p->n_heads, p->head_dim, p->ffn);
}

int rg_b200_decode_step(const rg_decode_step_params *p, void *ws, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !ws) return RG_ERR_NULL;
    const int rc = mega_validate(p);
    if (rc != RG_OK) return rc;
    const uint32_t G = static_cast<uint32_t>(sm_count());
    // no CTA may get more units of any phase than its partial-sum table holds: the same unit arithmetic as the kernel's
    {
        const uint32_t qd = p->n_heads * p->head_dim, D = p->head_dim, F = p->ffn, H = p->hidden;
        const uint32_t shapes[5][4] = {{PH_QKV, (p->n_heads + 2 * p->n_kv_heads) * D, H, 2}, {PH_O, H, qd, 1}, {PH_GU, 2 * F, H, 2}, {PH_DOWN, H, F, 1},
                                       {PH_LM, p->vocab, H, 1}};
        for (auto const &sh : shapes) {
            uint32_t g = 0;
            const uint32_t units = mega_phase_units(static_cast<int>(sh[0]), sh[1], sh[2], sh[3], D, F, g);
            if (g == 0 || (units + G - 1) / G > MG_PART_UNITS) return RG_ERR_SHAPE;
        }
    }
    if (p->n_heads > G) return RG_ERR_SHAPE;// the attention phase gives every head 1..8 CTAs
    MegaArgs a = {};
    // inputs: token, pos, embed, norm_f, lm_head, then per layer norm1, wqkv, wo, norm2, wgu, wd, k_cache, v_cache
    a.token = static_cast<int64_t *>(const_cast<void *>(in[0]));
    a.pos = static_cast<int64_t *>(const_cast<void *>(in[1]));
    a.embed = in[2], a.norm_f = in[3], a.lm_head = in[4];
    if (!a.token || !a.pos || !a.embed || !a.norm_f || !a.lm_head) return RG_ERR_NULL;
    for (uint32_t l = 0; l < p->layers; ++l) {
        const void *const *q = in + 5 + 8 * l;
        for (int j = 0; j < 8; ++j)
            if (!q[j]) return RG_ERR_NULL;
        a.layer[l] = {q[0], q[1], q[2], q[3], q[4], q[5], const_cast<void *>(q[6]), const_cast<void *>(q[7])};
        if (!aligned16(q[1]) || !aligned16(q[2]) || !aligned16(q[4]) || !aligned16(q[5]) || !aligned16(q[6]) || !aligned16(q[7])) return RG_ERR_ALIGN;
    }
    a.next = static_cast<int64_t *>(out[0]);
    a.prob = static_cast<float *>(out[1]);
    a.logits = out[2];
    if (!a.next || !a.prob || !a.logits) return RG_ERR_NULL;
    a.ws = static_cast<uint8_t *>(ws);
    a.layers = p->layers, a.H = p->hidden, a.nH = p->n_heads, a.nKV = p->n_kv_heads, a.D = p->head_dim, a.F = p->ffn, a.V = p->vocab;
    a.max_seq = p->max_seq;
    a.eps = p->epsilon, a.log2_theta = log2f(p->theta), a.scale = 1.0f / sqrtf(static_cast<float>(p->head_dim));
    const size_t smem = mega_smem_bytes();
    void *kern = p->dtype == RG_FP16 ? reinterpret_cast<void *>(decode_mega_kernel<__half>) : reinterpret_cast<void *>(decode_mega_kernel<__nv_bfloat16>);
    RG_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    // cooperative launch: all CTAs are resident together, which the grid barriers rely on
    void *args[] = {&a};
    RG_CHECK_CUDA(cudaLaunchCooperativeKernel(kern, dim3(G), dim3(MG_THREADS), args, smem, static_cast<cudaStream_t>(stream)));
    count_launch();
    return RG_OK;
}
}
