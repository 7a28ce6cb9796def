// AllReduce across the GPUs of one NVSwitch box, one process per GPU.  Replaces AllReduceNccl + NcclCommunicator
// (src/04kernel/src/kernels/all_reduce/nccl_kernel.cu:9-19, src/04kernel/src/utilities/cuda/nccl_communicator.cu:11-44).
//
// One-shot push over peer memory with the flag inside the data: every rank owns a "symmetric" allocation (header, data
// slots [parity][source rank]) that its peers map through CUDA IPC.  Call number s (kept in device memory, so a captured
// CUDA graph can replay it): every thread takes 16-byte chunks of the input, pairs each 32-bit word with the 32-bit call
// number and stores the resulting 32 bytes into slot [s&1][rank] of EVERY peer (two 16-byte stores over NVLink; an
// aligned 8-byte {data, flag} pair is written as one unit), then polls the same 32 bytes of every peer's slot in its OWN
// allocation until all four flags carry s, and combines the values in fp32 in rank order (so all ranks get bit-identical
// results).  There is no fence, no separate flag and no barrier on the path: the latency is one NVLink store flight.
// Parity s&1 is not rewritten before call s+2, which no rank starts before it has finished call s+1, whose data it sends
// only after it has read everything of call s.  Measured for 256 KiB per rank: a pull design (remote flag polls and remote
// loads) 26 / 49 us on 2 / 8 GPUs; push with a system fence and one flag per CTA 20 / 26 us; the sum formed inside NVSwitch
// (multimem.ld_reduce + multimem.st on a multicast mapping, two flag barriers) 30 us on 2 GPUs, where this push takes 8.9: six
// NVLink flights in a row instead of one.  Two-shot on 8 GPUs: 15.5 us.
// No TMA and no multicast instructions touch peer memory.
#include "gemm_dispatch.cuh"
#include "ar_slots.cuh"
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

namespace rg {

constexpr int AR_THREADS = 256;

struct ArArgs {
    uint8_t *mine;
    uint8_t *peer[AR_MAX_RANKS];// peer[rank] = mine
    const void *x, *res;// x == nullptr: this rank's input is already in its slots (written by a product's epilogue): receive only
    void *y;
    uint64_t count;
    size_t capacity;
    int world, rank, op;
    uint64_t wait_ns;
};

// Element traits: A is the type the combine runs in.  16-bit floats combine in fp32; every other type combines in its
// own type, as the NCCL call this replaces does (integer sums and products wrap).
template<class T> struct ArElem {
    using A = T;
    static __device__ __forceinline__ A up(T v) { return v; }
    static __device__ __forceinline__ T down(A v) { return v; }
};
template<> struct ArElem<__half> {
    using A = float;
    static __device__ __forceinline__ A up(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half down(A v) { return __float2half_rn(v); }
};
template<> struct ArElem<__nv_bfloat16> {
    using A = float;
    static __device__ __forceinline__ A up(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 down(A v) { return __float2bfloat16_rn(v); }
};
template<class A> __device__ __forceinline__ A ar_combine(int op, A a, A b) {
    switch (op) {
        case 2: return a < b ? a : b;
        case 3: return a > b ? a : b;
        case 4: return a * b;
        default: return a + b;
    }
}
template<> __device__ __forceinline__ float ar_combine<float>(int op, float a, float b) {
    switch (op) {
        case 2: return fminf(a, b);
        case 3: return fmaxf(a, b);
        case 4: return a * b;
        default: return a + b;
    }
}
template<> __device__ __forceinline__ double ar_combine<double>(int op, double a, double b) {
    switch (op) {
        case 2: return fmin(a, b);
        case 3: return fmax(a, b);
        case 4: return a * b;
        default: return a + b;
    }
}
// Avg: floating types multiply by 1 / world (fp32 for the 16-bit types and float, fp64 for double); integers divide.
template<class A> __device__ __forceinline__ A ar_average(A v, int world) { return v / static_cast<A>(world); }
template<> __device__ __forceinline__ float ar_average<float>(float v, int world) { return v * (1.0f / static_cast<float>(world)); }
template<> __device__ __forceinline__ double ar_average<double>(double v, int world) { return v * (1.0 / static_cast<double>(world)); }

// Combines the world chunks in rank order (bit-identical on every rank), applies Avg, then the optional residual: the reduced
// value is rounded to the storage type before the residual is added, exactly as if the all-reduce and the Add were two operators.
template<class T>
__device__ __forceinline__ uint4 ar_reduce_chunk(const uint4 (&raw)[8], int world, int op, const T *res, uint64_t e0, uint64_t count) {
    constexpr int N = 16 / sizeof(T);
    using A = typename ArElem<T>::A;
    A acc[N];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        if (r < world) {
            const T *v = reinterpret_cast<const T *>(&raw[r]);
#pragma unroll
            for (int j = 0; j < N; ++j) acc[j] = r == 0 ? ArElem<T>::up(v[j]) : ar_combine<A>(op, acc[j], ArElem<T>::up(v[j]));
        }
    }
    if (op == 1) {
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] = ar_average<A>(acc[j], world);
    }
    uint4 out;
    T *o = reinterpret_cast<T *>(&out);
#pragma unroll
    for (int j = 0; j < N; ++j) {
        o[j] = ArElem<T>::down(acc[j]);
        if (res && e0 + j < count) o[j] = ArElem<T>::down(ArElem<T>::up(o[j]) + ArElem<T>::up(res[e0 + j]));
    }
    return out;
}

// byte offset of the slot that holds rank `src`'s input of a call with parity q, inside any rank's allocation; a slot is
// 2 * capacity bytes because every 4 data bytes travel with a 4-byte flag
__device__ __forceinline__ size_t ar_slot_off(const ArArgs &a, unsigned q, int src) { return ar_slot_offset(a.capacity, a.world, q, src); }
__device__ __forceinline__ void st_volatile_v4(void *p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

template<class T>
__global__ void __launch_bounds__(AR_THREADS) all_reduce_kernel(const ArArgs a) {
    pdl_enter();
    constexpr int N = 16 / sizeof(T);
    ArHeader *hdr = reinterpret_cast<ArHeader *>(a.mine);
    __shared__ unsigned long long s_seq;
    if (threadIdx.x == 0) {
        const unsigned long long sq = *reinterpret_cast<volatile unsigned long long *>(&hdr->seq);
        s_seq = sq;
        // the last CTA to have read seq advances it for the next call
        if (atomicAdd(&hdr->done, 1u) == gridDim.x - 1) {
            hdr->done = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned long long *>(&hdr->seq) = sq + 1;
        }
    }
    __syncthreads();
    // A communicator whose earlier call gave up a wait is out of step with its peers for good: every later call is a no-op
    // (outputs untouched, status still set) until the host destroys and recreates it.
    if (*reinterpret_cast<volatile int *>(&hdr->status) != 0) return;
    const unsigned long long seq = s_seq;
    const unsigned q = static_cast<unsigned>(seq & 1ull);
    const uint32_t flag = ar_flag(seq);
    const uint64_t chunks = (a.count + N - 1) / N, full_chunks = a.count / N;
    const T *x = static_cast<const T *>(a.x);
    const T *res = static_cast<const T *>(a.res);
    T *y = static_cast<T *>(a.y);
    const size_t my_off = ar_slot_off(a, q, a.rank);
    const uint64_t t0 = global_timer_ns();

    for (uint64_t c = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < chunks; c += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        // 1. push chunk c of my input, every 32-bit word paired with the call's flag, into slot [q][rank] of every peer
        uint4 mine4 = make_uint4(0u, 0u, 0u, 0u);
        if (x) {
            if (c < full_chunks) {
                mine4 = *reinterpret_cast<const uint4 *>(x + c * N);
            } else {
                T *tail = reinterpret_cast<T *>(&mine4);
                for (uint64_t e = c * N; e < a.count; ++e) tail[e - c * N] = x[e];
            }
#pragma unroll
            for (int r = 0; r < AR_MAX_RANKS; ++r) {
                if (r < a.world && r != a.rank) {
                    uint8_t *dst = a.peer[r] + my_off + c * 32;
                    st_volatile_v4(dst, mine4.x, flag, mine4.y, flag);
                    st_volatile_v4(dst + 16, mine4.z, flag, mine4.w, flag);
                }
            }
        }
        // 2. the same chunk of every peer lands in my allocation: poll local memory until all four flags of a line match
        // (receive-only: this rank's own chunk is read from its own slot the same way)
        uint4 raw[AR_MAX_RANKS];
        bool ok = true;
#pragma unroll
        for (int r = 0; r < AR_MAX_RANKS; ++r) {
            raw[r] = mine4;
            if (r < a.world && (r != a.rank || !x) && ok) {
                const uint8_t *src = a.mine + ar_slot_off(a, q, r) + c * 32;
                for (uint32_t spin = 1;; ++spin) {
                    const uint4 lo = ld_volatile_v4(src), hi = ld_volatile_v4(src + 16);
                    if (lo.y == flag && lo.w == flag && hi.y == flag && hi.w == flag) {
                        raw[r] = make_uint4(lo.x, lo.z, hi.x, hi.z);
                        break;
                    }
                    if ((spin & 63u) == 0 && global_timer_ns() - t0 > a.wait_ns) {
                        ok = false;
                        break;
                    }
                }
            }
        }
        if (!ok) {
            hdr->status = 1;// the output stays untouched; the host sees the status word
            return;
        }
        // 3. combine in rank order, so that every rank computes bit-identical results
        const uint4 out4 = ar_reduce_chunk<T>(raw, a.world, a.op, res, c * N, a.count);
        if (c < full_chunks) {
            *reinterpret_cast<uint4 *>(y + c * N) = out4;
        } else {
            const T *tail = reinterpret_cast<const T *>(&out4);
            for (uint64_t e = c * N; e < a.count; ++e) y[e] = tail[e - c * N];
        }
    }
}

// Two-shot variant for large groups: a one-shot push moves (world - 1) x the vector out of every GPU, which on 8 GPUs costs
// more than a second NVLink flight.  Here warp-sized runs of 32 chunks have an owner rank ((c / 32) % world): every rank
// sends its chunk to the owner only; the owner combines the world values in rank order, adds the residual, and pushes the
// finished 16 bytes to every peer, which copies them to its output.  Same flag-in-data lines, same parity rule, a second
// slot (B) for the finished values.  Every thread sends before it waits, and all ranks walk the chunks in the same order.
template<class T>
__global__ void __launch_bounds__(AR_THREADS) all_reduce_two_shot_kernel(const ArArgs a) {
    pdl_enter();
    constexpr int N = 16 / sizeof(T);
    ArHeader *hdr = reinterpret_cast<ArHeader *>(a.mine);
    __shared__ unsigned long long s_seq;
    if (threadIdx.x == 0) {
        const unsigned long long sq = *reinterpret_cast<volatile unsigned long long *>(&hdr->seq);
        s_seq = sq;
        if (atomicAdd(&hdr->done, 1u) == gridDim.x - 1) {
            hdr->done = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned long long *>(&hdr->seq) = sq + 1;
        }
    }
    __syncthreads();
    // A communicator whose earlier call gave up a wait is out of step with its peers for good: every later call is a no-op
    // (outputs untouched, status still set) until the host destroys and recreates it.
    if (*reinterpret_cast<volatile int *>(&hdr->status) != 0) return;
    const unsigned long long seq = s_seq;
    const unsigned q = static_cast<unsigned>(seq & 1ull);
    const uint32_t flag = ar_flag(seq);
    const uint64_t chunks = (a.count + N - 1) / N, full_chunks = a.count / N;
    const T *x = static_cast<const T *>(a.x);
    const T *res = static_cast<const T *>(a.res);
    T *y = static_cast<T *>(a.y);
    const size_t my_off = ar_slot_off(a, q, a.rank);
    const size_t b_off = ar_slot_off(a, 2, 0) + static_cast<size_t>(q) * (2 * a.capacity);// slot B follows the 2 * world A slots
    const uint64_t t0 = global_timer_ns();

    for (uint64_t c = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < chunks; c += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const int owner = static_cast<int>((c / 32) % static_cast<uint64_t>(a.world));
        uint4 mine4 = make_uint4(0u, 0u, 0u, 0u);
        if (x) {
            if (c < full_chunks) {
                mine4 = *reinterpret_cast<const uint4 *>(x + c * N);
            } else {
                T *tail = reinterpret_cast<T *>(&mine4);
                for (uint64_t e = c * N; e < a.count; ++e) tail[e - c * N] = x[e];
            }
        }
        uint4 out4;
        bool ok = true;
        if (owner != a.rank) {
            if (x) {
                uint8_t *dst = a.peer[owner] + my_off + c * 32;
                st_volatile_v4(dst, mine4.x, flag, mine4.y, flag);
                st_volatile_v4(dst + 16, mine4.z, flag, mine4.w, flag);
            }
            const uint8_t *src = a.mine + b_off + c * 32;
            for (uint32_t spin = 1;; ++spin) {
                const uint4 lo = ld_volatile_v4(src), hi = ld_volatile_v4(src + 16);
                if (lo.y == flag && lo.w == flag && hi.y == flag && hi.w == flag) {
                    out4 = make_uint4(lo.x, lo.z, hi.x, hi.z);
                    break;
                }
                if ((spin & 63u) == 0 && global_timer_ns() - t0 > a.wait_ns) {
                    ok = false;
                    break;
                }
            }
        } else {
            uint4 raw[AR_MAX_RANKS];
#pragma unroll
            for (int r = 0; r < AR_MAX_RANKS; ++r) {
                raw[r] = mine4;
                if (r < a.world && (r != a.rank || !x) && ok) {
                    const uint8_t *src = a.mine + ar_slot_off(a, q, r) + c * 32;
                    for (uint32_t spin = 1;; ++spin) {
                        const uint4 lo = ld_volatile_v4(src), hi = ld_volatile_v4(src + 16);
                        if (lo.y == flag && lo.w == flag && hi.y == flag && hi.w == flag) {
                            raw[r] = make_uint4(lo.x, lo.z, hi.x, hi.z);
                            break;
                        }
                        if ((spin & 63u) == 0 && global_timer_ns() - t0 > a.wait_ns) {
                            ok = false;
                            break;
                        }
                    }
                }
            }
            out4 = ar_reduce_chunk<T>(raw, a.world, a.op, res, c * N, a.count);
            if (ok) {
#pragma unroll
                for (int r = 0; r < AR_MAX_RANKS; ++r) {
                    if (r < a.world && r != a.rank) {
                        uint8_t *dst = a.peer[r] + b_off + c * 32;
                        st_volatile_v4(dst, out4.x, flag, out4.y, flag);
                        st_volatile_v4(dst + 16, out4.z, flag, out4.w, flag);
                    }
                }
            }
        }
        if (!ok) {
            hdr->status = 1;// the output stays untouched; the host sees the status word
            return;
        }
        if (c < full_chunks) {
            *reinterpret_cast<uint4 *>(y + c * N) = out4;
        } else {
            const T *tail = reinterpret_cast<const T *>(&out4);
            for (uint64_t e = c * N; e < a.count; ++e) y[e] = tail[e - c * N];
        }
    }
}


// ---------------------------------------------------------------------------------------------------------------------
// AllReduce(Sum) + residual + RmsNormalization in one launch: what follows the row-parallel products (O and down) of a
// tensor-parallel decoder layer.  y = sum over ranks of x (+ res), n = y * rsqrt(mean(y^2) + eps) * w.  One CTA per row with
// the thread / chunk assignment and the summation order of rms_norm_vec_kernel, so y and n carry the same bits as the
// all-reduce kernel followed by the normalisation kernel.  The exchange is the one above: flag-in-data lines, one-shot up to
// 3 ranks, owner-reduces-and-broadcasts beyond; a thread sends everything it has to send before it waits for anything.
struct ArNormArgs {
    ArArgs a;
    const void *w;
    void *n;
    uint32_t dim;
    float eps;
};

// polls the 32-byte line at src until its four flags match; false when the wait expired
__device__ __forceinline__ bool ar_poll_line(const uint8_t *src, uint32_t flag, uint64_t t0, uint64_t wait_ns, uint4 &out) {
    for (uint32_t spin = 1;; ++spin) {
        const uint4 lo = ld_volatile_v4(src), hi = ld_volatile_v4(src + 16);
        if (lo.y == flag && lo.w == flag && hi.y == flag && hi.w == flag) {
            out = make_uint4(lo.x, lo.z, hi.x, hi.z);
            return true;
        }
        if ((spin & 63u) == 0 && global_timer_ns() - t0 > wait_ns) return false;
    }
}
__device__ __forceinline__ void ar_push_line(uint8_t *dst, const uint4 &v, uint32_t flag) {
    st_volatile_v4(dst, v.x, flag, v.y, flag);
    st_volatile_v4(dst + 16, v.z, flag, v.w, flag);
}

// polls the lines src[k] whose bit is set in `need` until each carries the flag; the loads of one round are independent, so a
// round costs one trip to L2 whatever the number of lines.  out[k] is written for the lines asked for only.
template<int NL>
__device__ __forceinline__ bool ar_poll_many(const uint8_t *const (&src)[NL], uint32_t need, uint32_t flag, uint64_t t0, uint64_t wait_ns, uint4 (&out)[NL]) {
    for (uint32_t spin = 1; need; ++spin) {
        uint4 lo[NL], hi[NL];
#pragma unroll
        for (int k = 0; k < NL; ++k)
            if (need >> k & 1u) lo[k] = ld_volatile_v4(src[k]), hi[k] = ld_volatile_v4(src[k] + 16);
#pragma unroll
        for (int k = 0; k < NL; ++k)
            if ((need >> k & 1u) && lo[k].y == flag && lo[k].w == flag && hi[k].y == flag && hi[k].w == flag) {
                out[k] = make_uint4(lo[k].x, lo[k].z, hi[k].x, hi[k].z);
                need &= ~(1u << k);
            }
        if (need && (spin & 63u) == 0 && global_timer_ns() - t0 > wait_ns) return false;
    }
    return true;
}

template<class T, int CH, bool TWO>
__global__ void __launch_bounds__(AR_THREADS) all_reduce_norm_kernel(const ArNormArgs p) {
    pdl_enter();
    constexpr int N = 16 / sizeof(T);
    const ArArgs &a = p.a;
    ArHeader *hdr = reinterpret_cast<ArHeader *>(a.mine);
    __shared__ unsigned long long s_seq;
    __shared__ int s_status;
    __shared__ float red[33];
    if (threadIdx.x == 0) {
        const unsigned long long sq = *reinterpret_cast<volatile unsigned long long *>(&hdr->seq);
        s_seq = sq;
        s_status = *reinterpret_cast<volatile int *>(&hdr->status);// one read per CTA: the CTA leaves as a whole or not at all
        if (atomicAdd(&hdr->done, 1u) == gridDim.x - 1) {
            hdr->done = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned long long *>(&hdr->seq) = sq + 1;
        }
    }
    __syncthreads();
    if (s_status != 0) return;// out of step with the peers: no-op, as the plain kernels
    const unsigned long long seq = s_seq;
    const unsigned q = static_cast<unsigned>(seq & 1ull);
    const uint32_t flag = ar_flag(seq);
    const uint32_t chunks = p.dim / N;
    const uint64_t row0 = static_cast<uint64_t>(blockIdx.x) * chunks;// first chunk of this CTA's row
    const T *x = static_cast<const T *>(a.x);
    const T *res = static_cast<const T *>(a.res);
    T *y = static_cast<T *>(a.y);
    const size_t my_off = ar_slot_off(a, q, a.rank);
    const size_t b_off = ar_slot_off(a, 2, 0) + static_cast<size_t>(q) * (2 * a.capacity);
    const uint64_t t0 = global_timer_ns();

    // 1. send: to every peer (one-shot) or to the owner of the 32-chunk run (two-shot)
    uint4 mine[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const uint32_t c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            const uint64_t gc = row0 + c;
            mine[i] = *reinterpret_cast<const uint4 *>(x + gc * N);
            if constexpr (TWO) {
                const int owner = static_cast<int>((gc / 32) % static_cast<uint64_t>(a.world));
                if (owner != a.rank) ar_push_line(a.peer[owner] + my_off + gc * 32, mine[i], flag);
            } else {
#pragma unroll
                for (int r = 0; r < AR_MAX_RANKS; ++r)
                    if (r < a.world && r != a.rank) ar_push_line(a.peer[r] + my_off + gc * 32, mine[i], flag);
            }
        }
    }
    // 2. owned chunks (all of them, one-shot): gather the peers' lines, combine in rank order, add the residual.  All the lines
    // a thread waits for are polled together, so the wait costs one round trip to L2 and not one per line.
    bool ok = true;
    if constexpr (!TWO) {
        constexpr int PEERS = 3;         // one-shot serves up to 4 ranks (the default uses it up to 3)
        constexpr int G = CH < 4 ? CH : 4;// chunks polled together (more would not fit the register file)
#pragma unroll
        for (int i0 = 0; i0 < CH; i0 += G) {
            const uint8_t *src[G * PEERS];
            uint4 got[G * PEERS];
            uint32_t need = 0;
#pragma unroll
            for (int i = 0; i < G; ++i) {
                const uint32_t c = threadIdx.x + (i0 + i) * blockDim.x;
#pragma unroll
                for (int k = 0; k < PEERS; ++k) {
                    const int r = k < a.rank ? k : k + 1;// the k-th rank that is not this one
                    src[i * PEERS + k] = a.mine + ar_slot_off(a, q, r < a.world ? r : 0) + (row0 + c) * 32;
                    if (c < chunks && r < a.world) need |= 1u << (i * PEERS + k);
                }
            }
            if (ok) ok = ar_poll_many<G * PEERS>(src, need, flag, t0, a.wait_ns, got);
#pragma unroll
            for (int i = 0; i < G; ++i) {
                const uint32_t c = threadIdx.x + (i0 + i) * blockDim.x;
                if (c < chunks) {
                    uint4 raw[AR_MAX_RANKS];
#pragma unroll
                    for (int r = 0; r < AR_MAX_RANKS; ++r) raw[r] = mine[i0 + i];
#pragma unroll
                    for (int k = 0; k < PEERS; ++k) {
                        const int r = k < a.rank ? k : k + 1;
#pragma unroll
                        for (int rr = 0; rr < 4; ++rr)
                            if (rr == r && r < a.world) raw[rr] = got[i * PEERS + k];
                    }
                    mine[i0 + i] = ar_reduce_chunk<T>(raw, a.world, 0, res, (row0 + c) * N, a.count);
                }
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const uint32_t c = threadIdx.x + i * blockDim.x;
            if (c < chunks) {
                const uint64_t gc = row0 + c;
                if (static_cast<int>((gc / 32) % static_cast<uint64_t>(a.world)) == a.rank) {
                    const uint8_t *src[AR_MAX_RANKS];
                    uint4 raw[AR_MAX_RANKS];
                    uint32_t need = 0;
#pragma unroll
                    for (int r = 0; r < AR_MAX_RANKS; ++r) {
                        raw[r] = mine[i];
                        src[r] = a.mine + ar_slot_off(a, q, r < a.world ? r : 0) + gc * 32;
                        if (r < a.world && r != a.rank) need |= 1u << r;
                    }
                    if (ok) ok = ar_poll_many<AR_MAX_RANKS>(src, need, flag, t0, a.wait_ns, raw);
                    mine[i] = ar_reduce_chunk<T>(raw, a.world, 0, res, gc * N, a.count);
                    if (ok) {
#pragma unroll
                        for (int r = 0; r < AR_MAX_RANKS; ++r)
                            if (r < a.world && r != a.rank) ar_push_line(a.peer[r] + b_off + gc * 32, mine[i], flag);
                    }
                }
            }
        }
        // 3. the finished values of the chunks other ranks own
        const uint8_t *src[CH];
        uint32_t need = 0;
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const uint32_t c = threadIdx.x + i * blockDim.x;
            const uint64_t gc = row0 + c;
            src[i] = a.mine + b_off + gc * 32;
            if (c < chunks && static_cast<int>((gc / 32) % static_cast<uint64_t>(a.world)) != a.rank) need |= 1u << i;
        }
        if (ok) ok = ar_poll_many<CH>(src, need, flag, t0, a.wait_ns, mine);
    }
    if (__syncthreads_or(!ok)) {
        if (threadIdx.x == 0) hdr->status = 1;// outputs untouched; the host sees the status word
        return;
    }
    // 4. y, then the normalisation of the rounded y exactly as rms_norm_vec_kernel computes it
    float v[CH][N];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const uint32_t c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            *reinterpret_cast<uint4 *>(y + (row0 + c) * N) = mine[i];
            Vec16<T> t;
            t.raw = mine[i];
            t.unpack(v[i]);
#pragma unroll
            for (int j = 0; j < N; ++j) ss += v[i][j] * v[i][j];
        }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / static_cast<float>(p.dim) + p.eps);
    const T *w = static_cast<const T *>(p.w);
    T *n = static_cast<T *>(p.n);
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const uint32_t c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            Vec16<T> g, o;
            float gw[N], out[N];
            g.load(w + c * N);
            g.unpack(gw);
#pragma unroll
            for (int j = 0; j < N; ++j) out[j] = v[i][j] * rstd * gw[j];
            o.pack(out);
            o.store(n + (row0 + c) * N);
        }
    }
}


}// namespace rg

using namespace rg;

struct rg_comm {
    int world, rank, device;
    bool failed;// a timeout has been observed by the host: every later call is refused
    size_t capacity, total_bytes;
    uint8_t *mine;
    uint8_t *peers[AR_MAX_RANKS];
    bool opened[AR_MAX_RANKS];
    bool connected;
    uint64_t wait_ns;
};

// Live communicators of this process, so that rg_b200_error_state can report a timed-out all-reduce (bit 3).
static std::mutex g_comms_mutex;
static std::vector<rg_comm *> g_comms;

static int comm_read_status(rg_comm *c) {
    int st = 0;
    if (cudaMemcpy(&st, c->mine + offsetof(ArHeader, status), sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (st) c->failed = true;
    return st;
}

namespace rg {
// 1 when any communicator that lives on the current device has given up a wait; the status is a property of the communicator
// (out of step with its peers), so `clear` does not reset it.
int all_reduce_error_word(bool) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    std::lock_guard<std::mutex> lock(g_comms_mutex);
    int any = 0;
    for (rg_comm *c : g_comms) {
        if (c->device != dev) continue;
        const int st = comm_read_status(c);
        if (st < 0) return -1;
        any |= st ? 1 : 0;
    }
    return any;
}
}// namespace rg

extern "C" {

int rg_b200_comm_create(int world, int rank, size_t capacity_bytes, rg_comm **out, void *handle64) {
    if (!out || !handle64) return RG_ERR_NULL;
    if (world < 1 || world > AR_MAX_RANKS || rank < 0 || rank >= world) return RG_ERR_SHAPE;
    auto *c = new (std::nothrow) rg_comm();
    if (!c) return RG_ERR_CUDA;
    c->world = world, c->rank = rank;
    if (cudaGetDevice(&c->device) != cudaSuccess) {
        delete c;
        return RG_ERR_CUDA;
    }
    c->capacity = (capacity_bytes + 255) / 256 * 256;
    // [2 parities][world] slots A of 2 * capacity, then [2 parities] slots B (finished values of the two-shot variant)
    c->total_bytes = AR_HEADER_BYTES + 4 * static_cast<size_t>(world + 1) * c->capacity;
    c->wait_ns = 2000000000ull;
    void *p = nullptr;
    if (cudaMalloc(&p, c->total_bytes) != cudaSuccess) {
        delete c;
        return RG_ERR_CUDA;
    }
    c->mine = static_cast<uint8_t *>(p);
    cudaMemset(c->mine, 0, c->total_bytes);
    const unsigned long long one = 1;
    cudaMemcpy(c->mine, &one, sizeof(one), cudaMemcpyHostToDevice);// seq starts at 1, flags at 0
    cudaDeviceSynchronize();
    c->peers[rank] = c->mine;
    cudaIpcMemHandle_t h;
    std::memset(&h, 0, sizeof(h));
    if (world > 1 && cudaIpcGetMemHandle(&h, c->mine) != cudaSuccess) {
        cudaFree(c->mine);
        delete c;
        return RG_ERR_CUDA;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    std::memcpy(handle64, &h, 64);
    c->connected = world == 1;
    {
        std::lock_guard<std::mutex> lock(g_comms_mutex);
        g_comms.push_back(c);
    }
    *out = c;
    return RG_OK;
}

int rg_b200_comm_connect(rg_comm *c, const void *all_handles) {
    if (!c || !all_handles) return RG_ERR_NULL;
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const uint8_t *>(all_handles) + 64 * r, 64);
        void *p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return RG_ERR_CUDA;
        c->peers[r] = static_cast<uint8_t *>(p);
        c->opened[r] = true;
    }
    c->connected = true;
    return RG_OK;
}

// Same-process wiring (one thread per GPU, as the reference's own all-reduce test runs, or a test double for a
// peer): bases[r] is the value rg_b200_comm_base returned for rank r; peer access must already be enabled.
void *rg_b200_comm_base(rg_comm *c) { return c ? c->mine : nullptr; }
size_t rg_b200_comm_bytes(rg_comm *c) { return c ? c->total_bytes : 0; }
int rg_b200_comm_connect_ptrs(rg_comm *c, const void *const *bases) {
    if (!c || !bases) return RG_ERR_NULL;
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        if (!bases[r]) return RG_ERR_NULL;
        c->peers[r] = static_cast<uint8_t *>(const_cast<void *>(bases[r]));
    }
    c->connected = true;
    return RG_OK;
}

// Shortens the bounded wait (nanoseconds) so that a missing peer is reported quickly.
int rg_b200_comm_set_wait_ns(rg_comm *c, uint64_t ns) {
    if (!c) return RG_ERR_NULL;
    c->wait_ns = ns;
    return RG_OK;
}

int rg_b200_comm_status(rg_comm *c) {
    if (!c) return RG_ERR_NULL;
    if (cudaDeviceSynchronize() != cudaSuccess) return RG_ERR_CUDA;
    const int st = comm_read_status(c);
    if (st < 0) return RG_ERR_CUDA;
    return (st || c->failed) ? RG_ERR_TIMEOUT : RG_OK;
}

int rg_b200_comm_destroy(rg_comm *c) {
    if (!c) return RG_ERR_NULL;
    {
        std::lock_guard<std::mutex> lock(g_comms_mutex);
        for (size_t i = 0; i < g_comms.size(); ++i)
            if (g_comms[i] == c) {
                g_comms.erase(g_comms.begin() + static_cast<long>(i));
                break;
            }
    }
    cudaDeviceSynchronize();
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank && c->opened[r]) cudaIpcCloseMemHandle(c->peers[r]);
    cudaFree(c->mine);
    delete c;
    return RG_OK;
}

// every rank must take the same variant: it depends on the group size and on RG_B200_AR_ALGO (1 one-shot, 2 two-shot) only
static bool comm_two_shot(const rg_comm *c) {
    static const int algo_env = std::getenv("RG_B200_AR_ALGO") ? atoi(std::getenv("RG_B200_AR_ALGO")) : 0;
    // measured on 4 GPUs, 256 KiB per rank: one-shot 14.7 us, two-shot 12.4 us (tensor-parallel step 15.20 vs 14.93 ms)
    return c->world > 1 && (algo_env == 2 || (algo_env != 1 && c->world >= 4));
}

// x == nullptr: receive only (this rank's input already lies in its slots)
static int all_reduce_launch(rg_comm *c, const rg_all_reduce_params *p, const void *x, const void *res, void *y, void *stream) {
    if (!c->connected) return RG_ERR_UNSUPPORTED;
    if (p->op < 0 || p->op > 4) return RG_ERR_UNSUPPORTED;
    if (c->failed) return RG_ERR_TIMEOUT;// out of step with its peers since a wait expired: destroy and recreate
    size_t es;
    switch (p->dtype) {
        case RG_U8: case RG_I8: es = 1; break;
        case RG_FP16: case RG_BF16: es = 2; break;
        case RG_F32: case RG_I32: case RG_U32: es = 4; break;
        case RG_I64: case RG_F64: es = 8; break;
        default: return RG_ERR_DTYPE;
    }
    if (p->count == 0) return RG_OK;
    if (!x && (p->count * es) % 16 != 0) return RG_ERR_SHAPE;// an epilogue writes whole 16-byte chunks
    const size_t bytes = (p->count * es + 15) / 16 * 16;
    if (bytes > c->capacity) return RG_ERR_LIMIT;
    if ((x && !aligned16(x)) || !aligned16(y)) return RG_ERR_ALIGN;
    ArArgs a = {};
    a.mine = c->mine;
    for (int r = 0; r < c->world; ++r) a.peer[r] = c->peers[r];
    a.x = x, a.res = res, a.y = y;
    a.count = p->count, a.capacity = c->capacity;
    a.world = c->world, a.rank = c->rank, a.op = p->op;
    a.wait_ns = c->wait_ns;
    const uint64_t chunks = bytes / 16;
    // every rank derives the same grid from the same count: CTA c of one rank pairs with CTA c of the others
    uint64_t grid = (chunks + AR_THREADS - 1) / AR_THREADS;
    if (grid < 1) grid = 1;
    if (grid > 128) grid = 128;
    auto st = static_cast<cudaStream_t>(stream);
    const bool two_shot = comm_two_shot(c);
    const dim3 g(static_cast<unsigned>(grid)), b(AR_THREADS);
    cudaError_t e;
#define RG_AR(T) e = two_shot ? launch_pdl(all_reduce_two_shot_kernel<T>, g, b, 0, st, a) : launch_pdl(all_reduce_kernel<T>, g, b, 0, st, a)
    switch (p->dtype) {
        case RG_F32: RG_AR(float); break;
        case RG_FP16: RG_AR(__half); break;
        case RG_BF16: RG_AR(__nv_bfloat16); break;
        case RG_U8: RG_AR(uint8_t); break;
        case RG_I8: RG_AR(int8_t); break;
        case RG_I32: RG_AR(int32_t); break;
        case RG_U32: RG_AR(uint32_t); break;
        case RG_I64: RG_AR(long long); break;
        default: RG_AR(double); break;
    }
#undef RG_AR
    if (e != cudaSuccess) return RG_ERR_CUDA;
    count_launch();
    return launch_status();
}

int rg_b200_all_reduce(rg_comm *c, const rg_all_reduce_params *p, const void *const *in, void *const *out, void *stream) {
    if (!c || !p || !in || !out || !in[0] || !out[0]) return RG_ERR_NULL;
    return all_reduce_launch(c, p, in[0], in[1], out[0], stream);
}

int rg_b200_all_reduce_recv(rg_comm *c, const rg_all_reduce_params *p, const void *const *in, void *const *out, void *stream) {
    if (!c || !p || !out || !out[0]) return RG_ERR_NULL;
    return all_reduce_launch(c, p, nullptr, in ? in[0] : nullptr, out[0], stream);
}

int rg_b200_mat_mul_push(rg_comm *c, const rg_mat_mul_params *p, void *ws, const void *const *in, void *stream) {
    if (!c || !p || !in || !in[0] || !in[1]) return RG_ERR_NULL;
    if (!c->connected) return RG_ERR_UNSUPPORTED;
    if (c->failed) return RG_ERR_TIMEOUT;
    if (static_cast<size_t>(p->m) * p->n * 2 > c->capacity) return RG_ERR_LIMIT;
    ArPeers peers = {};
    peers.mine = c->mine;
    for (int r = 0; r < c->world; ++r) peers.peer[r] = c->peers[r];
    peers.capacity = c->capacity, peers.world = c->world, peers.rank = c->rank;
    peers.two_shot = comm_two_shot(c) ? 1 : 0;
    return gemm_tc_push(p, ws, in, peers, static_cast<cudaStream_t>(stream));
}

int rg_b200_all_reduce_norm(rg_comm *c, const rg_all_reduce_norm_params *p, const void *const *in, void *const *out, void *stream) {
    if (!c || !p || !in || !out || !in[0] || !in[2] || !out[0] || !out[1]) return RG_ERR_NULL;
    if (!c->connected) return RG_ERR_UNSUPPORTED;
    if (c->failed) return RG_ERR_TIMEOUT;
    if (p->dtype != RG_FP16 && p->dtype != RG_BF16) return RG_ERR_DTYPE;
    if (p->rows == 0 || p->dim == 0) return RG_OK;
    // the row lives in registers: 16-byte chunks, at most 8 per thread of a 256-thread CTA
    if (p->dim % 8 != 0 || p->dim > 8u * 8u * AR_THREADS || p->rows > 65535u) return RG_ERR_SHAPE;
    const size_t bytes = static_cast<size_t>(p->rows) * p->dim * 2;
    if (bytes > c->capacity) return RG_ERR_LIMIT;
    for (int i = 0; i < 3; ++i)
        if (in[i] && !aligned16(in[i])) return RG_ERR_ALIGN;
    if (!aligned16(out[0]) || !aligned16(out[1])) return RG_ERR_ALIGN;
    ArNormArgs a = {};
    a.a.mine = c->mine;
    for (int r = 0; r < c->world; ++r) a.a.peer[r] = c->peers[r];
    a.a.x = in[0], a.a.res = in[1], a.a.y = out[0];
    a.a.count = static_cast<uint64_t>(p->rows) * p->dim, a.a.capacity = c->capacity;
    a.a.world = c->world, a.a.rank = c->rank, a.a.op = 0;
    a.a.wait_ns = c->wait_ns;
    a.w = in[2], a.n = out[1], a.dim = p->dim, a.eps = p->epsilon;
    // chunks per thread and CTA size exactly as the RmsNormalization launcher picks them (same bits as the two-kernel form)
    const uint32_t chunks = p->dim / 8;
    uint32_t ch = (chunks + 255) / 256;
    ch = ch <= 1 ? 1 : ch <= 2 ? 2 : ch <= 4 ? 4 : 8;
    uint32_t threads = ((chunks + ch - 1) / ch + 31) / 32 * 32;
    if (threads > 256) threads = 256;
    if (threads < 32) threads = 32;
    const bool two = comm_two_shot(c);
    auto st = static_cast<cudaStream_t>(stream);
    const dim3 g(p->rows), b(threads);
    cudaError_t e = cudaSuccess;
#define RG_ARN2(T, CH) e = two ? launch_pdl(all_reduce_norm_kernel<T, CH, true>, g, b, 0, st, a) : launch_pdl(all_reduce_norm_kernel<T, CH, false>, g, b, 0, st, a)
#define RG_ARN(T)                                                                                                      \
    switch (ch) {                                                                                                      \
        case 1: RG_ARN2(T, 1); break;                                                                                  \
        case 2: RG_ARN2(T, 2); break;                                                                                  \
        case 4: RG_ARN2(T, 4); break;                                                                                  \
        default: RG_ARN2(T, 8); break;                                                                                 \
    }
    if (p->dtype == RG_FP16) {
        RG_ARN(__half)
    } else {
        RG_ARN(__nv_bfloat16)
    }
#undef RG_ARN
#undef RG_ARN2
    if (e != cudaSuccess) return RG_ERR_CUDA;
    count_launch();
    return launch_status();
}
}
