// Shared device/host helpers for the sm_100a kernels: dtype traits, 128-bit access, warp/block reductions,
// mbarrier + bulk-copy (TMA) PTX wrappers with bounded waits, programmatic dependent launch.
#pragma once
#include "../../include/rg_b200.h"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <cstdlib>
#include <utility>

namespace rg {

// ---- host side -------------------------------------------------------------------------------
void count_launch(unsigned n = 1);// bumps the process-wide launch counter (api.cu)
int sm_count();                   // multiProcessorCount of the current device (cached per device)

#define RG_CHECK_CUDA(expr)                          \
    do {                                             \
        cudaError_t _e = (expr);                     \
        if (_e != cudaSuccess) return RG_ERR_CUDA;   \
    } while (0)

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? RG_OK : RG_ERR_CUDA; }

// Reads (and optionally zeroes) one of the per-file `static __device__ int` error words.
template<class T> inline int error_symbol(const T &sym, bool clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, sym, sizeof(int)) != cudaSuccess) return -1;
    if (clear && v) {
        const int z = 0;
        if (cudaMemcpyToSymbol(sym, &z, sizeof(int)) != cudaSuccess) return -1;
    }
    return v;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- dtype traits ----------------------------------------------------------------------------
template<class T> struct Num;
template<> struct Num<float> {
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float v) { return v; }
};
template<> struct Num<__half> {
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template<> struct Num<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// 16-byte vector of T with fp32 unpack/pack.
template<class T> struct Vec16 {
    static constexpr int N = 16 / sizeof(T);
    uint4 raw;
    __device__ __forceinline__ void load(const T *p) { raw = *reinterpret_cast<const uint4 *>(p); }
    __device__ __forceinline__ void store(T *p) const { *reinterpret_cast<uint4 *>(p) = raw; }
    __device__ __forceinline__ void unpack(float (&f)[N]) const {
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int i = 0; i < N; ++i) f[i] = Num<T>::to_f(e[i]);
    }
    __device__ __forceinline__ void pack(const float (&f)[N]) {
        T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
        for (int i = 0; i < N; ++i) e[i] = Num<T>::from_f(f[i]);
    }
};

// 8 fp16/bf16 values held in a uint4 -> 8 floats
template<class T> __device__ __forceinline__ void unpack8(const uint4 &r, float (&f)[8]);
template<> __device__ __forceinline__ void unpack8<__half>(const uint4 &r, float (&f)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
template<> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4 &r, float (&f)[8]) {
    const uint32_t *w = reinterpret_cast<const uint32_t *>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// two fp16/bf16 values held in a 32-bit word -> two floats
template<class T> __device__ __forceinline__ float2 unpack2(uint32_t w);
template<> __device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
    __half2 h;
    *reinterpret_cast<uint32_t *>(&h) = w;
    return __half22float2(h);
}
template<> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
// D += A(16x16, row) * B(16x8, col) on the warp-level tensor path, 16-bit inputs, fp32 accumulators
template<class T> __device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template<> __device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template<> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- device-read indices ----------------------------------------------------------------------
// Positions, sequence lengths, token ids and block-table entries are read from device memory that a generation
// loop advances on its own, so no kernel trusts them: an index that does not fit its buffer is never used for an
// access.  The kernel records the fact in its file's index-error word (reported as bit 5 of rg_b200_error_state),
// skips the store (or clamps the read range) and carries on; nothing traps.
__device__ __forceinline__ bool kv_pos_ok(int64_t p, const rg_kv_layout &kv, bool paged) {
    if (p < 0) return false;
    if (paged) return kv.page_size != 0 && static_cast<uint64_t>(p) / kv.page_size < kv.max_blocks_per_seq;
    return static_cast<uint64_t>(p) < kv.max_seq;
}
__device__ __forceinline__ bool kv_block_ok(int32_t blk, const rg_kv_layout &kv) {
    return blk >= 0 && (kv.n_blocks == 0 || static_cast<uint32_t>(blk) < kv.n_blocks);
}
// The reference-layout operator's past_seq_len (a device scalar): negative counts as 0, anything beyond the cache as full.
__device__ __forceinline__ uint32_t past_clamped(const int64_t *p, uint32_t cap) {
    if (!p) return 0u;
    const int64_t v = *p;
    return v <= 0 ? 0u : (static_cast<uint64_t>(v) > cap ? cap : static_cast<uint32_t>(v));
}
// Number of cached tokens a decode kernel may read for a sequence whose device-side length is len64.
__device__ __forceinline__ uint32_t kv_len_clamped(int64_t len64, uint32_t max_len, const rg_kv_layout &kv, bool paged, int *err) {
    if (len64 <= 0) return 0u;
    uint64_t cap = max_len;
    const uint64_t room = paged ? static_cast<uint64_t>(kv.page_size) * kv.max_blocks_per_seq : kv.max_seq;
    if (room < cap) cap = room;
    if (static_cast<uint64_t>(len64) > cap) {
        *err = 1;
        return static_cast<uint32_t>(cap);
    }
    return static_cast<uint32_t>(len64);
}

// ---- reductions ------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide sum for blockDim.x <= 1024 (multiple of 32); `red` is >= 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// ---- PTX: shared addresses, mbarrier, bulk copy, PDL -----------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Wait for the phase with the given parity, for at most ~2 s of wall time.  Returns false on expiry (the
// caller records an error and leaves the kernel); never spins without a bound.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > 2000000000ull) return false;
    }
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted on `bar`.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// Same with an L2 eviction policy (weights are read once per step: evict-first keeps L2 for activations).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void bulk_g2s_hint(void *dst, const void *src, uint32_t bytes, uint64_t *bar,
                                              uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
            "r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
// Programmatic dependent launch: wait for the producer grid's memory to be visible / let dependents start.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// First statement of a kernel launched through launch_pdl: lets the next kernel of the stream be scheduled, then waits
// until the previous one has completed and its writes are visible.  Everything before the call overlaps the predecessor.
__device__ __forceinline__ void pdl_enter() {
    pdl_launch_dependents();
    pdl_wait();
}
// RG_B200_PDL=0 turns programmatic dependent launch off (every kernel then waits for its predecessor to drain).
inline bool pdl_enabled() {
    static const bool on = [] {
        const char *e = std::getenv("RG_B200_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}
// Launch with the programmatic-stream-serialization attribute: the kernel may start while its predecessor in the stream is
// still running and must call pdl_enter() (or pdl_wait()) before it touches anything the predecessor wrote.
template<class... K, class... A>
inline cudaError_t launch_pdl(void (*kern)(K...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, std::forward<A>(args)...);
}
// The same for a kernel whose CTAs form clusters of `cluster_x` consecutive CTAs (grid.x a multiple of it)
template<class... K, class... A>
inline cudaError_t launch_pdl_cluster(void (*kern)(K...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, unsigned cluster_x, A &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kern, std::forward<A>(args)...);
}

}// namespace rg
