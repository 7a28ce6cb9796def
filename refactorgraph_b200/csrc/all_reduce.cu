// AllReduce across the GPUs of one NVSwitch box, one process per GPU.  Replaces AllReduceNccl + NcclCommunicator
// (src/04kernel/src/kernels/all_reduce/nccl_kernel.cu:9-19, src/04kernel/src/utilities/cuda/nccl_communicator.cu:11-44).
//
// One-shot pull over peer memory: every rank owns a "symmetric" allocation (header, per-CTA flags, two data slots)
// that its peers map through CUDA IPC.  Call number s (kept in device memory, so a captured CUDA graph can replay
// it): CTA c of every rank copies its 16-byte chunks of the input into slot s&1 of its own allocation, publishes
// flags[c] = s with a system-scope release, waits (bounded) until flags[c] >= s is visible in every peer's
// allocation, then loads the same chunks from all ranks with plain 128-bit loads, combines them in fp32 in rank
// order (so all ranks get bit-identical results) and writes the output.  Slot s&1 is not rewritten before call
// s+2, which cannot start on any rank before every rank has finished call s+1's wait, i.e. finished reading
// call s.  No TMA and no multicast instructions touch peer memory.
#include "gemm_dispatch.cuh"
#include <cstring>
#include <new>

namespace rg {

constexpr int AR_MAX_RANKS = 8;
constexpr int AR_MAX_CTAS = 512;
constexpr int AR_THREADS = 256;
constexpr size_t AR_HEADER_BYTES = 4096;
constexpr size_t AR_FLAGS_BYTES = AR_MAX_CTAS * sizeof(unsigned long long);

struct ArHeader {
    unsigned long long seq;// number of the call in flight (starts at 1)
    unsigned int done;     // CTAs of the current call that have read seq
    int status;            // 0 ok; 1 = a wait on a peer flag expired
};

struct ArArgs {
    uint8_t *mine;
    const uint8_t *peer[AR_MAX_RANKS];// peer[rank] = mine
    const void *x, *res;
    void *y;
    uint64_t count;
    size_t capacity;
    int world, rank, op;
    uint64_t wait_ns;
};

__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ar_combine(int op, float a, float b) {
    switch (op) {
        case 2: return fminf(a, b);
        case 3: return fmaxf(a, b);
        case 4: return a * b;
        default: return a + b;
    }
}

template<class T>
__global__ void __launch_bounds__(AR_THREADS) all_reduce_kernel(const ArArgs a) {
    pdl_enter();
    constexpr int N = Vec16<T>::N;
    ArHeader *hdr = reinterpret_cast<ArHeader *>(a.mine);
    unsigned long long *my_flags = reinterpret_cast<unsigned long long *>(a.mine + AR_HEADER_BYTES);
    __shared__ unsigned long long s_seq;
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        s_seq = *reinterpret_cast<volatile unsigned long long *>(&hdr->seq);
        s_ok = 1;
    }
    __syncthreads();
    const unsigned long long seq = s_seq;
    const size_t slot_off = AR_HEADER_BYTES + AR_FLAGS_BYTES + (seq & 1ull) * a.capacity;
    const uint64_t chunks = (a.count + N - 1) / N;// the last chunk may run past count: buffers are padded to 16 B
    const uint64_t per = (chunks + gridDim.x - 1) / gridDim.x;
    const uint64_t c0 = per * blockIdx.x, c1 = c0 + per < chunks ? c0 + per : chunks;
    const T *x = static_cast<const T *>(a.x);
    const T *res = static_cast<const T *>(a.res);
    T *y = static_cast<T *>(a.y);
    T *slot = reinterpret_cast<T *>(a.mine + slot_off);
    const uint64_t full_chunks = a.count / N;

    // 1. publish my part of the input
    for (uint64_t c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        if (c < full_chunks) {
            *reinterpret_cast<uint4 *>(slot + c * N) = *reinterpret_cast<const uint4 *>(x + c * N);
        } else {
            for (uint64_t e = c * N; e < a.count; ++e) slot[e] = x[e];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        st_release_sys(&my_flags[blockIdx.x], seq);
        // the last CTA to have read seq advances it for the next call
        if (atomicAdd(&hdr->done, 1u) == gridDim.x - 1) {
            hdr->done = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned long long *>(&hdr->seq) = seq + 1;
        }
    }
    // 2. wait for the same part of every peer (bounded)
    if (threadIdx.x < static_cast<unsigned>(a.world) && static_cast<int>(threadIdx.x) != a.rank) {
        const unsigned long long *pf = reinterpret_cast<const unsigned long long *>(a.peer[threadIdx.x] + AR_HEADER_BYTES) + blockIdx.x;
        const uint64_t t0 = global_timer_ns();
        bool ok = false;
        for (;;) {
            if (ld_acquire_sys(pf) >= seq) {
                ok = true;
                break;
            }
            if (global_timer_ns() - t0 > a.wait_ns) break;
        }
        if (!ok) {
            s_ok = 0;
            hdr->status = 1;
        }
    }
    __syncthreads();
    if (!s_ok) return;// leave the output untouched; the host sees the status word
    // 3. pull and combine in rank order
    const float scale = a.op == 1 ? 1.0f / static_cast<float>(a.world) : 1.0f;
    for (uint64_t c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float acc[N];
#pragma unroll
        for (int r = 0; r < AR_MAX_RANKS; ++r) {
            if (r < a.world) {
                const T *src = reinterpret_cast<const T *>(a.peer[r] + slot_off) + c * N;
                Vec16<T> v;
                v.raw = *reinterpret_cast<const uint4 *>(src);
                float f[N];
                v.unpack(f);
#pragma unroll
                for (int j = 0; j < N; ++j) acc[j] = r == 0 ? f[j] : ar_combine(a.op, acc[j], f[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] *= scale;
        if (res) {
            // the reduced value is rounded to the storage type before the residual is added, exactly as if the
            // all-reduce and the Add were two operators
            for (int j = 0; j < N; ++j) {
                const uint64_t e = c * N + j;
                if (e < a.count) acc[j] = Num<T>::to_f(Num<T>::from_f(acc[j])) + Num<T>::to_f(res[e]);
            }
        }
        if (c < full_chunks) {
            Vec16<T> o;
            o.pack(acc);
            o.store(y + c * N);
        } else {
            for (uint64_t e = c * N; e < a.count; ++e) y[e] = Num<T>::from_f(acc[e - c * N]);
        }
    }
}

int all_reduce_error_word() { return 0; }// per-communicator status words are read by rg_b200_comm_status

}// namespace rg

using namespace rg;

struct rg_comm {
    int world, rank;
    size_t capacity, total_bytes;
    uint8_t *mine;
    uint8_t *peers[AR_MAX_RANKS];
    bool opened[AR_MAX_RANKS];
    bool connected;
    uint64_t wait_ns;
};

extern "C" {

int rg_b200_comm_create(int world, int rank, size_t capacity_bytes, rg_comm **out, void *handle64) {
    if (!out || !handle64) return RG_ERR_NULL;
    if (world < 1 || world > AR_MAX_RANKS || rank < 0 || rank >= world) return RG_ERR_SHAPE;
    auto *c = new (std::nothrow) rg_comm();
    if (!c) return RG_ERR_CUDA;
    c->world = world, c->rank = rank;
    c->capacity = (capacity_bytes + 255) / 256 * 256;
    c->total_bytes = AR_HEADER_BYTES + AR_FLAGS_BYTES + 2 * c->capacity;
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
    int st = 0;
    if (cudaMemcpy(&st, c->mine + offsetof(ArHeader, status), sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return RG_ERR_CUDA;
    return st ? RG_ERR_TIMEOUT : RG_OK;
}

int rg_b200_comm_destroy(rg_comm *c) {
    if (!c) return RG_ERR_NULL;
    cudaDeviceSynchronize();
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank && c->opened[r]) cudaIpcCloseMemHandle(c->peers[r]);
    cudaFree(c->mine);
    delete c;
    return RG_OK;
}

int rg_b200_all_reduce(rg_comm *c, const rg_all_reduce_params *p, const void *const *in, void *const *out, void *stream) {
    if (!c || !p || !in || !out || !in[0] || !out[0]) return RG_ERR_NULL;
    if (!c->connected) return RG_ERR_UNSUPPORTED;
    if (p->op < 0 || p->op > 4) return RG_ERR_UNSUPPORTED;
    size_t es;
    switch (p->dtype) {
        case RG_F32: es = 4; break;
        case RG_FP16: case RG_BF16: es = 2; break;
        default: return RG_ERR_DTYPE;
    }
    if (p->count == 0) return RG_OK;
    const size_t bytes = (p->count * es + 15) / 16 * 16;
    if (bytes > c->capacity) return RG_ERR_LIMIT;
    if (!aligned16(in[0]) || !aligned16(out[0])) return RG_ERR_ALIGN;
    ArArgs a = {};
    a.mine = c->mine;
    for (int r = 0; r < c->world; ++r) a.peer[r] = c->peers[r];
    a.x = in[0], a.res = in[1], a.y = out[0];
    a.count = p->count, a.capacity = c->capacity;
    a.world = c->world, a.rank = c->rank, a.op = p->op;
    a.wait_ns = c->wait_ns;
    const uint64_t chunks = bytes / 16;
    // every rank derives the same grid from the same count: CTA c of one rank pairs with CTA c of the others
    uint64_t grid = (chunks + AR_THREADS * 2 - 1) / (AR_THREADS * 2);
    if (grid < 1) grid = 1;
    if (grid > 128) grid = 128;
    auto st = static_cast<cudaStream_t>(stream);
    switch (p->dtype) {
        case RG_F32: launch_pdl(all_reduce_kernel<float>, dim3(static_cast<unsigned>(grid)), dim3(AR_THREADS), 0, st, a); break;
        case RG_FP16: launch_pdl(all_reduce_kernel<__half>, dim3(static_cast<unsigned>(grid)), dim3(AR_THREADS), 0, st, a); break;
        default: launch_pdl(all_reduce_kernel<__nv_bfloat16>, dim3(static_cast<unsigned>(grid)), dim3(AR_THREADS), 0, st, a); break;
    }
    count_launch();
    return launch_status();
}
}
