// TopK and top-k sampling over vocabulary-sized rows (no reference counterpart; the ordering rule is
// "value descending, ties by lower index, NaN below every number").
//
// One CTA per row.  The row is turned into order-preserving 32-bit keys staged in shared memory (one HBM read),
// the k-th largest key is found by an MSB-first radix select (4 passes of 8 bits with shared-memory
// histograms); if the k-th key is tied, four more passes over ~index pick the lowest indices, so the
// selection is a radix select over the distinct 64-bit composite (key, ~index) and is deterministic.
// The k winners are then rank-sorted and written out.
#include "common.cuh"

namespace rg {

constexpr int TOPK_MAX = 64;
constexpr int TOPK_THREADS = 1024;
constexpr uint32_t TOPK_STAGE_MAX = 40960;// keys staged in smem (160 KiB)

template<class T> __device__ __forceinline__ uint32_t key_of(T v) {
    const float f = Num<T>::to_f(v);
    if (f != f) return 0u;
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float float_of_key(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct TopkShared {
    uint32_t hist[256];
    uint32_t bin, kk, cnt_eq, count;
    uint32_t cand_key[TOPK_MAX];
    uint32_t cand_idx[TOPK_MAX];
    uint32_t sort_key[TOPK_MAX];
    uint32_t sort_idx[TOPK_MAX];
    float red[33];
};

// Selects the k largest (key, ~idx) composites of the row into sh.sort_key/sort_idx (descending).
// `skeys` holds the staged keys when staged != 0, else keys are recomputed from x.
template<class T>
__device__ void topk_select(const T *__restrict__ xr, uint32_t n, uint32_t k, uint32_t *skeys, bool staged,
                            TopkShared &sh) {
    const uint32_t tid = threadIdx.x, nt = blockDim.x;
    if (staged)
        for (uint32_t i = tid; i < n; i += nt) skeys[i] = key_of<T>(xr[i]);
    __syncthreads();
    auto key_at = [&](uint32_t i) -> uint32_t { return staged ? skeys[i] : key_of<T>(xr[i]); };

    uint32_t prefix = 0, mask = 0, prefix2 = 0, mask2 = 0, kk = k;
    bool tie_break = false;
    for (int pass = 0; pass < 8; ++pass) {
        const int shift = 24 - 8 * (pass & 3);
        for (uint32_t b = tid; b < 256; b += nt) sh.hist[b] = 0;
        __syncthreads();
        if (pass < 4) {
            for (uint32_t i = tid; i < n; i += nt) {
                const uint32_t key = key_at(i);
                if ((key & mask) == prefix) atomicAdd(&sh.hist[(key >> shift) & 255u], 1u);
            }
        } else {
            for (uint32_t i = tid; i < n; i += nt) {
                const uint32_t key = key_at(i), inv = ~i;
                if (key == prefix && (inv & mask2) == prefix2) atomicAdd(&sh.hist[(inv >> shift) & 255u], 1u);
            }
        }
        __syncthreads();
        if (tid < 32) {
            // lane L owns bins 255-8L .. 248-8L (descending); find the bin holding the kk-th largest
            uint32_t local = 0;
            const int top = 255 - 8 * static_cast<int>(tid);
#pragma unroll
            for (int j = 0; j < 8; ++j) local += sh.hist[top - j];
            uint32_t incl = local;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                if (static_cast<int>(tid) >= o) incl += t;
            }
            const uint32_t excl = incl - local;
            if (excl < kk && kk <= incl) {
                uint32_t above = excl;
                for (int j = 0; j < 8; ++j) {
                    const uint32_t c = sh.hist[top - j];
                    if (above + c >= kk) {
                        sh.bin = static_cast<uint32_t>(top - j);
                        sh.kk = kk - above;
                        sh.cnt_eq = c;
                        break;
                    }
                    above += c;
                }
            }
        }
        __syncthreads();
        kk = sh.kk;
        if (pass < 4) {
            prefix |= sh.bin << shift;
            mask |= 255u << shift;
            if (pass == 3) {
                if (sh.cnt_eq == kk) break;// every element equal to the k-th key is taken
                tie_break = true;
            }
        } else {
            prefix2 |= sh.bin << shift;
            mask2 |= 255u << shift;
        }
        __syncthreads();
    }
    __syncthreads();
    if (tid == 0) sh.count = 0;
    __syncthreads();
    for (uint32_t i = tid; i < n; i += nt) {
        const uint32_t key = key_at(i);
        const bool take = key > prefix || (key == prefix && (!tie_break || (~i) >= prefix2));
        if (take) {
            const uint32_t pos = atomicAdd(&sh.count, 1u);
            if (pos < TOPK_MAX) {
                sh.cand_key[pos] = key;
                sh.cand_idx[pos] = i;
            }
        }
    }
    __syncthreads();
    const uint32_t cnt = sh.count < k ? sh.count : k;
    if (tid < cnt) {
        const uint32_t mk = sh.cand_key[tid], mi = sh.cand_idx[tid];
        uint32_t rank = 0;
        for (uint32_t j = 0; j < cnt; ++j) {
            const uint32_t ok = sh.cand_key[j], oi = sh.cand_idx[j];
            rank += (ok > mk || (ok == mk && oi < mi)) ? 1u : 0u;
        }
        sh.sort_key[rank] = mk;
        sh.sort_idx[rank] = mi;
    }
    __syncthreads();
}

template<class T, bool SOFTMAX>
__global__ void __launch_bounds__(TOPK_THREADS) topk_kernel(const T *__restrict__ x, void *__restrict__ values,
                                                            int64_t *__restrict__ indices, uint32_t n, uint32_t k,
                                                            int staged) {
    pdl_enter();
    extern __shared__ __align__(16) uint32_t skeys[];
    __shared__ TopkShared sh;
    const T *xr = x + static_cast<size_t>(blockIdx.x) * n;
    topk_select<T>(xr, n, k, skeys, staged != 0, sh);
    float inv_sum = 0.f, mx = 0.f;
    if constexpr (SOFTMAX) {
        mx = float_of_key(sh.sort_key[0]);
        float s = 0.f;
        for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
            const float f = staged ? float_of_key(skeys[i]) : Num<T>::to_f(xr[i]);
            if (f == f) s += expf(f - mx);
        }
        s = block_sum(s, sh.red);
        inv_sum = 1.f / s;
    }
    if (threadIdx.x < k) {
        const uint32_t idx = sh.sort_idx[threadIdx.x];
        const size_t o = static_cast<size_t>(blockIdx.x) * k + threadIdx.x;
        indices[o] = static_cast<int64_t>(idx);
        if constexpr (SOFTMAX) static_cast<float *>(values)[o] = expf(Num<T>::to_f(xr[idx]) - mx) * inv_sum;
        else
            static_cast<T *>(values)[o] = xr[idx];
    }
}

// Philox-4x32-10 (Salmon, Moraes, Dror, Shaw, "Parallel random numbers: as easy as 1, 2, 3", SC'11).
__device__ __forceinline__ uint32_t philox_u32(uint64_t seed, uint32_t row, uint64_t step) {
    uint32_t c0 = row, c1 = 0u, c2 = static_cast<uint32_t>(step), c3 = static_cast<uint32_t>(step >> 32);
    uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0, c1 = n1, c2 = n2, c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c0;
}

template<class T>
__global__ void __launch_bounds__(TOPK_THREADS) topk_sample_kernel(const T *__restrict__ x,
                                                                   const uint64_t *__restrict__ step,
                                                                   int64_t *__restrict__ token, uint32_t n, uint32_t k,
                                                                   float inv_temp, uint64_t seed, int staged) {
    pdl_enter();
    extern __shared__ __align__(16) uint32_t skeys[];
    __shared__ TopkShared sh;
    const T *xr = x + static_cast<size_t>(blockIdx.x) * n;
    topk_select<T>(xr, n, k, skeys, staged != 0, sh);
    if (threadIdx.x == 0) {
        const float x0 = float_of_key(sh.sort_key[0]);
        float total = 0.f;
        for (uint32_t j = 0; j < k; ++j) total += expf((float_of_key(sh.sort_key[j]) - x0) * inv_temp);
        const uint32_t r = philox_u32(seed, blockIdx.x, *step);
        const float u = static_cast<float>(r >> 8) * (1.0f / 16777216.0f);
        const float target = u * total;
        float cum = 0.f;
        uint32_t pick = k - 1;
        for (uint32_t j = 0; j < k; ++j) {
            cum += expf((float_of_key(sh.sort_key[j]) - x0) * inv_temp);
            if (cum > target) {
                pick = j;
                break;
            }
        }
        token[blockIdx.x] = static_cast<int64_t>(sh.sort_idx[pick]);
    }
}

static uint32_t topk_threads(uint32_t n) {
    uint32_t t = (n + 31) / 32 * 32;
    if (t > TOPK_THREADS) t = TOPK_THREADS;
    if (t < 64) t = 64;
    return t;
}

template<class T>
static int topk_launch(const rg_topk_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    const int staged = p->n <= TOPK_STAGE_MAX;
    const size_t smem = staged ? static_cast<size_t>(p->n) * 4 : 0;
    auto x = static_cast<const T *>(in[0]);
    auto idx = static_cast<int64_t *>(out[1]);
    if (p->softmax) {
        RG_CHECK_CUDA(cudaFuncSetAttribute(topk_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 163840));
        launch_pdl(topk_kernel<T, true>, dim3(p->rows), dim3(topk_threads(p->n)), smem, st, x, out[0], idx, p->n, p->k, staged);
    } else {
        RG_CHECK_CUDA(cudaFuncSetAttribute(topk_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 163840));
        launch_pdl(topk_kernel<T, false>, dim3(p->rows), dim3(topk_threads(p->n)), smem, st, x, out[0], idx, p->n, p->k, staged);
    }
    count_launch();
    return launch_status();
}

template<class T>
static int topk_sample_launch(const rg_topk_sample_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    const int staged = p->n <= TOPK_STAGE_MAX;
    const size_t smem = staged ? static_cast<size_t>(p->n) * 4 : 0;
    RG_CHECK_CUDA(cudaFuncSetAttribute(topk_sample_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 163840));
    launch_pdl(topk_sample_kernel<T>, dim3(p->rows), dim3(topk_threads(p->n)), smem, st, 
        static_cast<const T *>(in[0]), static_cast<const uint64_t *>(in[1]), static_cast<int64_t *>(out[0]), p->n, p->k,
        1.0f / p->temperature, p->seed, staged);
    count_launch();
    return launch_status();
}

}// namespace rg

using namespace rg;

extern "C" {

size_t rg_b200_topk_workspace(const rg_topk_params *) { return 0; }
int rg_b200_topk(const rg_topk_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !out[0] || !out[1]) return RG_ERR_NULL;
    if (p->k == 0 || p->k > TOPK_MAX || p->k > p->n) return RG_ERR_SHAPE;
    if (p->rows == 0) return RG_OK;
    auto st = static_cast<cudaStream_t>(stream);
    switch (p->dtype) {
        case RG_F32: return topk_launch<float>(p, in, out, st);
        case RG_FP16: return topk_launch<__half>(p, in, out, st);
        case RG_BF16: return topk_launch<__nv_bfloat16>(p, in, out, st);
        default: return RG_ERR_DTYPE;
    }
}

size_t rg_b200_topk_sample_workspace(const rg_topk_sample_params *) { return 0; }
int rg_b200_topk_sample(const rg_topk_sample_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !in[1] || !out[0]) return RG_ERR_NULL;
    if (p->k == 0 || p->k > TOPK_MAX || p->k > p->n || !(p->temperature > 0.f)) return RG_ERR_SHAPE;
    if (p->rows == 0) return RG_OK;
    auto st = static_cast<cudaStream_t>(stream);
    switch (p->dtype) {
        case RG_F32: return topk_sample_launch<float>(p, in, out, st);
        case RG_FP16: return topk_sample_launch<__half>(p, in, out, st);
        case RG_BF16: return topk_sample_launch<__nv_bfloat16>(p, in, out, st);
        default: return RG_ERR_DTYPE;
    }
}
}
