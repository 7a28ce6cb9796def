// RMSNorm and Softmax for sm_100a: HBM-bound row kernels with 128-bit accesses, fp32 statistics and
// warp-shuffle reductions.  Semantics follow RmsNormalizationCpu
// (src/04kernel/src/kernels/rms_normalization/cpu_kernel.cc:41-66) and the reference's CUDA softmax
// (src/04kernel/src/kernels/softmax/cuda_kernel.cu:21-105).
#include "common.cuh"

namespace rg {

// ---------------------------------------------------------------------------------------------
// RMSNorm.  One CTA per row; each thread keeps CH 16-byte chunks of the row in registers so x is read from
// HBM exactly once.  Optional residual add (s = x + r is written back and normalised).
template<class T, int CH, bool RES>
__global__ void __launch_bounds__(256) rms_norm_vec_kernel(const T *__restrict__ x, const T *__restrict__ w,
                                                           const T *__restrict__ r, T *__restrict__ y,
                                                           T *__restrict__ s, uint32_t dim, float eps) {
    pdl_enter();
    constexpr int N = Vec16<T>::N;
    __shared__ float red[33];
    const size_t row = blockIdx.x;
    const uint32_t chunks = dim / N;
    const T *xr = x + row * dim;
    float v[CH][N];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const uint32_t c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            Vec16<T> a;
            a.load(xr + c * N);
            a.unpack(v[i]);
            if constexpr (RES) {
                Vec16<T> b;
                float rb[N];
                b.load(r + row * dim + c * N);
                b.unpack(rb);
#pragma unroll
                for (int j = 0; j < N; ++j) v[i][j] += rb[j];
                // the stored sum is what the next layer reads, so normalise the rounded value
                a.pack(v[i]);
                a.store(s + row * dim + c * N);
                a.unpack(v[i]);
            }
#pragma unroll
            for (int j = 0; j < N; ++j) ss += v[i][j] * v[i][j];
        }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / static_cast<float>(dim) + eps);
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
            o.store(y + row * dim + c * N);
        }
    }
}

// Any dim / alignment: scalar accesses, x read twice (the second read hits L2).
template<class T, bool RES>
__global__ void rms_norm_scalar_kernel(const T *__restrict__ x, const T *__restrict__ w, const T *__restrict__ r,
                                       T *__restrict__ y, T *__restrict__ s, uint32_t dim, float eps) {
    pdl_enter();
    __shared__ float red[33];
    const size_t row = blockIdx.x;
    float ss = 0.f;
    for (uint32_t j = threadIdx.x; j < dim; j += blockDim.x) {
        float v = Num<T>::to_f(x[row * dim + j]);
        if constexpr (RES) {
            v += Num<T>::to_f(r[row * dim + j]);
            T sv = Num<T>::from_f(v);
            s[row * dim + j] = sv;
            v = Num<T>::to_f(sv);
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / static_cast<float>(dim) + eps);
    for (uint32_t j = threadIdx.x; j < dim; j += blockDim.x) {
        const float v = RES ? Num<T>::to_f(s[row * dim + j]) : Num<T>::to_f(x[row * dim + j]);
        y[row * dim + j] = Num<T>::from_f(v * rstd * Num<T>::to_f(w[j]));
    }
}

template<class T, bool RES>
static int rms_norm_launch(const rg_rms_norm_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    constexpr int N = Vec16<T>::N;
    auto x = static_cast<const T *>(in[0]);
    auto w = static_cast<const T *>(in[1]);
    auto r = RES ? static_cast<const T *>(in[2]) : nullptr;
    auto y = static_cast<T *>(out[0]);
    auto s = RES ? static_cast<T *>(out[1]) : nullptr;
    const bool vec = p->dim % N == 0 && aligned16(x) && aligned16(w) && aligned16(y) && (!RES || (aligned16(r) && aligned16(s)));
    const uint32_t chunks = p->dim / N;
    if (vec && chunks <= 256 * 8) {
        uint32_t ch = (chunks + 255) / 256;
        ch = ch <= 1 ? 1 : ch <= 2 ? 2 : ch <= 4 ? 4 : 8;
        uint32_t threads = ((chunks + ch - 1) / ch + 31) / 32 * 32;
        if (threads > 256) threads = 256;
        if (threads < 32) threads = 32;
        switch (ch) {
            case 1: launch_pdl(rms_norm_vec_kernel<T, 1, RES>, dim3(p->rows), dim3(threads), 0, st, x, w, r, y, s, p->dim, p->epsilon); break;
            case 2: launch_pdl(rms_norm_vec_kernel<T, 2, RES>, dim3(p->rows), dim3(threads), 0, st, x, w, r, y, s, p->dim, p->epsilon); break;
            case 4: launch_pdl(rms_norm_vec_kernel<T, 4, RES>, dim3(p->rows), dim3(threads), 0, st, x, w, r, y, s, p->dim, p->epsilon); break;
            default: launch_pdl(rms_norm_vec_kernel<T, 8, RES>, dim3(p->rows), dim3(threads), 0, st, x, w, r, y, s, p->dim, p->epsilon); break;
        }
    } else {
        uint32_t threads = p->dim >= 1024 ? 256 : ((p->dim + 31) / 32 * 32 > 256 ? 256 : (p->dim + 31) / 32 * 32);
        launch_pdl(rms_norm_scalar_kernel<T, RES>, dim3(p->rows), dim3(threads), 0, st, x, w, r, y, s, p->dim, p->epsilon);
    }
    count_launch();
    return launch_status();
}

// ---------------------------------------------------------------------------------------------
// Softmax, post == 1: one CTA per row.  Pass 1: online (max, sum) per thread over 16-byte chunks, merged
// with warp shuffles; pass 2 re-reads the row (L1/L2 resident for vocabulary-sized rows) and writes.
struct MaxSum {
    float m, s;
};
__device__ __forceinline__ MaxSum ms_merge(MaxSum a, MaxSum b) {
    if (b.m > a.m) {
        MaxSum t = a;
        a = b;
        b = t;
    }
    // a.m >= b.m ; exp(-inf - -inf) guarded
    const float e = (b.m == -INFINITY) ? 0.f : expf(b.m - a.m);
    return {a.m, a.s + b.s * e};
}
__device__ __forceinline__ MaxSum ms_add(MaxSum a, float v) {
    if (v > a.m) {
        const float e = (a.m == -INFINITY) ? 0.f : expf(a.m - v);
        return {v, a.s * e + 1.f};
    }
    return {a.m, a.s + expf(v - a.m)};
}
__device__ __forceinline__ MaxSum ms_block(MaxSum v, MaxSum *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxSum t{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
        v = ms_merge(v, t);
    }
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        MaxSum t = lane < nw ? red[lane] : MaxSum{-INFINITY, 0.f};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            MaxSum u{__shfl_xor_sync(0xffffffffu, t.m, o), __shfl_xor_sync(0xffffffffu, t.s, o)};
            t = ms_merge(t, u);
        }
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

template<class T, bool VEC>
__global__ void softmax_row_kernel(const T *__restrict__ x, T *__restrict__ y, uint32_t n) {
    constexpr int N = Vec16<T>::N;
    __shared__ MaxSum red[33];
    const T *xr = x + static_cast<size_t>(blockIdx.x) * n;
    T *yr = y + static_cast<size_t>(blockIdx.x) * n;
    MaxSum acc{-INFINITY, 0.f};
    if constexpr (VEC) {
        for (uint32_t c = threadIdx.x; c < n / N; c += blockDim.x) {
            Vec16<T> a;
            float f[N];
            a.load(xr + c * N);
            a.unpack(f);
#pragma unroll
            for (int j = 0; j < N; ++j) acc = ms_add(acc, f[j]);
        }
    } else {
        for (uint32_t j = threadIdx.x; j < n; j += blockDim.x) acc = ms_add(acc, Num<T>::to_f(xr[j]));
    }
    acc = ms_block(acc, red);
    const float inv = 1.f / acc.s;
    if constexpr (VEC) {
        for (uint32_t c = threadIdx.x; c < n / N; c += blockDim.x) {
            Vec16<T> a;
            float f[N];
            a.load(xr + c * N);
            a.unpack(f);
#pragma unroll
            for (int j = 0; j < N; ++j) f[j] = expf(f[j] - acc.m) * inv;
            a.pack(f);
            a.store(yr + c * N);
        }
    } else {
        for (uint32_t j = threadIdx.x; j < n; j += blockDim.x)
            yr[j] = Num<T>::from_f(expf(Num<T>::to_f(xr[j]) - acc.m) * inv);
    }
}

// post == 1, rows of up to 8192 16-byte chunks: the row lives in registers (CH chunks per thread), so it is read once and
// every element costs one exponential: maximum, then exp and sum, then the scaled store.  (The online kernel above pays two
// exponentials per element and reads the row twice: on [65536, 2048] fp16 it measured 289 us, issue-bound at 93 % SM throughput.)
template<class T, int CH>
__global__ void __launch_bounds__(1024) softmax_row_reg_kernel(const T *__restrict__ x, T *__restrict__ y, uint32_t n) {
    constexpr int N = Vec16<T>::N;
    __shared__ float red[33];
    const uint32_t chunks = n / N;
    const T *xr = x + static_cast<size_t>(blockIdx.x) * n;
    T *yr = y + static_cast<size_t>(blockIdx.x) * n;
    float v[CH][N];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const uint32_t c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            Vec16<T> a;
            a.load(xr + c * N);
            a.unpack(v[i]);
#pragma unroll
            for (int j = 0; j < N; ++j) m = fmaxf(m, v[i][j]);
        }
    }
    m = block_max(m, red);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const uint32_t c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
#pragma unroll
            for (int j = 0; j < N; ++j) {
                v[i][j] = expf(v[i][j] - m);// a row of -inf gives nan, as exp(x - max) / sum does in the reference
                s += v[i][j];
            }
        }
    }
    s = block_sum(s, red);
    const float inv = 1.f / s;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const uint32_t c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
#pragma unroll
            for (int j = 0; j < N; ++j) v[i][j] *= inv;
            Vec16<T> a;
            a.pack(v[i]);
            a.store(yr + c * N);
        }
    }
}

// post > 1: one thread per (pre, post) column, consecutive threads on consecutive `post` (coalesced).
template<class T>
__global__ void softmax_strided_kernel(const T *__restrict__ x, T *__restrict__ y, uint32_t pre, uint32_t mid,
                                       uint32_t post) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<size_t>(pre) * post) return;
    const size_t base = (i / post) * mid * post + (i % post);
    MaxSum acc{-INFINITY, 0.f};
    for (uint32_t j = 0; j < mid; ++j) acc = ms_add(acc, Num<T>::to_f(x[base + static_cast<size_t>(j) * post]));
    const float inv = 1.f / acc.s;
    for (uint32_t j = 0; j < mid; ++j) {
        const size_t k = base + static_cast<size_t>(j) * post;
        y[k] = Num<T>::from_f(expf(Num<T>::to_f(x[k]) - acc.m) * inv);
    }
}

template<class T>
static int softmax_launch(const rg_softmax_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    constexpr int N = Vec16<T>::N;
    auto x = static_cast<const T *>(in[0]);
    auto y = static_cast<T *>(out[0]);
    if (p->post == 1) {
        const bool vec = p->mid % N == 0 && aligned16(x) && aligned16(y);
        const uint32_t work = vec ? p->mid / N : p->mid;
        uint32_t threads = work >= 2048 ? 1024 : work >= 256 ? 256 : (work + 31) / 32 * 32;
        if (threads < 32) threads = 32;
        if (vec && work <= 8192) {
            uint32_t ch = (work + 1023) / 1024;
            ch = ch <= 1 ? 1 : ch <= 2 ? 2 : ch <= 4 ? 4 : 8;
            uint32_t t = ((work + ch - 1) / ch + 31) / 32 * 32;
            if (t < 32) t = 32;
            switch (ch) {
                case 1: softmax_row_reg_kernel<T, 1><<<p->pre, t, 0, st>>>(x, y, p->mid); break;
                case 2: softmax_row_reg_kernel<T, 2><<<p->pre, t, 0, st>>>(x, y, p->mid); break;
                case 4: softmax_row_reg_kernel<T, 4><<<p->pre, t, 0, st>>>(x, y, p->mid); break;
                default: softmax_row_reg_kernel<T, 8><<<p->pre, t, 0, st>>>(x, y, p->mid); break;
            }
        } else if (vec) softmax_row_kernel<T, true><<<p->pre, threads, 0, st>>>(x, y, p->mid);
        else
            softmax_row_kernel<T, false><<<p->pre, threads, 0, st>>>(x, y, p->mid);
    } else {
        const size_t cols = static_cast<size_t>(p->pre) * p->post;
        softmax_strided_kernel<T><<<static_cast<unsigned>((cols + 127) / 128), 128, 0, st>>>(x, y, p->pre, p->mid, p->post);
    }
    count_launch();
    return launch_status();
}

}// namespace rg

using namespace rg;

extern "C" {

size_t rg_b200_rms_norm_workspace(const rg_rms_norm_params *) { return 0; }
int rg_b200_rms_norm(const rg_rms_norm_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !in[1] || !out[0]) return RG_ERR_NULL;
    if (p->add_residual && (!in[2] || !out[1])) return RG_ERR_NULL;
    if (p->dim == 0) return RG_ERR_SHAPE;
    if (p->rows == 0) return RG_OK;
    auto st = static_cast<cudaStream_t>(stream);
#define RG_GO(T) (p->add_residual ? rms_norm_launch<T, true>(p, in, out, st) : rms_norm_launch<T, false>(p, in, out, st))
    switch (p->dtype) {
        case RG_F32: return RG_GO(float);
        case RG_FP16: return RG_GO(__half);
        case RG_BF16: return RG_GO(__nv_bfloat16);
        default: return RG_ERR_DTYPE;
    }
#undef RG_GO
}

size_t rg_b200_softmax_workspace(const rg_softmax_params *) { return 0; }
int rg_b200_softmax(const rg_softmax_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !out[0]) return RG_ERR_NULL;
    if (p->mid == 0) return RG_ERR_SHAPE;
    if (p->pre == 0 || p->post == 0) return RG_OK;
    auto st = static_cast<cudaStream_t>(stream);
    switch (p->dtype) {
        case RG_F32: return softmax_launch<float>(p, in, out, st);
        case RG_FP16: return softmax_launch<__half>(p, in, out, st);
        case RG_BF16: return softmax_launch<__nv_bfloat16>(p, in, out, st);
        default: return RG_ERR_DTYPE;
    }
}
}
