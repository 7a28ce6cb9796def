// General MatMul on CUDA cores: any transpose combination, batch strides with broadcast, bias, alpha/beta,
// fp32 accumulation.  This is the catch-all behind rg_b200_mat_mul (MatMulInfo semantics,
// src/04kernel/src/attributes/mat_mul_info.cc:27-42); the decoder's large and skinny GEMMs are routed to the
// tcgen05 and streaming kernels instead.
#include "common.cuh"
#include "gemm_dispatch.cuh"

namespace rg {

constexpr int TM = 64, TN = 64, TK = 16;

template<class T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T *__restrict__ A, const T *__restrict__ B,
                                                        const T *__restrict__ C, T *__restrict__ Y,
                                                        rg_mat_mul_params p) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];
    const uint32_t b = blockIdx.z;
    A += b * p.stride_a;
    B += b * p.stride_b;
    Y += b * p.stride_y;
    if (C) C += b * p.stride_c;
    const uint32_t m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const uint32_t tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    // element strides of op(A)[m,k] and op(B)[k,n]
    const uint64_t a_sm = p.trans_a ? 1 : p.k, a_sk = p.trans_a ? p.m : 1;
    const uint64_t b_sk = p.trans_b ? 1 : p.n, b_sn = p.trans_b ? p.k : 1;
    float acc[4][4] = {};
    for (uint32_t k0 = 0; k0 < p.k; k0 += TK) {
        // 64x16 tile of A and 16x64 tile of B: 1024 elements each, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t e = threadIdx.x + i * 256;
            uint32_t mm, kk;
            if (p.trans_a) mm = e % TM, kk = e / TM;
            else
                kk = e % TK, mm = e / TK;
            const uint32_t gm = m0 + mm, gk = k0 + kk;
            As[kk][mm] = (gm < p.m && gk < p.k) ? Num<T>::to_f(A[gm * a_sm + gk * a_sk]) : 0.f;
            uint32_t nn, kb;
            if (p.trans_b) kb = e % TK, nn = e / TK;
            else
                nn = e % TN, kb = e / TN;
            const uint32_t gn = n0 + nn, gkb = k0 + kb;
            Bs[kb][nn] = (gn < p.n && gkb < p.k) ? Num<T>::to_f(B[gkb * b_sk + gn * b_sn]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], bb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i], bb[i] = Bs[kk][tx * 4 + i];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t gm = m0 + ty * 4 + i;
        if (gm >= p.m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t gn = n0 + tx * 4 + j;
            if (gn >= p.n) continue;
            float v = p.alpha * acc[i][j];
            if (C) v += p.beta * Num<T>::to_f(C[static_cast<uint64_t>(gm) * p.bias_row_stride + static_cast<uint64_t>(gn) * p.bias_col_stride]);
            Y[static_cast<uint64_t>(gm) * p.n + gn] = Num<T>::from_f(v);
        }
    }
}

template<class T>
static int simt_launch(const rg_mat_mul_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    dim3 grid((p->n + TN - 1) / TN, (p->m + TM - 1) / TM, p->batch);
    gemm_simt_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T *>(in[0]), static_cast<const T *>(in[1]),
                                              p->has_bias ? static_cast<const T *>(in[2]) : nullptr,
                                              static_cast<T *>(out[0]), *p);
    count_launch();
    return launch_status();
}

int gemm_simt(const rg_mat_mul_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    switch (p->dtype) {
        case RG_F32: return simt_launch<float>(p, in, out, st);
        case RG_FP16: return simt_launch<__half>(p, in, out, st);
        case RG_BF16: return simt_launch<__nv_bfloat16>(p, in, out, st);
        default: return RG_ERR_DTYPE;
    }
}

}// namespace rg
