// Causal flash attention for prefill (head_dim 128, fp16 / bf16): the tensor-core path behind the Attention operator
// (semantics: src/08-01llm/README.md:29-63) for sequences longer than a few tokens.
//
// One CTA = 64 query rows of one (sequence, head); four warps of 16 rows.  K and V tiles of 64 keys are staged into
// shared memory with 16-byte cp.async (XOR-swizzled 16-byte chunks, double-buffered), S = Q K^T and O += P V run on
// mma.sync.m16n8k16 with fp32 accumulators, the softmax is the online (running max / sum) form in fp32 with exp2, P
// is re-used from the S accumulator registers as the A operand of the second product, and only the key blocks at or
// below the causal diagonal are visited.  Q / K / V / O are addressed through element strides, so the same kernel
// serves the reference layout [N, heads, S, D] and the token-major [N, S, heads, D] produced by a fused QKV GEMM.
// (The legacy warp-level MMA is used here; the GEMMs of the path run on tcgen05.)
#include "common.cuh"

namespace rg {

constexpr int PF_BM = 64, PF_BN = 64, PF_D = 128, PF_THREADS = 128;

struct PrefillArgs {
    const void *q, *k, *v;
    void *o;
    const int64_t *past;// device scalar or nullptr (= 0)
    int64_t q_sn, q_sh, q_st;// element strides: sequence, head, token (d is contiguous)
    int64_t k_sn, k_sh, k_st;
    int64_t v_sn, v_sh, v_st;
    int64_t o_sn, o_sh, o_st;
    uint32_t n_heads, n_kv, S, kv_cap;// kv_cap = tokens addressable in k/v per (sequence, head)
    float scale_log2e;
};

template<class T> struct Mma;
template<> struct Mma<__half> {
    static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
};
template<> struct Mma<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
    const int sz = valid ? 16 : 0;// src-size 0 = zero fill
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template<int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// byte offset of 16-byte chunk c of row r in a [rows][128 x 2 B] tile with the XOR swizzle
__device__ __forceinline__ uint32_t sw_off(uint32_t r, uint32_t c) { return r * 256u + ((c ^ (r & 7u)) << 4); }

template<class T>
__device__ __forceinline__ void load_tile(uint32_t smem_base, const T *src, int64_t row_stride, uint32_t row0, uint32_t rows_valid_end) {
    // 64 rows x 16 chunks, 8 chunks per thread; rows >= rows_valid_end are zero-filled
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t id = threadIdx.x + i * PF_THREADS, r = id >> 4, c = id & 15u;
        const bool valid = row0 + r < rows_valid_end;
        const T *p = src + static_cast<int64_t>(valid ? row0 + r : 0) * row_stride + c * 8;
        cp_async16(smem_base + sw_off(r, c), p, valid);
    }
}

template<class T>
__global__ void __launch_bounds__(PF_THREADS) attn_prefill_kernel(const PrefillArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sQ = smem_u32(smem), sK = sQ + 16384, sV = sK + 2 * 16384;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t qb = blockIdx.x, h = blockIdx.y, n = blockIdx.z;
    const uint32_t kvh = h / (a.n_heads / a.n_kv);
    const uint32_t past = past_clamped(a.past, a.kv_cap);
    const uint32_t q0 = qb * PF_BM;
    const uint32_t kv_len = past + a.S < a.kv_cap ? past + a.S : a.kv_cap;
    uint32_t last_key = past + q0 + PF_BM;// exclusive bound of keys any row of this tile may see
    if (last_key > kv_len) last_key = kv_len;
    const uint32_t nblk = (last_key + PF_BN - 1) / PF_BN;

    const T *Q = static_cast<const T *>(a.q) + n * a.q_sn + h * a.q_sh;
    const T *K = static_cast<const T *>(a.k) + n * a.k_sn + kvh * a.k_sh;
    const T *V = static_cast<const T *>(a.v) + n * a.v_sn + kvh * a.v_sh;
    T *O = static_cast<T *>(a.o) + n * a.o_sn + h * a.o_sh;

    load_tile<T>(sQ, Q, a.q_st, q0, a.S);
    load_tile<T>(sK, K, a.k_st, 0, kv_len);
    load_tile<T>(sV, V, a.v_st, 0, kv_len);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // Q fragments of this warp's 16 rows: 8 k-steps x 4 registers
    uint32_t qf[8][4];
    {
        const uint32_t m = lane >> 3, rin = lane & 7u;
        const uint32_t row = warp * 16 + (m & 1u) * 8 + rin;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) ldsm_x4(qf[kk], sQ + sw_off(row, 2 * kk + (m >> 1)));
    }
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const uint32_t row_g[2] = {q0 + warp * 16 + g, q0 + warp * 16 + g + 8};

    for (uint32_t kb = 0; kb < nblk; ++kb) {
        const uint32_t buf = kb & 1u;
        if (kb + 1 < nblk) {// prefetch the next K/V tile into the other buffer
            load_tile<T>(sK + (buf ^ 1u) * 16384, K, a.k_st, (kb + 1) * PF_BN, kv_len);
            load_tile<T>(sV + (buf ^ 1u) * 16384, V, a.v_st, (kb + 1) * PF_BN, kv_len);
        }
        cp_async_commit();
        const uint32_t sKb = sK + buf * 16384, sVb = sV + buf * 16384;
        // ---- S = Q K^T : 16 x 64 per warp ----
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        {
            const uint32_t m = lane >> 3, rin = lane & 7u;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
                for (int nb = 0; nb < 8; nb += 2) {
                    uint32_t kf[4];
                    ldsm_x4(kf, sKb + sw_off((nb + (m >> 1)) * 8 + rin, 2 * kk + (m & 1u)));
                    Mma<T>::run(s[nb], qf[kk], kf[0], kf[1]);
                    Mma<T>::run(s[nb + 1], qf[kk], kf[2], kf[3]);
                }
            }
        }
        // ---- causal mask + online softmax (base-2, scale folded in) ----
        const uint32_t key0 = kb * PF_BN;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t key = key0 + nb * 8 + 2 * t + (e & 1);
                const uint32_t r = e >> 1;
                const bool ok = key < kv_len && key <= past + row_g[r];
                s[nb][e] = ok ? s[nb][e] * a.scale_log2e : -INFINITY;
                mx[r] = fmaxf(mx[r], s[nb][e]);
            }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            corr[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        uint32_t pf[4][4];// P as A fragments: 4 k-steps of 16 keys
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t r = e >> 1;
                p[e] = (m_run[r] == -INFINITY) ? 0.f : exp2f(s[nb][e] - m_run[r]);
                rs[r] += p[e];
            }
            pf[nb >> 1][(nb & 1) * 2 + 0] = Mma<T>::pack(p[0], p[1]);
            pf[nb >> 1][(nb & 1) * 2 + 1] = Mma<T>::pack(p[2], p[3]);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
            l_run[r] = l_run[r] * corr[r] + rs[r];
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            o[i][0] *= corr[0], o[i][1] *= corr[0];
            o[i][2] *= corr[1], o[i][3] *= corr[1];
        }
        // ---- O += P V ----
        {
            const uint32_t m = lane >> 3, rin = lane & 7u;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                for (int db = 0; db < 16; db += 2) {
                    uint32_t vf[4];
                    ldsm_x4_t(vf, sVb + sw_off(kk * 16 + (m & 1u) * 8 + rin, db + (m >> 1)));
                    Mma<T>::run(o[db], pf[kk], vf[0], vf[1]);
                    Mma<T>::run(o[db + 1], pf[kk], vf[2], vf[3]);
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();
    }
    // ---- normalise and store ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (row_g[r] < a.S) {
            const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
            T *dst = O + static_cast<int64_t>(row_g[r]) * a.o_st;
#pragma unroll
            for (int db = 0; db < 16; ++db)
                *reinterpret_cast<uint32_t *>(dst + db * 8 + 2 * t) = Mma<T>::pack(o[db][2 * r] * inv, o[db][2 * r + 1] * inv);
        }
    }
}

int attn_prefill_launch(int dtype, const PrefillArgs &a, uint32_t batch, cudaStream_t st) {
    const size_t smem = 16384 * 5;
    dim3 grid((a.S + PF_BM - 1) / PF_BM, a.n_heads, batch);
    if (dtype == RG_FP16) {
        RG_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attn_prefill_kernel<__half><<<grid, PF_THREADS, smem, st>>>(a);
    } else if (dtype == RG_BF16) {
        RG_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attn_prefill_kernel<__nv_bfloat16><<<grid, PF_THREADS, smem, st>>>(a);
    } else {
        return RG_ERR_DTYPE;
    }
    count_launch();
    return launch_status();
}

// the tcgen05 / TMEM kernel (attn_prefill_tc.cu)
bool attn_prefill_tc_applies(const rg_attn_prefill_params *p, const void *const *in);
int attn_prefill_tc_launch(const rg_attn_prefill_params *p, const void *const *in, void *const *out, cudaStream_t st);

// reference layout [N, heads, S, D] for q / o and [N, kv_heads, kv_tokens, D] for k / v
int attn_prefill_ref_layout(int dtype, const void *q, const void *K, const void *V, void *o, const int64_t *past, uint32_t batch,
                            uint32_t n_heads, uint32_t n_kv, uint32_t S, uint32_t kv_tokens, cudaStream_t st) {
    PrefillArgs a = {};
    a.q = q, a.k = K, a.v = V, a.o = o, a.past = past;
    a.q_sn = static_cast<int64_t>(n_heads) * S * PF_D, a.q_sh = static_cast<int64_t>(S) * PF_D, a.q_st = PF_D;
    a.o_sn = a.q_sn, a.o_sh = a.q_sh, a.o_st = PF_D;
    a.k_sn = static_cast<int64_t>(n_kv) * kv_tokens * PF_D, a.k_sh = static_cast<int64_t>(kv_tokens) * PF_D, a.k_st = PF_D;
    a.v_sn = a.k_sn, a.v_sh = a.k_sh, a.v_st = PF_D;
    a.n_heads = n_heads, a.n_kv = n_kv, a.S = S, a.kv_cap = kv_tokens;
    a.scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(PF_D));
    {
        rg_attn_prefill_params p = {};
        p.dtype = dtype, p.batch = batch, p.n_heads = n_heads, p.n_kv_heads = n_kv, p.seq_len = S, p.head_dim = PF_D, p.kv_capacity = kv_tokens;
        const int64_t strides[12] = {a.q_sn, a.q_sh, a.q_st, a.k_sn, a.k_sh, a.k_st, a.v_sn, a.v_sh, a.v_st, a.o_sn, a.o_sh, a.o_st};
        for (int i = 0; i < 12; ++i) p.strides[i] = strides[i];
        const void *in[4] = {q, K, V, past};
        void *out[1] = {o};
        if (attn_prefill_tc_applies(&p, in) && aligned16(o)) return attn_prefill_tc_launch(&p, in, out, st);
    }
    return attn_prefill_launch(dtype, a, batch, st);
}

}// namespace rg

using namespace rg;

extern "C" {

size_t rg_b200_attn_prefill_workspace(const rg_attn_prefill_params *) { return 0; }
int rg_b200_attn_prefill(const rg_attn_prefill_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !in[1] || !in[2] || !out[0]) return RG_ERR_NULL;
    if (p->head_dim != PF_D || p->n_kv_heads == 0 || p->n_heads % p->n_kv_heads != 0) return RG_ERR_SHAPE;
    if (p->batch == 0 || p->seq_len == 0) return RG_OK;
    if (p->batch > 65535 || p->n_heads > 65535) return RG_ERR_SHAPE;
    for (int i = 0; i < 3; ++i)
        if (!aligned16(in[i])) return RG_ERR_ALIGN;
    const int64_t *s = p->strides;
    for (int i = 0; i < 12; ++i)
        if (s[i] % 8 != 0) return RG_ERR_ALIGN;// 16-byte rows
    // 128 query rows and more, from position 0: the tcgen05 kernel; the warp-level kernel serves the rest
    if (attn_prefill_tc_applies(p, in) && aligned16(out[0])) return attn_prefill_tc_launch(p, in, out, static_cast<cudaStream_t>(stream));
    PrefillArgs a = {};
    a.q = in[0], a.k = in[1], a.v = in[2], a.past = static_cast<const int64_t *>(in[3]), a.o = out[0];
    a.q_sn = s[0], a.q_sh = s[1], a.q_st = s[2];
    a.k_sn = s[3], a.k_sh = s[4], a.k_st = s[5];
    a.v_sn = s[6], a.v_sh = s[7], a.v_st = s[8];
    a.o_sn = s[9], a.o_sh = s[10], a.o_st = s[11];
    a.n_heads = p->n_heads, a.n_kv = p->n_kv_heads, a.S = p->seq_len, a.kv_cap = p->kv_capacity;
    a.scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(p->head_dim));
    return attn_prefill_launch(p->dtype, a, p->batch, static_cast<cudaStream_t>(stream));
}
}
