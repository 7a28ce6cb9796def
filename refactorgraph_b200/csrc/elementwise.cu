// Data-movement and element-wise kernels of the decoder path: Gather (embedding), binary/unary/where with
// broadcast, Transpose, rotary position embedding.  All HBM-bound; the wide paths move 16 bytes per thread
// and size the grid as a multiple of the SM count.
#include "common.cuh"

namespace rg {

static __device__ int s_elementwise_index_error;// a gathered index, append position or block-table entry was out of range (access skipped)
int elementwise_index_error_word(bool clear) { return error_symbol(s_elementwise_index_error, clear); }

static unsigned grid_for(size_t work_items, unsigned threads) {
    const size_t want = (work_items + threads - 1) / threads;
    const size_t cap = static_cast<size_t>(sm_count()) * 16;
    return static_cast<unsigned>(want < 1 ? 1 : (want > cap ? cap : want));
}

// ---- Gather ----------------------------------------------------------------------------------
// out[p, i, :] = data[p, idx[i], :] in units of U bytes (U = 16 when everything is 16-byte aligned).
template<class U, class I>
__global__ void gather_kernel(const U *__restrict__ data, const I *__restrict__ idx, U *__restrict__ out,
                              uint32_t prefix, uint32_t mid_in, uint32_t mid_out, uint64_t units) {
    pdl_enter();
    const uint64_t total = static_cast<uint64_t>(prefix) * mid_out * units;
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
         t += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint64_t u = t % units, row = t / units;
        const uint64_t i = row % mid_out, p = row / mid_out;
        int64_t k = static_cast<int64_t>(idx[i]);
        if (k < 0) k += mid_in;
        if (k < 0 || k >= static_cast<int64_t>(mid_in)) {// the row is left unwritten
            s_elementwise_index_error = 1;
            continue;
        }
        out[t] = data[(p * mid_in + static_cast<uint64_t>(k)) * units + u];
    }
}

template<class I>
static int gather_launch(const rg_gather_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    const uint64_t pb = p->postfix_bytes;
    const bool v16 = pb % 16 == 0 && aligned16(in[0]) && aligned16(out[0]);
    const uint64_t rows = static_cast<uint64_t>(p->prefix) * p->mid_out;
    auto idx = static_cast<const I *>(in[1]);
#define RG_GATHER(U)                                                                                      \
    launch_pdl(gather_kernel<U, I>, dim3(grid_for(rows * (pb / sizeof(U)), 256)), dim3(256), 0, st,                           \
        static_cast<const U *>(in[0]), idx, static_cast<U *>(out[0]), p->prefix, p->mid_in, p->mid_out,   \
        pb / sizeof(U))
    if (v16) RG_GATHER(uint4);
    else if (pb % 4 == 0 && (reinterpret_cast<uintptr_t>(in[0]) | reinterpret_cast<uintptr_t>(out[0])) % 4 == 0)
        RG_GATHER(uint32_t);
    else if (pb % 2 == 0 && (reinterpret_cast<uintptr_t>(in[0]) | reinterpret_cast<uintptr_t>(out[0])) % 2 == 0)
        RG_GATHER(uint16_t);
    else
        RG_GATHER(uint8_t);
#undef RG_GATHER
    count_launch();
    return launch_status();
}

// ---- Binary / Where with rank-4 broadcast -----------------------------------------------------
struct Idx4 {
    uint32_t shape[4];
    uint32_t sa[4], sb[4], sc[4];
};
__device__ __forceinline__ void locate(const Idx4 &ix, uint64_t t, uint64_t &a, uint64_t &b, uint64_t &c) {
    a = b = c = 0;
#pragma unroll
    for (int d = 3; d >= 0; --d) {
        const uint32_t i = static_cast<uint32_t>(t % ix.shape[d]);
        t /= ix.shape[d];
        a += static_cast<uint64_t>(i) * ix.sa[d];
        b += static_cast<uint64_t>(i) * ix.sb[d];
        c += static_cast<uint64_t>(i) * ix.sc[d];
    }
}
// SimpleBinaryType values (src/04kernel/include/kernel/collectors/simple_binary.h:8-19): 0 Add, 1 Sub, 2 Mul, 3 Div, 4 Pow, 5 And,
// 6 Or, 7 Xor, 8 Mod, 9 Fmod.  Floating types: 0-4 and 9 (std::pow / std::fmod as BinaryCpu computes them,
// src/04kernel/src/kernels/simple_binary/cpu_kernel.cc:88-150).
__device__ __forceinline__ float binary_op(int op, float a, float b) {
    switch (op) {
        case 0: return a + b;
        case 1: return a - b;
        case 2: return a * b;
        case 4: return powf(a, b);
        case 9: return fmodf(a, b);
        default: return a / b;
    }
}
// Integer types: 0-3, 4 (through double, as std::pow does), 8 / 9 (the C++ `%`: sign of the dividend); a zero divisor gives 0
// instead of the reference's undefined behaviour.  Bool (one byte): 5 And, 6 Or, 7 Xor.
template<class T> __device__ __forceinline__ T binary_op_int(int op, T a, T b) {
    switch (op) {
        case 0: return static_cast<T>(a + b);
        case 1: return static_cast<T>(a - b);
        case 2: return static_cast<T>(a * b);
        case 3: return b ? static_cast<T>(a / b) : T(0);
        case 4: return static_cast<T>(pow(static_cast<double>(a), static_cast<double>(b)));
        case 5: return static_cast<T>((a != 0) && (b != 0));
        case 6: return static_cast<T>((a != 0) || (b != 0));
        case 7: return static_cast<T>((a != 0) != (b != 0));
        default: return b ? static_cast<T>(a % b) : T(0);
    }
}
template<class T>
__global__ void binary_int_kernel(const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ y, Idx4 ix, int op, uint64_t total) {
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        uint64_t ia, ib, ic;
        locate(ix, t, ia, ib, ic);
        y[t] = binary_op_int<T>(op, a[ia], b[ib]);
    }
}
template<class T>
__global__ void binary_kernel(const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ y, Idx4 ix, int op,
                              uint64_t total) {
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
         t += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        uint64_t ia, ib, ic;
        locate(ix, t, ia, ib, ic);
        y[t] = Num<T>::from_f(binary_op(op, Num<T>::to_f(a[ia]), Num<T>::to_f(b[ib])));
    }
}
// same shape, contiguous, 16-byte aligned
template<class T>
__global__ void binary_vec_kernel(const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ y, int op,
                                  uint64_t chunks) {
    constexpr int N = Vec16<T>::N;
    for (uint64_t c = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < chunks;
         c += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        Vec16<T> va, vb;
        float fa[N], fb[N];
        va.load(a + c * N);
        vb.load(b + c * N);
        va.unpack(fa);
        vb.unpack(fb);
#pragma unroll
        for (int j = 0; j < N; ++j) fa[j] = binary_op(op, fa[j], fb[j]);
        va.pack(fa);
        va.store(y + c * N);
    }
}
template<class T>
__global__ void where_kernel(const uint8_t *__restrict__ c, const T *__restrict__ a, const T *__restrict__ b,
                             T *__restrict__ y, Idx4 ix, uint64_t total) {
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
         t += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        uint64_t ia, ib, ic;
        locate(ix, t, ia, ib, ic);
        y[t] = c[ic] ? a[ia] : b[ib];
    }
}

template<class T>
static int binary_launch(const rg_binary_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    constexpr int N = Vec16<T>::N;
    uint64_t total = 1;
    bool same = true;
    uint32_t expect = 1;
    for (int d = 3; d >= 0; --d) {
        total *= p->shape[d];
        if (p->shape[d] > 1 && (p->a_stride[d] != expect || p->b_stride[d] != expect)) same = false;
        expect *= p->shape[d];
    }
    if (total == 0) return RG_OK;
    auto a = static_cast<const T *>(in[0]);
    auto b = static_cast<const T *>(in[1]);
    auto y = static_cast<T *>(out[0]);
    if (same && total % N == 0 && aligned16(a) && aligned16(b) && aligned16(y)) {
        binary_vec_kernel<T><<<grid_for(total / N, 256), 256, 0, st>>>(a, b, y, p->op, total / N);
    } else {
        Idx4 ix;
        for (int d = 0; d < 4; ++d) ix.shape[d] = p->shape[d], ix.sa[d] = p->a_stride[d], ix.sb[d] = p->b_stride[d], ix.sc[d] = 0;
        binary_kernel<T><<<grid_for(total, 256), 256, 0, st>>>(a, b, y, ix, p->op, total);
    }
    count_launch();
    return launch_status();
}

template<class T>
static int binary_int_launch(const rg_binary_params *p, const void *const *in, void *const *out, cudaStream_t st) {
    uint64_t total = 1;
    Idx4 ix;
    for (int d = 0; d < 4; ++d) ix.shape[d] = p->shape[d], ix.sa[d] = p->a_stride[d], ix.sb[d] = p->b_stride[d], ix.sc[d] = 0, total *= p->shape[d];
    if (total == 0) return RG_OK;
    binary_int_kernel<T><<<grid_for(total, 256), 256, 0, st>>>(static_cast<const T *>(in[0]), static_cast<const T *>(in[1]), static_cast<T *>(out[0]), ix, p->op, total);
    count_launch();
    return launch_status();
}

// ---- Unary ------------------------------------------------------------------------------------
// SimpleUnaryType values (src/04kernel/include/kernel/collectors/simple_unary.h:8-30), computed in fp32 as SimpleUnaryCpu does
// for F32 (src/04kernel/src/kernels/simple_unary/cpu_kernel.cc:42-59, 100-200); HardSwish is x * clamp(x / 6 + 0.5, 0, 1).
__device__ __forceinline__ float unary_op(int op, float x) {
    switch (op) {
        case 0: return fabsf(x);
        case 1: return acosf(x);
        case 2: return acoshf(x);
        case 3: return asinf(x);
        case 4: return asinhf(x);
        case 5: return atanf(x);
        case 6: return atanhf(x);
        case 7: return cosf(x);
        case 8: return coshf(x);
        case 9: return sinf(x);
        case 10: return sinhf(x);
        case 11: return tanf(x);
        case 16: return erff(x);
        case 19: {
            const float mid = x / 6.f + .5f;
            return mid <= 0.f ? 0.f : (1.f <= mid ? x : x * mid);
        }
        case 12: return tanhf(x);
        case 13: return x > 0.f ? x : 0.f;
        case 14: return sqrtf(x);
        case 15: return 1.f / (1.f + expf(-x));
        case 17: return -x;
        case 20: return expf(x);
        default: return x / (1.f + expf(-x));// 100: SiLU
    }
}
template<class T>
__global__ void unary_kernel(const T *__restrict__ x, T *__restrict__ y, int op, uint64_t n) {
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < n;
         t += static_cast<uint64_t>(gridDim.x) * blockDim.x)
        y[t] = Num<T>::from_f(unary_op(op, Num<T>::to_f(x[t])));
}

// 18 Not on bool bytes
__global__ void not_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, uint64_t n) {
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < n; t += static_cast<uint64_t>(gridDim.x) * blockDim.x)
        y[t] = x[t] ? 0 : 1;
}

// ---- Transpose ----------------------------------------------------------------------------------
template<class U>
__global__ void transpose_kernel(const U *__restrict__ x, U *__restrict__ y, Idx4 ix, uint64_t total) {
    // ix.shape = output shape, ix.sa = input stride of each output axis
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
         t += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        uint64_t ia, ib, ic;
        locate(ix, t, ia, ib, ic);
        y[t] = x[ia];
    }
}

// ---- RoPE -------------------------------------------------------------------------------------
// One thread per (token, head, i < D/2): rotates the pair (i, i + D/2).
template<class T>
__global__ void rope_kernel(const T *__restrict__ x, const int64_t *__restrict__ pos, T *__restrict__ y,
                            uint32_t tokens, uint32_t heads, uint32_t dim, float log2_theta) {
    const uint32_t half = dim / 2;
    const uint64_t total = static_cast<uint64_t>(tokens) * heads * half;
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
         t += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t i = static_cast<uint32_t>(t % half);
        const uint64_t th = t / half;// token*heads + head
        const uint64_t tok = th / heads;
        const float inv_freq = exp2f(-log2_theta * (2.0f * static_cast<float>(i) / static_cast<float>(dim)));
        const float ang = static_cast<float>(pos[tok]) * inv_freq;
        float sn, cs;
        sincosf(ang, &sn, &cs);
        const uint64_t base = th * dim;
        const float a = Num<T>::to_f(x[base + i]), b = Num<T>::to_f(x[base + i + half]);
        y[base + i] = Num<T>::from_f(a * cs - b * sn);
        y[base + i + half] = Num<T>::from_f(b * cs + a * sn);
    }
}

// ---- QKV split + RoPE + cache append (batched decode; the m <= 4 path fuses this into the linear kernel) -----
// One thread per (token, head, run of N pair indices i < D/2) of the fused projection qkv[m, (nH + 2 nKV) * D]; N = one
// 16-byte vector when the rows allow it (VEC), else 1.
template<class T, bool VEC>
__global__ void qkv_rope_append_kernel(const T *__restrict__ qkv, const int64_t *__restrict__ pos,
                                       const int32_t *__restrict__ table, T *__restrict__ q, T *__restrict__ kc,
                                       T *__restrict__ vc, uint32_t tokens, uint32_t nq, rg_kv_layout kv, float log2_theta,
                                       uint32_t tokens_per_seq) {
    pdl_enter();
    constexpr int N = VEC ? Vec16<T>::N : 1;
    const uint32_t D = kv.head_dim, half = D / 2, nkv = kv.n_kv_heads, heads = nq + 2 * nkv, cph = half / N;
    const uint64_t total = static_cast<uint64_t>(tokens) * heads * cph;
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
         t += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t i0 = static_cast<uint32_t>(t % cph) * N;
        const uint32_t h = static_cast<uint32_t>((t / cph) % heads);
        const uint32_t m = static_cast<uint32_t>(t / cph / heads);
        const T *src = qkv + (static_cast<uint64_t>(m) * heads + h) * D;
        float lo[N], hi[N];
        if constexpr (VEC) {
            Vec16<T> a, b;
            a.load(src + i0), b.load(src + i0 + half);
            a.unpack(lo), b.unpack(hi);
        } else {
            lo[0] = Num<T>::to_f(src[i0]), hi[0] = Num<T>::to_f(src[i0 + half]);
        }
        const int64_t p = pos[m];
        if (h < nq + nkv) {
#pragma unroll
            for (int j = 0; j < N; ++j) {
                const float inv_freq = exp2f(-log2_theta * (2.0f * static_cast<float>(i0 + j) / static_cast<float>(D)));
                float sn, cs;
                sincosf(static_cast<float>(p) * inv_freq, &sn, &cs);
                const float a0 = lo[j] * cs - hi[j] * sn, b0 = hi[j] * cs + lo[j] * sn;
                lo[j] = a0, hi[j] = b0;
            }
        }
        T *dst;
        if (h < nq) {
            dst = q + (static_cast<uint64_t>(m) * nq + h) * D;
        } else {
            const bool is_k = h < nq + nkv;
            const uint32_t kvh = is_k ? h - nq : h - nq - nkv;
            T *cache = is_k ? kc : vc;
            uint64_t base;
            const uint32_t seq = tokens_per_seq > 1 ? m / tokens_per_seq : m;
            if (!kv_pos_ok(p, kv, table != nullptr)) {
                s_elementwise_index_error = 1;
                continue;
            }
            if (table) {
                const uint32_t page = kv.page_size;
                const int32_t blk = table[static_cast<uint64_t>(seq) * kv.max_blocks_per_seq + static_cast<uint32_t>(p) / page];
                if (!kv_block_ok(blk, kv)) {
                    s_elementwise_index_error = 1;
                    continue;
                }
                base = ((static_cast<uint64_t>(blk) * nkv + kvh) * page + static_cast<uint32_t>(p) % page) * D;
            } else {
                base = ((static_cast<uint64_t>(seq) * nkv + kvh) * kv.max_seq + static_cast<uint64_t>(p)) * D;
            }
            dst = cache + base;
        }
        if constexpr (VEC) {
            Vec16<T> a, b;
            a.pack(lo), b.pack(hi);
            a.store(dst + i0), b.store(dst + i0 + half);
        } else {
            dst[i0] = Num<T>::from_f(lo[0]);
            dst[i0 + half] = Num<T>::from_f(hi[0]);
        }
    }
}

// y[r, j] = silu(x[r, j]) * x[r, f + j]; one 16-byte vector per thread when f and the pointers allow it (VEC)
template<class T, bool VEC>
__global__ void swiglu_kernel(const T *__restrict__ x, T *__restrict__ y, uint32_t rows, uint32_t f) {
    pdl_enter();
    constexpr int N = VEC ? Vec16<T>::N : 1;
    const uint32_t cpr = f / N;
    const uint64_t total = static_cast<uint64_t>(rows) * cpr;
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
         t += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint64_t r = t / cpr, j = (t % cpr) * N;
        const T *gp = x + r * 2 * f + j;
        if constexpr (VEC) {
            Vec16<T> gv, uv, o;
            gv.load(gp), uv.load(gp + f);
            float g[N], u[N];
            gv.unpack(g), uv.unpack(u);
#pragma unroll
            for (int e = 0; e < N; ++e) g[e] = g[e] / (1.f + expf(-g[e])) * u[e];
            o.pack(g);
            o.store(y + r * f + j);
        } else {
            const float g = Num<T>::to_f(gp[0]), u = Num<T>::to_f(gp[f]);
            y[r * f + j] = Num<T>::from_f(g / (1.f + expf(-g)) * u);
        }
    }
}

__global__ void state_update_kernel(const int64_t *__restrict__ src, int64_t *__restrict__ state, uint32_t n,
                                    int64_t delta) {
    pdl_enter();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) state[i] = (src ? src[i] : state[i]) + delta;
}

}// namespace rg

using namespace rg;

extern "C" {

size_t rg_b200_gather_workspace(const rg_gather_params *) { return 0; }
int rg_b200_gather(const rg_gather_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out) return RG_ERR_NULL;
    if (p->prefix == 0 || p->mid_out == 0 || p->postfix_bytes == 0) return RG_OK;// empty index list / rows
    if (!in[0] || !in[1] || !out[0]) return RG_ERR_NULL;
    if (p->mid_in == 0) return RG_ERR_SHAPE;
    auto st = static_cast<cudaStream_t>(stream);
    switch (p->idx_dtype) {
        case RG_I32: return gather_launch<int32_t>(p, in, out, st);
        case RG_I64: return gather_launch<int64_t>(p, in, out, st);
        default: return RG_ERR_DTYPE;
    }
}

size_t rg_b200_binary_workspace(const rg_binary_params *) { return 0; }
int rg_b200_binary(const rg_binary_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !in[1] || !out[0]) return RG_ERR_NULL;
    if (p->op < 0 || p->op > 9) return RG_ERR_UNSUPPORTED;
    auto st = static_cast<cudaStream_t>(stream);
    const bool logic = p->op >= 5 && p->op <= 7;
    switch (p->dtype) {
        case RG_F32: case RG_FP16: case RG_BF16:
            if (logic || p->op == 8) return RG_ERR_UNSUPPORTED;// And / Or / Xor are for bool, Mod for integers
            return p->dtype == RG_F32 ? binary_launch<float>(p, in, out, st) : p->dtype == RG_FP16 ? binary_launch<__half>(p, in, out, st) : binary_launch<__nv_bfloat16>(p, in, out, st);
        case RG_BOOL: return logic ? binary_int_launch<uint8_t>(p, in, out, st) : RG_ERR_UNSUPPORTED;
        case RG_U8: return logic ? RG_ERR_UNSUPPORTED : binary_int_launch<uint8_t>(p, in, out, st);
        case RG_I8: return logic ? RG_ERR_UNSUPPORTED : binary_int_launch<int8_t>(p, in, out, st);
        case RG_I16: return logic ? RG_ERR_UNSUPPORTED : binary_int_launch<int16_t>(p, in, out, st);
        case RG_I32: return logic ? RG_ERR_UNSUPPORTED : binary_int_launch<int32_t>(p, in, out, st);
        case RG_U32: return logic ? RG_ERR_UNSUPPORTED : binary_int_launch<uint32_t>(p, in, out, st);
        case RG_I64: return logic ? RG_ERR_UNSUPPORTED : binary_int_launch<long long>(p, in, out, st);
        default: return RG_ERR_DTYPE;
    }
}

size_t rg_b200_unary_workspace(const rg_unary_params *) { return 0; }
int rg_b200_unary(const rg_unary_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !out[0]) return RG_ERR_NULL;
    if (!((p->op >= 0 && p->op <= 20) || p->op == 100)) return RG_ERR_UNSUPPORTED;
    if (p->n == 0) return RG_OK;
    auto st = static_cast<cudaStream_t>(stream);
    const unsigned g = grid_for(p->n, 256);
    if (p->op == 18) {// Not: bool bytes only
        if (p->dtype != RG_BOOL) return RG_ERR_DTYPE;
        not_kernel<<<g, 256, 0, st>>>(static_cast<const uint8_t *>(in[0]), static_cast<uint8_t *>(out[0]), p->n);
        count_launch();
        return launch_status();
    }
    switch (p->dtype) {
        case RG_F32: unary_kernel<float><<<g, 256, 0, st>>>(static_cast<const float *>(in[0]), static_cast<float *>(out[0]), p->op, p->n); break;
        case RG_FP16: unary_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half *>(in[0]), static_cast<__half *>(out[0]), p->op, p->n); break;
        case RG_BF16: unary_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(in[0]), static_cast<__nv_bfloat16 *>(out[0]), p->op, p->n); break;
        default: return RG_ERR_DTYPE;
    }
    count_launch();
    return launch_status();
}

size_t rg_b200_where_workspace(const rg_where_params *) { return 0; }
int rg_b200_where(const rg_where_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !in[1] || !in[2] || !out[0]) return RG_ERR_NULL;
    Idx4 ix;
    uint64_t total = 1;
    for (int d = 0; d < 4; ++d) {
        ix.shape[d] = p->shape[d], ix.sa[d] = p->a_stride[d], ix.sb[d] = p->b_stride[d], ix.sc[d] = p->c_stride[d];
        total *= p->shape[d];
    }
    if (total == 0) return RG_OK;
    auto st = static_cast<cudaStream_t>(stream);
    auto c = static_cast<const uint8_t *>(in[0]);
    const unsigned g = grid_for(total, 256);
    switch (p->dtype) {
        case RG_F32: case RG_I32: case RG_U32:
            where_kernel<uint32_t><<<g, 256, 0, st>>>(c, static_cast<const uint32_t *>(in[1]), static_cast<const uint32_t *>(in[2]), static_cast<uint32_t *>(out[0]), ix, total);
            break;
        case RG_FP16: case RG_BF16:
            where_kernel<uint16_t><<<g, 256, 0, st>>>(c, static_cast<const uint16_t *>(in[1]), static_cast<const uint16_t *>(in[2]), static_cast<uint16_t *>(out[0]), ix, total);
            break;
        case RG_I64: case RG_F64:
            where_kernel<uint64_t><<<g, 256, 0, st>>>(c, static_cast<const uint64_t *>(in[1]), static_cast<const uint64_t *>(in[2]), static_cast<uint64_t *>(out[0]), ix, total);
            break;
        case RG_U8: case RG_I8: case RG_BOOL:
            where_kernel<uint8_t><<<g, 256, 0, st>>>(c, static_cast<const uint8_t *>(in[1]), static_cast<const uint8_t *>(in[2]), static_cast<uint8_t *>(out[0]), ix, total);
            break;
        default: return RG_ERR_DTYPE;
    }
    count_launch();
    return launch_status();
}

size_t rg_b200_transpose_workspace(const rg_transpose_params *) { return 0; }
int rg_b200_transpose(const rg_transpose_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !out[0]) return RG_ERR_NULL;
    if (p->rank == 0 || p->rank > 4) return RG_ERR_SHAPE;
    uint32_t in_stride[4], stride = 1;
    for (int d = static_cast<int>(p->rank) - 1; d >= 0; --d) {
        in_stride[d] = stride;
        stride *= p->in_shape[d];
    }
    Idx4 ix;
    uint64_t total = 1;
    const int pad = 4 - static_cast<int>(p->rank);
    for (int d = 0; d < 4; ++d) ix.shape[d] = 1, ix.sa[d] = ix.sb[d] = ix.sc[d] = 0;
    for (uint32_t d = 0; d < p->rank; ++d) {
        if (p->perm[d] >= p->rank) return RG_ERR_SHAPE;
        ix.shape[pad + d] = p->in_shape[p->perm[d]];
        ix.sa[pad + d] = in_stride[p->perm[d]];
        total *= ix.shape[pad + d];
    }
    if (total == 0) return RG_OK;
    auto st = static_cast<cudaStream_t>(stream);
    const unsigned g = grid_for(total, 256);
    switch (p->elem_bytes) {
        case 1: transpose_kernel<uint8_t><<<g, 256, 0, st>>>(static_cast<const uint8_t *>(in[0]), static_cast<uint8_t *>(out[0]), ix, total); break;
        case 2: transpose_kernel<uint16_t><<<g, 256, 0, st>>>(static_cast<const uint16_t *>(in[0]), static_cast<uint16_t *>(out[0]), ix, total); break;
        case 4: transpose_kernel<uint32_t><<<g, 256, 0, st>>>(static_cast<const uint32_t *>(in[0]), static_cast<uint32_t *>(out[0]), ix, total); break;
        case 8: transpose_kernel<uint64_t><<<g, 256, 0, st>>>(static_cast<const uint64_t *>(in[0]), static_cast<uint64_t *>(out[0]), ix, total); break;
        default: return RG_ERR_DTYPE;
    }
    count_launch();
    return launch_status();
}

size_t rg_b200_rope_workspace(const rg_rope_params *) { return 0; }
int rg_b200_rope(const rg_rope_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !in[1] || !out[0]) return RG_ERR_NULL;
    if (p->head_dim == 0 || p->head_dim % 2 != 0 || !(p->theta > 0.f)) return RG_ERR_SHAPE;
    const uint64_t total = static_cast<uint64_t>(p->tokens) * p->heads * (p->head_dim / 2);
    if (total == 0) return RG_OK;
    auto st = static_cast<cudaStream_t>(stream);
    const unsigned g = grid_for(total, 256);
    const float l2t = log2f(p->theta);
    auto pos = static_cast<const int64_t *>(in[1]);
    switch (p->dtype) {
        case RG_F32: rope_kernel<float><<<g, 256, 0, st>>>(static_cast<const float *>(in[0]), pos, static_cast<float *>(out[0]), p->tokens, p->heads, p->head_dim, l2t); break;
        case RG_FP16: rope_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half *>(in[0]), pos, static_cast<__half *>(out[0]), p->tokens, p->heads, p->head_dim, l2t); break;
        case RG_BF16: rope_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(in[0]), pos, static_cast<__nv_bfloat16 *>(out[0]), p->tokens, p->heads, p->head_dim, l2t); break;
        default: return RG_ERR_DTYPE;
    }
    count_launch();
    return launch_status();
}

size_t rg_b200_state_update_workspace(const rg_state_update_params *) { return 0; }
int rg_b200_state_update(const rg_state_update_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !out[0]) return RG_ERR_NULL;
    if (p->n == 0) return RG_OK;
    launch_pdl(state_update_kernel, dim3((p->n + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream), 
        static_cast<const int64_t *>(in[0]), static_cast<int64_t *>(out[0]), p->n, p->delta);
    count_launch();
    return launch_status();
}

size_t rg_b200_qkv_rope_append_workspace(const rg_qkv_rope_append_params *) { return 0; }
int rg_b200_qkv_rope_append(const rg_qkv_rope_append_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !in[1] || !out[0] || !out[1] || !out[2]) return RG_ERR_NULL;
    const uint32_t D = p->kv.head_dim;
    if (D == 0 || D % 2 != 0 || p->kv.n_kv_heads == 0 || !(p->theta > 0.f)) return RG_ERR_SHAPE;
    if (in[2] && p->kv.page_size == 0) return RG_ERR_SHAPE;
    const uint64_t total = static_cast<uint64_t>(p->tokens) * (p->n_heads + 2 * p->kv.n_kv_heads) * (D / 2);
    if (total == 0) return RG_OK;
    auto st = static_cast<cudaStream_t>(stream);
    const float l2t = log2f(p->theta);
    auto pos = static_cast<const int64_t *>(in[1]);
    auto tab = static_cast<const int32_t *>(in[2]);
    const unsigned esz = p->dtype == RG_F32 ? 4u : 2u, vn = 16u / esz;
    const bool vec = (D / 2) % vn == 0 && aligned16(in[0]) && aligned16(out[0]) && aligned16(out[1]) && aligned16(out[2]);
    const unsigned g = grid_for(vec ? total / vn : total, 256);
#define RG_QRA(T)                                                                                                                      \
    (vec ? launch_pdl(qkv_rope_append_kernel<T, true>, dim3(g), dim3(256), 0, st, static_cast<const T *>(in[0]), pos, tab,            \
                      static_cast<T *>(out[0]), static_cast<T *>(out[1]), static_cast<T *>(out[2]), p->tokens, p->n_heads, p->kv, l2t, \
                      p->tokens_per_seq)                                                                                               \
         : launch_pdl(qkv_rope_append_kernel<T, false>, dim3(g), dim3(256), 0, st, static_cast<const T *>(in[0]), pos, tab,           \
                      static_cast<T *>(out[0]), static_cast<T *>(out[1]), static_cast<T *>(out[2]), p->tokens, p->n_heads, p->kv, l2t, \
                      p->tokens_per_seq))
    switch (p->dtype) {
        case RG_F32: RG_QRA(float); break;
        case RG_FP16: RG_QRA(__half); break;
        case RG_BF16: RG_QRA(__nv_bfloat16); break;
        default: return RG_ERR_DTYPE;
    }
#undef RG_QRA
    count_launch();
    return launch_status();
}

size_t rg_b200_swiglu_workspace(const rg_swiglu_params *) { return 0; }
int rg_b200_swiglu(const rg_swiglu_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0] || !out[0]) return RG_ERR_NULL;
    const uint64_t total = static_cast<uint64_t>(p->rows) * p->f;
    if (total == 0) return RG_OK;
    auto st = static_cast<cudaStream_t>(stream);
    const unsigned vn = p->dtype == RG_F32 ? 4u : 8u;
    const bool vec = p->f % vn == 0 && aligned16(in[0]) && aligned16(out[0]);
    const unsigned g = grid_for(vec ? total / vn : total, 256);
#define RG_SWIGLU(T)                                                                                                               \
    (vec ? launch_pdl(swiglu_kernel<T, true>, dim3(g), dim3(256), 0, st, static_cast<const T *>(in[0]), static_cast<T *>(out[0]), \
                      p->rows, p->f)                                                                                               \
         : launch_pdl(swiglu_kernel<T, false>, dim3(g), dim3(256), 0, st, static_cast<const T *>(in[0]), static_cast<T *>(out[0]), \
                      p->rows, p->f))
    switch (p->dtype) {
        case RG_F32: RG_SWIGLU(float); break;
        case RG_FP16: RG_SWIGLU(__half); break;
        case RG_BF16: RG_SWIGLU(__nv_bfloat16); break;
        default: return RG_ERR_DTYPE;
    }
#undef RG_SWIGLU
    count_launch();
    return launch_status();
}
}
