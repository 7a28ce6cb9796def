// Byte-exact data movement the reference graph uses around the decoder's arithmetic: Concat, Split, Slice, Expand and Cast.
// Replaces ConcatCuda / SplitCuda / SliceCuda / ExpandCuda / CastCuda (src/04kernel/src/kernels/{concat,split,slice,expand,cast}/,
// selected by src/04kernel/include/kernel/collectors/{concat,split,slice,cast}.h and src/04kernel/src/collectors/expand.cc).
//
// The four movers are one kernel: a rank <= 6 index space whose input and output both have a base offset and a signed element
// stride per dimension (0 = broadcast, negative = reversed slice).  The innermost dimension is copied in the widest unit (16, 8,
// 4, 2 or 1 bytes) that divides the run length, every stride and offset and both base addresses; one thread moves one unit,
// consecutive threads consecutive units, so contiguous runs are coalesced.  Cast is an elementwise conversion kernel over a
// (from, to) type pair.
#include "common.cuh"

namespace rg {

constexpr int DM_RANK = 6;

static unsigned grid_for(size_t work_items, unsigned threads) {
    const size_t want = (work_items + threads - 1) / threads;
    const size_t cap = static_cast<size_t>(sm_count()) * 16;
    return static_cast<unsigned>(want < 1 ? 1 : (want > cap ? cap : want));
}

struct DmIndex {
    uint32_t shape[DM_RANK];       // right-aligned, leading dimensions 1
    int64_t in_stride[DM_RANK];    // in units
    int64_t out_stride[DM_RANK];   // in units
    int64_t in_offset, out_offset;// in units
};

template<class U>
__global__ void __launch_bounds__(256) strided_copy_kernel(const U *__restrict__ in, U *__restrict__ out, const DmIndex ix, uint64_t total) {
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        uint64_t rem = i;
        int64_t si = ix.in_offset, so = ix.out_offset;
#pragma unroll
        for (int d = DM_RANK - 1; d >= 0; --d) {
            const uint32_t c = static_cast<uint32_t>(rem % ix.shape[d]);
            rem /= ix.shape[d];
            si += static_cast<int64_t>(c) * ix.in_stride[d];
            so += static_cast<int64_t>(c) * ix.out_stride[d];
        }
        out[so] = in[si];
    }
}

// shape / strides / offsets in ELEMENTS of elem_bytes; picks the copy unit and launches
static int strided_copy(uint32_t elem_bytes, int rank, const uint32_t *shape, const int64_t *in_stride, const int64_t *out_stride, int64_t in_offset,
                        int64_t out_offset, const void *in, void *out, cudaStream_t st) {
    if (rank < 0 || rank > DM_RANK) return RG_ERR_SHAPE;
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8 && elem_bytes != 16) return RG_ERR_DTYPE;
    DmIndex ix;
    const int pad = DM_RANK - rank;
    for (int d = 0; d < DM_RANK; ++d) ix.shape[d] = 1, ix.in_stride[d] = ix.out_stride[d] = 0;
    uint64_t total = 1;
    for (int d = 0; d < rank; ++d) {
        ix.shape[pad + d] = shape[d], ix.in_stride[pad + d] = in_stride[d], ix.out_stride[pad + d] = out_stride[d];
        total *= shape[d];
    }
    if (total == 0) return RG_OK;
    ix.in_offset = in_offset, ix.out_offset = out_offset;
    // widen the unit while the innermost run is contiguous on both sides and everything stays aligned
    uint32_t unit = elem_bytes;
    const int last = DM_RANK - 1;
    if (rank > 0 && ix.in_stride[last] == 1 && ix.out_stride[last] == 1) {
        while (unit < 16) {
            const uint32_t f = 2;// elements of the current unit per next unit
            bool ok = ix.shape[last] % f == 0 && ix.in_offset % f == 0 && ix.out_offset % f == 0 &&
                      reinterpret_cast<uintptr_t>(in) % (unit * f) == 0 && reinterpret_cast<uintptr_t>(out) % (unit * f) == 0;
            for (int d = 0; d < last && ok; ++d) ok = ix.in_stride[d] % f == 0 && ix.out_stride[d] % f == 0;
            if (!ok) break;
            ix.shape[last] /= f, ix.in_offset /= f, ix.out_offset /= f;
            for (int d = 0; d < last; ++d) ix.in_stride[d] /= f, ix.out_stride[d] /= f;
            total /= f, unit *= f;
        }
    }
    const unsigned g = grid_for(total, 256);
    switch (unit) {
        case 1: strided_copy_kernel<uint8_t><<<g, 256, 0, st>>>(static_cast<const uint8_t *>(in), static_cast<uint8_t *>(out), ix, total); break;
        case 2: strided_copy_kernel<uint16_t><<<g, 256, 0, st>>>(static_cast<const uint16_t *>(in), static_cast<uint16_t *>(out), ix, total); break;
        case 4: strided_copy_kernel<uint32_t><<<g, 256, 0, st>>>(static_cast<const uint32_t *>(in), static_cast<uint32_t *>(out), ix, total); break;
        case 8: strided_copy_kernel<uint64_t><<<g, 256, 0, st>>>(static_cast<const uint64_t *>(in), static_cast<uint64_t *>(out), ix, total); break;
        default: strided_copy_kernel<uint4><<<g, 256, 0, st>>>(static_cast<const uint4 *>(in), static_cast<uint4 *>(out), ix, total); break;
    }
    count_launch();
    return launch_status();
}

// ---- Cast ---------------------------------------------------------------------------------------------------------
// Conversions follow C++ static_cast (float -> integer truncates toward zero; anything -> bool is `!= 0`), with 16-bit floats
// rounded to nearest even, as the CUDA kernels of the reference do (its host-side fp16_t truncates instead).
template<class To, class From> struct CastOne {
    static __device__ __forceinline__ To run(From v) { return static_cast<To>(v); }
};
template<class From> struct CastOne<__half, From> {
    static __device__ __forceinline__ __half run(From v) { return __float2half_rn(static_cast<float>(v)); }
};
template<class From> struct CastOne<__nv_bfloat16, From> {
    static __device__ __forceinline__ __nv_bfloat16 run(From v) { return __float2bfloat16_rn(static_cast<float>(v)); }
};
template<> struct CastOne<__half, double> {// double -> half through float would round twice
    static __device__ __forceinline__ __half run(double v) { return __double2half(v); }
};
template<class To> struct CastOne<To, __half> {
    static __device__ __forceinline__ To run(__half v) { return static_cast<To>(__half2float(v)); }
};
template<class To> struct CastOne<To, __nv_bfloat16> {
    static __device__ __forceinline__ To run(__nv_bfloat16 v) { return static_cast<To>(__bfloat162float(v)); }
};
template<> struct CastOne<__half, __half> {
    static __device__ __forceinline__ __half run(__half v) { return v; }
};
template<> struct CastOne<__nv_bfloat16, __nv_bfloat16> {
    static __device__ __forceinline__ __nv_bfloat16 run(__nv_bfloat16 v) { return v; }
};
template<> struct CastOne<__half, __nv_bfloat16> {
    static __device__ __forceinline__ __half run(__nv_bfloat16 v) { return __float2half_rn(__bfloat162float(v)); }
};
template<> struct CastOne<__nv_bfloat16, __half> {
    static __device__ __forceinline__ __nv_bfloat16 run(__half v) { return __float2bfloat16_rn(__half2float(v)); }
};
// bool is stored as one byte holding 0 or 1
struct BoolByte {
    uint8_t v;
};
template<class From> struct CastOne<BoolByte, From> {
    static __device__ __forceinline__ BoolByte run(From v) { return BoolByte{static_cast<uint8_t>(v != From(0) ? 1 : 0)}; }
};
template<> struct CastOne<BoolByte, __half> {
    static __device__ __forceinline__ BoolByte run(__half v) { return BoolByte{static_cast<uint8_t>(__half2float(v) != 0.f ? 1 : 0)}; }
};
template<> struct CastOne<BoolByte, __nv_bfloat16> {
    static __device__ __forceinline__ BoolByte run(__nv_bfloat16 v) { return BoolByte{static_cast<uint8_t>(__bfloat162float(v) != 0.f ? 1 : 0)}; }
};
template<class To> struct CastOne<To, BoolByte> {
    static __device__ __forceinline__ To run(BoolByte v) { return CastOne<To, uint8_t>::run(static_cast<uint8_t>(v.v ? 1 : 0)); }
};
template<> struct CastOne<__half, BoolByte> {
    static __device__ __forceinline__ __half run(BoolByte v) { return __float2half_rn(v.v ? 1.f : 0.f); }
};
template<> struct CastOne<__nv_bfloat16, BoolByte> {
    static __device__ __forceinline__ __nv_bfloat16 run(BoolByte v) { return __float2bfloat16_rn(v.v ? 1.f : 0.f); }
};
template<> struct CastOne<BoolByte, BoolByte> {
    static __device__ __forceinline__ BoolByte run(BoolByte v) { return BoolByte{static_cast<uint8_t>(v.v ? 1 : 0)}; }
};

template<class To, class From>
__global__ void __launch_bounds__(256) cast_kernel(const From *__restrict__ x, To *__restrict__ y, uint64_t n) {
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<uint64_t>(gridDim.x) * blockDim.x)
        y[i] = CastOne<To, From>::run(x[i]);
}

template<class From>
static int cast_from(int to, const void *x, void *y, uint64_t n, cudaStream_t st) {
    const unsigned g = grid_for(n, 256);
    const From *xs = static_cast<const From *>(x);
#define RG_CAST_TO(T) cast_kernel<T, From><<<g, 256, 0, st>>>(xs, static_cast<T *>(y), n)
    switch (to) {
        case RG_F32: RG_CAST_TO(float); break;
        case RG_F64: RG_CAST_TO(double); break;
        case RG_FP16: RG_CAST_TO(__half); break;
        case RG_BF16: RG_CAST_TO(__nv_bfloat16); break;
        case RG_I8: RG_CAST_TO(int8_t); break;
        case RG_U8: RG_CAST_TO(uint8_t); break;
        case RG_I16: RG_CAST_TO(int16_t); break;
        case RG_U16: RG_CAST_TO(uint16_t); break;
        case RG_I32: RG_CAST_TO(int32_t); break;
        case RG_U32: RG_CAST_TO(uint32_t); break;
        case RG_I64: RG_CAST_TO(long long); break;
        case RG_U64: RG_CAST_TO(unsigned long long); break;
        case RG_BOOL: RG_CAST_TO(BoolByte); break;
        default: return RG_ERR_DTYPE;
    }
#undef RG_CAST_TO
    count_launch();
    return launch_status();
}

}// namespace rg

using namespace rg;

extern "C" {

size_t rg_b200_concat_workspace(const rg_concat_params *) { return 0; }
size_t rg_b200_split_workspace(const rg_concat_params *) { return 0; }
size_t rg_b200_slice_workspace(const rg_slice_params *) { return 0; }
size_t rg_b200_expand_workspace(const rg_expand_params *) { return 0; }
size_t rg_b200_cast_workspace(const rg_cast_params *) { return 0; }

static int concat_or_split(const rg_concat_params *p, const void *const *parts_in, void *const *parts_out, const void *whole_in, void *whole_out,
                           void *stream) {
    if (p->n_parts == 0 || p->n_parts > RG_CONCAT_MAX_PARTS) return RG_ERR_SHAPE;
    uint64_t total_axis = 0;
    for (uint32_t i = 0; i < p->n_parts; ++i) total_axis += p->axis_len[i];
    auto st = static_cast<cudaStream_t>(stream);
    uint64_t before = 0;
    for (uint32_t i = 0; i < p->n_parts; ++i) {
        const uint64_t run = static_cast<uint64_t>(p->axis_len[i]) * p->inner;// elements of one outer slice of part i
        if (run == 0 || p->outer == 0) {
            before += run;
            continue;
        }
        if (run > 0xffffffffull) return RG_ERR_SHAPE;
        const uint32_t shape[2] = {p->outer, static_cast<uint32_t>(run)};
        const int64_t part_stride[2] = {static_cast<int64_t>(run), 1};
        const int64_t whole_stride[2] = {static_cast<int64_t>(total_axis * p->inner), 1};
        int rc;
        if (whole_out) {// concat: part i -> its band of the whole
            if (!parts_in[i]) return RG_ERR_NULL;
            rc = strided_copy(p->elem_bytes, 2, shape, part_stride, whole_stride, 0, static_cast<int64_t>(before), parts_in[i], whole_out, st);
        } else {
            if (!parts_out[i]) return RG_ERR_NULL;
            rc = strided_copy(p->elem_bytes, 2, shape, whole_stride, part_stride, static_cast<int64_t>(before), 0, whole_in, parts_out[i], st);
        }
        if (rc != RG_OK) return rc;
        before += run;
    }
    return RG_OK;
}

int rg_b200_concat(const rg_concat_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !out[0]) return RG_ERR_NULL;
    return concat_or_split(p, in, nullptr, nullptr, out[0], stream);
}

int rg_b200_split(const rg_concat_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out || !in[0]) return RG_ERR_NULL;
    return concat_or_split(p, nullptr, out, in[0], nullptr, stream);
}

int rg_b200_slice(const rg_slice_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out) return RG_ERR_NULL;
    if (p->rank > RG_MOVE_MAX_RANK) return RG_ERR_SHAPE;
    {// an empty result needs no buffers
        uint64_t total = 1;
        for (uint32_t d = 0; d < p->rank; ++d) total *= p->length[d];
        if (total == 0) return RG_OK;
    }
    if (!in[0] || !out[0]) return RG_ERR_NULL;
    int64_t base[RG_MOVE_MAX_RANK], in_stride[RG_MOVE_MAX_RANK], out_stride[RG_MOVE_MAX_RANK];
    int64_t s = 1;
    for (int d = static_cast<int>(p->rank) - 1; d >= 0; --d) base[d] = s, s *= p->in_shape[d];
    int64_t off = 0, so = 1;
    for (int d = static_cast<int>(p->rank) - 1; d >= 0; --d) {
        // every index start + i * step, 0 <= i < length, must lie inside the input dimension
        if (p->length[d]) {
            const int64_t first = p->start[d], last = p->start[d] + static_cast<int64_t>(p->length[d] - 1) * p->step[d];
            if (first < 0 || last < 0 || first >= static_cast<int64_t>(p->in_shape[d]) || last >= static_cast<int64_t>(p->in_shape[d])) return RG_ERR_SHAPE;
        }
        off += p->start[d] * base[d];
        in_stride[d] = p->step[d] * base[d];
        out_stride[d] = so, so *= p->length[d];
    }
    return strided_copy(p->elem_bytes, static_cast<int>(p->rank), p->length, in_stride, out_stride, off, 0, in[0], out[0], static_cast<cudaStream_t>(stream));
}

int rg_b200_expand(const rg_expand_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out) return RG_ERR_NULL;
    if (p->rank > RG_MOVE_MAX_RANK) return RG_ERR_SHAPE;
    {
        uint64_t total = 1;
        for (uint32_t d = 0; d < p->rank; ++d) total *= p->out_shape[d];
        if (total == 0) return RG_OK;
    }
    if (!in[0] || !out[0]) return RG_ERR_NULL;
    int64_t in_stride[RG_MOVE_MAX_RANK], out_stride[RG_MOVE_MAX_RANK];
    int64_t si = 1, so = 1;
    for (int d = static_cast<int>(p->rank) - 1; d >= 0; --d) {
        if (p->in_shape[d] != p->out_shape[d] && p->in_shape[d] != 1) return RG_ERR_SHAPE;
        in_stride[d] = p->in_shape[d] == 1 ? 0 : si;
        si *= p->in_shape[d];
        out_stride[d] = so, so *= p->out_shape[d];
    }
    return strided_copy(p->elem_bytes, static_cast<int>(p->rank), p->out_shape, in_stride, out_stride, 0, 0, in[0], out[0], static_cast<cudaStream_t>(stream));
}

int rg_b200_cast(const rg_cast_params *p, void *, const void *const *in, void *const *out, void *stream) {
    if (!p || !in || !out) return RG_ERR_NULL;
    if (p->n == 0) return RG_OK;
    if (!in[0] || !out[0]) return RG_ERR_NULL;
    auto st = static_cast<cudaStream_t>(stream);
    switch (p->from) {
        case RG_F32: return cast_from<float>(p->to, in[0], out[0], p->n, st);
        case RG_F64: return cast_from<double>(p->to, in[0], out[0], p->n, st);
        case RG_FP16: return cast_from<__half>(p->to, in[0], out[0], p->n, st);
        case RG_BF16: return cast_from<__nv_bfloat16>(p->to, in[0], out[0], p->n, st);
        case RG_I8: return cast_from<int8_t>(p->to, in[0], out[0], p->n, st);
        case RG_U8: return cast_from<uint8_t>(p->to, in[0], out[0], p->n, st);
        case RG_I16: return cast_from<int16_t>(p->to, in[0], out[0], p->n, st);
        case RG_U16: return cast_from<uint16_t>(p->to, in[0], out[0], p->n, st);
        case RG_I32: return cast_from<int32_t>(p->to, in[0], out[0], p->n, st);
        case RG_U32: return cast_from<uint32_t>(p->to, in[0], out[0], p->n, st);
        case RG_I64: return cast_from<long long>(p->to, in[0], out[0], p->n, st);
        case RG_U64: return cast_from<unsigned long long>(p->to, in[0], out[0], p->n, st);
        case RG_BOOL: return cast_from<BoolByte>(p->to, in[0], out[0], p->n, st);
        default: return RG_ERR_DTYPE;
    }
}
}
