// B200 kernels behind the reference's Kernel interface.  Each `XxxB200 final : Kernel` follows the pattern of
// src/04kernel/src/kernels/rms_normalization/cuda_kernel.{hh,cc}: a POD info filled from tensor shapes, a static
// build() that returns nullptr when the case is unsupported (never throws), typeId() as the address of a
// function-local static, and lower(Resources&) returning {routine, workspace bytes}.  The routine calls the C ABI
// (include/rg_b200.h) on the stream held in Resources and turns a non-zero status into RUNTIME_ERROR.
#include "rg/collectors.h"
#include "../../../include/rg_b200.h"
#include <cstring>
#include <cuda_runtime_api.h>

namespace refactor::runtime {
    CudaStream::~CudaStream() {
        if (stream) cudaStreamDestroy(static_cast<cudaStream_t>(stream));
    }
    size_t CudaStream::typeId() noexcept {
        static uint8_t ID = 1;
        return reinterpret_cast<size_t>(&ID);
    }
    ResourceBox CudaStream::build() {
        cudaStream_t s = nullptr;
        if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) RUNTIME_ERROR("cudaStreamCreate failed");
        return std::make_unique<CudaStream>(s);
    }
}// namespace refactor::runtime

namespace refactor::kernel {
    using runtime::CudaStream;

    static void check(int status, char const *what) {
        if (status != RG_OK) RUNTIME_ERROR(std::string(what) + ": " + rg_b200_status_string(status));
    }
    static bool halfOrFloat(DataType t) { return t == DataType::F32 || t == DataType::FP16 || t == DataType::BF16; }
    static bool half(DataType t) { return t == DataType::FP16 || t == DataType::BF16; }

#define RG_KERNEL_IDS(NAME, DESC)                                         \
    static size_t typeId() noexcept {                                     \
        static uint8_t ID = 1;                                            \
        return reinterpret_cast<size_t>(&ID);                             \
    }                                                                     \
    size_t kernelTypeId() const noexcept final { return typeId(); }       \
    std::string_view description() const noexcept final { return DESC; }

    // Simple kernels: params struct P, C entry points FN / FN_workspace.
#define RG_SIMPLE_KERNEL(NAME, P, FN, DESC)                                                                     \
    struct NAME final : public Kernel {                                                                         \
        P info;                                                                                                 \
        explicit NAME(P info_) noexcept : info(info_) {}                                                        \
        RG_KERNEL_IDS(NAME, DESC)                                                                               \
        RoutineWorkspace lower(Resources &res) const final {                                                    \
            auto st = res.fetchOrStore<CudaStream>();                                                           \
            return RoutineWorkspace(                                                                            \
                [info = info, st](Resources &, void *ws, void const *const *in, void *const *out) {             \
                    check(FN(&info, ws, in, out, st->stream), #FN);                                             \
                },                                                                                              \
                FN##_workspace(&info));                                                                         \
        }                                                                                                       \
    }

    RG_SIMPLE_KERNEL(RmsNormalizationB200, rg_rms_norm_params, rg_b200_rms_norm, "RMS normalization on B200 (128-bit loads, fp32 statistics)");
    RG_SIMPLE_KERNEL(SoftmaxB200, rg_softmax_params, rg_b200_softmax, "Softmax on B200 (online max/sum, warp-shuffle reductions)");
    RG_SIMPLE_KERNEL(GatherB200, rg_gather_params, rg_b200_gather, "Gather on B200 (16-byte row copies)");
    RG_SIMPLE_KERNEL(BinaryB200, rg_binary_params, rg_b200_binary, "Element-wise binary with broadcast on B200");
    RG_SIMPLE_KERNEL(UnaryB200, rg_unary_params, rg_b200_unary, "Element-wise unary on B200");
    RG_SIMPLE_KERNEL(WhereB200, rg_where_params, rg_b200_where, "Where on B200");
    RG_SIMPLE_KERNEL(TransposeB200, rg_transpose_params, rg_b200_transpose, "Transpose on B200");
    RG_SIMPLE_KERNEL(RopeB200, rg_rope_params, rg_b200_rope, "Rotary position embedding on B200");
    RG_SIMPLE_KERNEL(ConcatB200, rg_concat_params, rg_b200_concat, "Concat on B200 (strided copy in the widest aligned unit)");
    RG_SIMPLE_KERNEL(SplitB200, rg_concat_params, rg_b200_split, "Split on B200 (strided copy in the widest aligned unit)");
    RG_SIMPLE_KERNEL(SliceB200, rg_slice_params, rg_b200_slice, "Slice on B200 (strided copy, negative steps allowed)");
    RG_SIMPLE_KERNEL(ExpandB200, rg_expand_params, rg_b200_expand, "Expand on B200 (broadcast copy)");
    RG_SIMPLE_KERNEL(CastB200, rg_cast_params, rg_b200_cast, "Cast on B200");
    RG_SIMPLE_KERNEL(TopKB200, rg_topk_params, rg_b200_topk, "TopK on B200 (radix select in shared memory)");
    RG_SIMPLE_KERNEL(TopKSampleB200, rg_topk_sample_params, rg_b200_topk_sample, "Top-k sampling on B200 (radix select + Philox)");
    RG_SIMPLE_KERNEL(AttentionB200, rg_attention_params, rg_b200_attention, "Causal attention with KV cache on B200");

    struct StateUpdateB200 final : public Kernel {
        rg_state_update_params info;
        bool hasSrc;
        StateUpdateB200(rg_state_update_params p, bool hasSrc_) noexcept : info(p), hasSrc(hasSrc_) {}
        RG_KERNEL_IDS(StateUpdateB200, "In-place int64 state update on B200")
        RoutineWorkspace lower(Resources &res) const final {
            auto st = res.fetchOrStore<CudaStream>();
            return RoutineWorkspace([info = info, hasSrc = hasSrc, st](Resources &, void *ws, void const *const *in, void *const *) {
                void const *in_[1] = {hasSrc ? in[1] : nullptr};
                void *out_[1] = {const_cast<void *>(in[0])};
                check(rg_b200_state_update(&info, ws, in_, out_, st->stream), "rg_b200_state_update");
            });
        }
    };

    // ---- RmsNormalization ---------------------------------------------------------------------------------------
    std::vector<KernelBox> RmsNormalizationCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        if (_target != Target::Nvidia || !halfOrFloat(x.dataType) || x.shape.empty()) return ans;
        rg_rms_norm_params p{};
        p.dtype = x.dataType;
        p.dim = x.shape.back();
        p.rows = p.dim ? static_cast<uint32_t>(x.elementsSize() / p.dim) : 0;
        p.epsilon = epsilon;
        ans.emplace_back(std::make_unique<RmsNormalizationB200>(p));
        return ans;
    }

    // ---- Softmax: SoftmaxInfo{pre, mid, post} (src/04kernel/src/attributes/softmax_info.cc:6-13) -------------------
    std::vector<KernelBox> SoftmaxCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        if (_target != Target::Nvidia || !halfOrFloat(x.dataType) || axis >= x.shape.size()) return ans;
        rg_softmax_params p{};
        p.dtype = x.dataType;
        p.pre = p.post = 1;
        for (size_t i = 0; i < axis; ++i) p.pre *= x.shape[i];
        p.mid = x.shape[axis];
        for (size_t i = axis + 1; i < x.shape.size(); ++i) p.post *= x.shape[i];
        ans.emplace_back(std::make_unique<SoftmaxB200>(p));
        return ans;
    }

    // ---- Gather: GatherInfo (src/04kernel/src/attributes/gather_info.cc:19-27) ---------------------------------------
    std::vector<KernelBox> GatherCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &d = inputs[0].get();
        auto const &i = inputs[1].get();
        if (_target != Target::Nvidia || axis >= d.shape.size()) return ans;
        if (i.dataType != DataType::I32 && i.dataType != DataType::I64) return ans;
        rg_gather_params p{};
        p.prefix = 1;
        for (size_t k = 0; k < axis; ++k) p.prefix *= d.shape[k];
        p.mid_in = d.shape[axis];
        p.postfix_bytes = d.dataType.size();
        for (size_t k = axis + 1; k < d.shape.size(); ++k) p.postfix_bytes *= d.shape[k];
        p.mid_out = static_cast<uint32_t>(i.elementsSize());
        p.idx_dtype = i.dataType;
        ans.emplace_back(std::make_unique<GatherB200>(p));
        return ans;
    }

    // ---- broadcasting helpers (rank <= 4) -------------------------------------------------------------------------
    static bool broadcast4(Shape const &out, Shape const &in, uint32_t (&stride)[4]) {
        if (out.size() > 4 || in.size() > out.size()) return false;
        uint32_t acc = 1;
        for (int d = 3; d >= 0; --d) {
            const int od = d - (4 - static_cast<int>(out.size()));
            const int id = od - static_cast<int>(out.size() - in.size());
            const uint32_t o = od >= 0 ? out[od] : 1, i = id >= 0 ? in[id] : 1;
            if (i != o && i != 1) return false;
            stride[d] = (i == 1 && o != 1) ? 0 : acc;
            acc *= i;
        }
        return true;
    }
    static void shape4(Shape const &out, uint32_t (&s)[4]) {
        for (int d = 0; d < 4; ++d) {
            const int od = d - (4 - static_cast<int>(out.size()));
            s[d] = od >= 0 ? out[od] : 1;
        }
    }

    std::vector<KernelBox> SimpleBinaryCollector::filter(TensorRefs inputs, TensorRefs outputs) const {
        std::vector<KernelBox> ans;
        auto const &a = inputs[0].get();
        auto const &b = inputs[1].get();
        auto const &y = outputs[0].get();
        if (_target != Target::Nvidia || a.dataType != b.dataType) return ans;
        {// the (operator, type) pairs the kernel library has: the sets BinaryCpu implements (simple_binary/cpu_kernel.cc:88-150)
            const bool logic = type == SimpleBinaryType::And || type == SimpleBinaryType::Or || type == SimpleBinaryType::Xor;
            bool ok;
            switch (a.dataType) {
                case DataType::F32: case DataType::FP16: case DataType::BF16: ok = !logic && type != SimpleBinaryType::Mod; break;
                case DataType::Bool: ok = logic; break;
                case DataType::U8: case DataType::I8: case DataType::I16: case DataType::I32: case DataType::U32: case DataType::I64: ok = !logic; break;
                default: ok = false;
            }
            if (!ok) return ans;
        }
        rg_binary_params p{};
        p.op = static_cast<int>(type);
        p.dtype = a.dataType;
        if (y.shape.size() > 4) return ans;
        shape4(y.shape, p.shape);
        if (!broadcast4(y.shape, a.shape, p.a_stride) || !broadcast4(y.shape, b.shape, p.b_stride)) return ans;
        ans.emplace_back(std::make_unique<BinaryB200>(p));
        return ans;
    }

    std::vector<KernelBox> SimpleUnaryCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        if (_target != Target::Nvidia) return ans;
        if (type == SimpleUnaryType::Not ? x.dataType != DataType::Bool : !halfOrFloat(x.dataType)) return ans;
        rg_unary_params p{};
        p.op = static_cast<int>(type);
        p.dtype = x.dataType;
        p.n = x.elementsSize();
        ans.emplace_back(std::make_unique<UnaryB200>(p));
        return ans;
    }

    std::vector<KernelBox> WhereCollector::filter(TensorRefs inputs, TensorRefs outputs) const {
        std::vector<KernelBox> ans;
        auto const &c = inputs[0].get();
        auto const &a = inputs[1].get();
        auto const &b = inputs[2].get();
        auto const &y = outputs[0].get();
        if (_target != Target::Nvidia || a.dataType != b.dataType || y.shape.size() > 4) return ans;
        rg_where_params p{};
        p.dtype = a.dataType;
        shape4(y.shape, p.shape);
        if (!broadcast4(y.shape, c.shape, p.c_stride) || !broadcast4(y.shape, a.shape, p.a_stride) ||
            !broadcast4(y.shape, b.shape, p.b_stride))
            return ans;
        ans.emplace_back(std::make_unique<WhereB200>(p));
        return ans;
    }

    std::vector<KernelBox> TransposeCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        if (_target != Target::Nvidia || x.shape.size() > 4 || x.shape.empty() || perm.size() != x.shape.size()) return ans;
        rg_transpose_params p{};
        p.elem_bytes = static_cast<uint32_t>(x.dataType.size());
        p.rank = static_cast<uint32_t>(x.shape.size());
        for (size_t i = 0; i < x.shape.size(); ++i) p.in_shape[i] = x.shape[i], p.perm[i] = perm[i];
        ans.emplace_back(std::make_unique<TransposeB200>(p));
        return ans;
    }

    // ---- Concat / Split / Slice / Expand / Cast: byte-exact movement, any data type ------------------------------------
    static bool asOuterAxisInner(Shape const &s, dim_t axis, rg_concat_params &p) {
        if (axis >= s.size()) return false;
        uint64_t outer = 1, inner = 1;
        for (size_t i = 0; i < axis; ++i) outer *= s[i];
        for (size_t i = axis + 1; i < s.size(); ++i) inner *= s[i];
        if (outer > 0xffffffffull || inner > 0xffffffffull) return false;
        p.outer = static_cast<uint32_t>(outer), p.inner = static_cast<uint32_t>(inner);
        return true;
    }
    std::vector<KernelBox> ConcatCollector::filter(TensorRefs inputs, TensorRefs outputs) const {
        std::vector<KernelBox> ans;
        if (_target != Target::Nvidia || inputs.empty() || inputs.size() > RG_CONCAT_MAX_PARTS || outputs.size() != 1) return ans;
        rg_concat_params p{};
        p.elem_bytes = static_cast<uint32_t>(outputs[0].get().dataType.size());
        p.n_parts = static_cast<uint32_t>(inputs.size());
        if (!asOuterAxisInner(outputs[0].get().shape, axis, p)) return ans;
        for (size_t i = 0; i < inputs.size(); ++i) {
            auto const &t = inputs[i].get();
            if (t.dataType != outputs[0].get().dataType || t.shape.size() != outputs[0].get().shape.size()) return ans;
            p.axis_len[i] = t.shape[axis];
        }
        ans.emplace_back(std::make_unique<ConcatB200>(p));
        return ans;
    }
    std::vector<KernelBox> SplitCollector::filter(TensorRefs inputs, TensorRefs outputs) const {
        std::vector<KernelBox> ans;
        if (_target != Target::Nvidia || inputs.empty() || outputs.empty() || outputs.size() > RG_CONCAT_MAX_PARTS) return ans;
        rg_concat_params p{};
        p.elem_bytes = static_cast<uint32_t>(inputs[0].get().dataType.size());
        p.n_parts = static_cast<uint32_t>(outputs.size());
        if (!asOuterAxisInner(inputs[0].get().shape, axis, p)) return ans;
        for (size_t i = 0; i < outputs.size(); ++i) {
            auto const &t = outputs[i].get();
            if (t.shape.size() != inputs[0].get().shape.size()) return ans;
            p.axis_len[i] = t.shape[axis];
        }
        ans.emplace_back(std::make_unique<SplitB200>(p));
        return ans;
    }
    std::vector<KernelBox> SliceCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        if (_target != Target::Nvidia || x.shape.size() > RG_MOVE_MAX_RANK || dims.size() != x.shape.size()) return ans;
        rg_slice_params p{};
        p.elem_bytes = static_cast<uint32_t>(x.dataType.size());
        p.rank = static_cast<uint32_t>(x.shape.size());
        for (size_t i = 0; i < dims.size(); ++i) {
            if (dims[i].length < 0) return ans;
            p.in_shape[i] = x.shape[i], p.start[i] = dims[i].start, p.step[i] = dims[i].step, p.length[i] = static_cast<uint32_t>(dims[i].length);
        }
        ans.emplace_back(std::make_unique<SliceB200>(p));
        return ans;
    }
    std::vector<KernelBox> ExpandCollector::filter(TensorRefs inputs, TensorRefs outputs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        auto const &y = outputs[0].get();
        if (_target != Target::Nvidia || y.shape.size() > RG_MOVE_MAX_RANK || x.shape.size() > y.shape.size() || x.dataType != y.dataType) return ans;
        rg_expand_params p{};
        p.elem_bytes = static_cast<uint32_t>(x.dataType.size());
        p.rank = static_cast<uint32_t>(y.shape.size());
        const size_t lead = y.shape.size() - x.shape.size();
        for (size_t i = 0; i < y.shape.size(); ++i) {
            p.out_shape[i] = y.shape[i];
            p.in_shape[i] = i < lead ? 1 : x.shape[i - lead];
            if (p.in_shape[i] != 1 && p.in_shape[i] != p.out_shape[i]) return ans;
        }
        ans.emplace_back(std::make_unique<ExpandB200>(p));
        return ans;
    }
    std::vector<KernelBox> CastCollector::filter(TensorRefs inputs, TensorRefs outputs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        auto const &y = outputs[0].get();
        if (_target != Target::Nvidia || x.elementsSize() != y.elementsSize()) return ans;
        auto known = [](int t) {
            switch (t) {
                case RG_F32: case RG_F64: case RG_FP16: case RG_BF16: case RG_I8: case RG_U8: case RG_I16: case RG_U16: case RG_I32: case RG_U32:
                case RG_I64: case RG_U64: case RG_BOOL: return true;
                default: return false;
            }
        };
        if (!known(x.dataType) || !known(y.dataType)) return ans;
        rg_cast_params p{};
        p.from = x.dataType, p.to = y.dataType, p.n = x.elementsSize();
        ans.emplace_back(std::make_unique<CastB200>(p));
        return ans;
    }

    std::vector<KernelBox> RotaryPositionEmbeddingCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        if (_target != Target::Nvidia || !halfOrFloat(x.dataType) || x.shape.size() != 3) return ans;
        if (inputs[1].get().dataType != DataType::I64) return ans;
        rg_rope_params p{};
        p.dtype = x.dataType;
        p.tokens = x.shape[0], p.heads = x.shape[1], p.head_dim = x.shape[2];
        p.theta = theta;
        ans.emplace_back(std::make_unique<RopeB200>(p));
        return ans;
    }

    std::vector<KernelBox> TopKCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        if (_target != Target::Nvidia || !halfOrFloat(x.dataType) || x.shape.empty()) return ans;
        rg_topk_params p{};
        p.dtype = x.dataType;
        p.n = x.shape.back();
        p.rows = p.n ? static_cast<uint32_t>(x.elementsSize() / p.n) : 0;
        p.k = k;
        p.softmax = softmax;
        if (k == 0 || k > 64 || k > p.n) return ans;
        ans.emplace_back(std::make_unique<TopKB200>(p));
        return ans;
    }

    std::vector<KernelBox> TopKSampleCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        if (_target != Target::Nvidia || !halfOrFloat(x.dataType) || x.shape.empty()) return ans;
        rg_topk_sample_params p{};
        p.dtype = x.dataType;
        p.n = x.shape.back();
        p.rows = p.n ? static_cast<uint32_t>(x.elementsSize() / p.n) : 0;
        p.k = k, p.temperature = temperature, p.seed = seed;
        if (k == 0 || k > 64 || k > p.n || !(temperature > 0)) return ans;
        ans.emplace_back(std::make_unique<TopKSampleB200>(p));
        return ans;
    }

    // ---- MatMul: MatMulInfo (src/04kernel/src/attributes/mat_mul_info.cc:27-42) -------------------------------------
    // Leading dims are multidirectionally broadcast (Broadcaster).  Equal or one-sided batches become one strided
    // launch; a general two-sided broadcast becomes one launch per output matrix, like the reference's host loop of
    // cublasGemmEx calls (src/04kernel/src/kernels/mat_mul/cublas_kernel.cu:60-85).
    struct MatMulB200 final : public Kernel {
        rg_mat_mul_params info;
        std::vector<std::pair<uint64_t, uint64_t>> offsets;// per output matrix (a, b) element offsets; empty = strided
        MatMulB200(rg_mat_mul_params p, decltype(offsets) o) noexcept : info(p), offsets(std::move(o)) {}
        RG_KERNEL_IDS(MatMulB200, "MatMul on B200 (tcgen05 / streaming GEMV / tiled CUDA-core kernels, no vendor GEMM)")
        void hintStaticInputs(std::vector<bool> const &isStatic) final {
            if (isStatic.size() > 1 && isStatic[1]) info.flags |= RG_MM_B_STATIC;
        }
        RoutineWorkspace lower(Resources &res) const final {
            auto st = res.fetchOrStore<CudaStream>();
            return RoutineWorkspace(
                [info = info, offsets = offsets, st](Resources &, void *ws, void const *const *in, void *const *out) {
                    if (offsets.empty()) {
                        check(rg_b200_mat_mul(&info, ws, in, out, st->stream), "rg_b200_mat_mul");
                        return;
                    }
                    const size_t es = DataType(static_cast<decltype(DataType::internal)>(info.dtype)).size();
                    for (size_t i = 0; i < offsets.size(); ++i) {
                        void const *in_[3] = {static_cast<uint8_t const *>(in[0]) + offsets[i].first * es,
                                              static_cast<uint8_t const *>(in[1]) + offsets[i].second * es,
                                              info.has_bias ? in[2] : nullptr};
                        void *out_[1] = {static_cast<uint8_t *>(out[0]) + i * static_cast<size_t>(info.m) * info.n * es};
                        check(rg_b200_mat_mul(&info, ws, in_, out_, st->stream), "rg_b200_mat_mul");
                    }
                },
                rg_b200_mat_mul_workspace(&info));
        }
    };

    std::vector<KernelBox> MatMulCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &a = inputs[0].get();
        auto const &b = inputs[1].get();
        if (_target != Target::Nvidia || !halfOrFloat(a.dataType) || a.dataType != b.dataType) return ans;
        if (a.shape.size() < 2 || b.shape.size() < 2) return ans;
        rg_mat_mul_params p{};
        p.dtype = a.dataType;
        p.trans_a = transA, p.trans_b = transB;
        p.alpha = alpha, p.beta = beta;
        auto ar = a.shape.rbegin(), br = b.shape.rbegin();
        p.m = transA ? ar[0] : ar[1];
        p.k = transA ? ar[1] : ar[0];
        p.n = transB ? br[1] : br[0];
        const dim_t kB = transB ? br[0] : br[1];
        if (p.k != kB) return ans;
        Shape la(a.shape.begin(), a.shape.end() - 2), lb(b.shape.begin(), b.shape.end() - 2);
        size_t na = 1, nb = 1;
        for (auto d : la) na *= d;
        for (auto d : lb) nb *= d;
        const size_t rank = std::max(la.size(), lb.size());
        Shape lo(rank, 1);
        for (size_t i = 0; i < rank; ++i) {
            const dim_t da = i < rank - la.size() ? 1 : la[i - (rank - la.size())];
            const dim_t db = i < rank - lb.size() ? 1 : lb[i - (rank - lb.size())];
            if (da != db && da != 1 && db != 1) return ans;
            lo[i] = std::max(da, db);
        }
        size_t no = 1;
        for (auto d : lo) no *= d;
        std::vector<std::pair<uint64_t, uint64_t>> offsets;
        const uint64_t sa = static_cast<uint64_t>(p.m) * p.k, sb = static_cast<uint64_t>(p.k) * p.n;
        if ((na == no || na == 1) && (nb == no || nb == 1)) {
            p.batch = static_cast<uint32_t>(no);
            p.stride_a = na == no && no > 1 ? sa : 0;
            p.stride_b = nb == no && no > 1 ? sb : 0;
        } else {
            p.batch = 1;
            for (size_t i = 0; i < no; ++i) {
                size_t rem = i, ia = 0, ib = 0, ma = 1, mb = 1;
                for (size_t d = rank; d-- > 0;) {
                    const dim_t idx = rem % lo[d];
                    rem /= lo[d];
                    const dim_t da = d < rank - la.size() ? 1 : la[d - (rank - la.size())];
                    const dim_t db = d < rank - lb.size() ? 1 : lb[d - (rank - lb.size())];
                    ia += (da == 1 ? 0 : idx) * ma, ma *= da;
                    ib += (db == 1 ? 0 : idx) * mb, mb *= db;
                }
                offsets.emplace_back(ia * sa, ib * sb);
            }
        }
        p.stride_y = static_cast<uint64_t>(p.m) * p.n;
        if (inputs.size() > 2) {
            auto const &c = inputs[2].get();
            // C must broadcast to [m, n] (unidirectional, no batch dims)
            Shape cs = c.shape;
            while (cs.size() > 2 && cs.front() == 1) cs.erase(cs.begin());
            if (cs.size() > 2) return ans;
            const dim_t cn = cs.empty() ? 1 : cs.back(), cm = cs.size() == 2 ? cs[0] : 1;
            if ((cn != 1 && cn != p.n) || (cm != 1 && cm != p.m)) return ans;
            p.has_bias = 1;
            p.bias_col_stride = cn == 1 ? 0 : 1;
            p.bias_row_stride = cm == 1 ? 0 : cn;
        }
        ans.emplace_back(std::make_unique<MatMulB200>(p, std::move(offsets)));
        return ans;
    }

    // ---- Attention (operator spec src/08-01llm/README.md:29-63) -----------------------------------------------------
    // inputs  {q, k, v} | {q, k, v, past_seq_len} | {q, k, v, past_seq_len, k_cache, v_cache}
    // outputs {o} | {o, k_cache, v_cache};  cache length = outputs[1].shape[2]
    // past_seq_len is read on the device at run time, so one lowered kernel serves every decode step.
    struct AttentionAdapterB200 final : public Kernel {
        rg_attention_params info;
        int nInputs;
        AttentionAdapterB200(rg_attention_params p, int n) noexcept : info(p), nInputs(n) {}
        RG_KERNEL_IDS(AttentionAdapterB200, "Causal attention with KV cache on B200")
        RoutineWorkspace lower(Resources &res) const final {
            auto st = res.fetchOrStore<CudaStream>();
            return RoutineWorkspace(
                [info = info, n = nInputs, st](Resources &, void *ws, void const *const *in, void *const *out) {
                    void const *in_[6] = {in[0], in[1], in[2], n > 3 ? in[3] : nullptr, n > 5 ? in[4] : nullptr, n > 5 ? in[5] : nullptr};
                    void *out_[3] = {out[0], info.has_cache ? out[1] : nullptr, info.has_cache ? out[2] : nullptr};
                    check(rg_b200_attention(&info, ws, in_, out_, st->stream), "rg_b200_attention");
                },
                rg_b200_attention_workspace(&info));
        }
    };
    std::vector<KernelBox> AttentionCollector::filter(TensorRefs inputs, TensorRefs outputs) const {
        std::vector<KernelBox> ans;
        auto const &q = inputs[0].get();
        auto const &k = inputs[1].get();
        if (_target != Target::Nvidia || !halfOrFloat(q.dataType) || q.shape.size() != 4 || k.shape.size() != 4) return ans;
        if (inputs.size() != 3 && inputs.size() != 4 && inputs.size() != 6) return ans;
        rg_attention_params p{};
        p.dtype = q.dataType;
        p.batch = q.shape[0], p.n_heads = q.shape[1], p.seq_len = q.shape[2], p.head_dim = q.shape[3];
        p.n_kv_heads = k.shape[1];
        p.has_cache = outputs.size() == 3;
        p.max_seq = p.has_cache ? outputs[1].get().shape[2] : p.seq_len;
        if (p.n_kv_heads == 0 || p.n_heads % p.n_kv_heads != 0) return ans;
        ans.emplace_back(std::make_unique<AttentionAdapterB200>(p, static_cast<int>(inputs.size())));
        return ans;
    }

    // ---- fused decode linear ---------------------------------------------------------------------------------------
    struct FusedLinearB200 final : public Kernel {
        rg_linear_params info;
        bool paged;
        FusedLinearB200(rg_linear_params p, bool paged_) noexcept : info(p), paged(paged_) {}
        RG_KERNEL_IDS(FusedLinearB200, "Fused RMSNorm + linear + epilogue on B200 (bulk-copy weight streaming for up to 32 tokens; tcgen05 GEMM for the prefill forms)")
        RoutineWorkspace lower(Resources &res) const final {
            auto st = res.fetchOrStore<CudaStream>();
            return RoutineWorkspace(
                [info = info, paged = paged, st](Resources &, void *ws, void const *const *in, void *const *out) {
                    // operator order {X, W, [G], [R], [positions, (block_table), k_cache, v_cache]} -> C ABI order.
                    // The caches are state edges of the graph: listed as inputs, appended to in place.
                    int i = 2;
                    void const *in_[6] = {in[0], in[1], nullptr, nullptr, nullptr, nullptr};
                    void *out_[3] = {out[0], nullptr, nullptr};
                    if (info.prologue == 1) in_[2] = in[i++];
                    if (info.epilogue == 1) in_[3] = in[i++];
                    if (info.epilogue == 3) {
                        in_[4] = in[i++];
                        if (paged) in_[5] = in[i++];
                        out_[1] = const_cast<void *>(in[i++]);
                        out_[2] = const_cast<void *>(in[i++]);
                    }
                    check(rg_b200_linear(&info, ws, in_, out_, st->stream), "rg_b200_linear");
                },
                rg_b200_linear_workspace(&info));
        }
    };
    std::vector<KernelBox> FusedLinearCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        auto const &w = inputs[1].get();
        if (_target != Target::Nvidia || !half(x.dataType) || w.dataType != x.dataType) return ans;
        if (x.shape.size() != 2 || w.shape.size() != 2 || x.shape[1] != w.shape[1]) return ans;
        // up to 4 tokens: the streaming kernel; 5..32 tokens without a norm prologue: the streaming skinny kernel; 5..64 tokens
        // with the SiLU gate, and more than 64 tokens with the QKV or SiLU-gate form: the tensor-core GEMM
        if (x.shape[0] > 4) {
            const bool qkv = epilogue == 3 && headDim == 128, gate = epilogue == 2 && w.shape[0] % 256 == 0;
            const bool skinny = x.shape[0] <= 32 && prologue == 0 && x.shape[1] % 128 == 0;
            // 5..64 tokens, SiLU gate: the tensor-core GEMM with the weights on the instruction's M side (gate rows in 64s)
            const bool gateSmall = x.shape[0] <= 64 && prologue == 0 && epilogue == 2 && w.shape[0] % 128 == 0 && x.shape[1] % 8 == 0 && x.shape[1] >= 64;
            // ... and the QKV split + RoPE + cache append (a 128-row tile of the weights = one head)
            const bool qkvSmall = x.shape[0] <= 64 && prologue == 0 && qkv && x.shape[1] % 8 == 0 && x.shape[1] >= 64;
            if (!skinny && !gateSmall && !qkvSmall && !(x.shape[0] > 64 && prologue == 0 && (qkv || gate))) return ans;
        }
        rg_linear_params p{};
        p.tokens_per_seq = static_cast<uint32_t>(tokensPerSeq);
        p.dtype = x.dataType;
        p.m = x.shape[0], p.k = x.shape[1], p.n = w.shape[0];
        p.prologue = prologue, p.epilogue = epilogue;
        p.epsilon = epsilon, p.theta = theta, p.n_heads = nHeads;
        p.kv.n_kv_heads = nKVHeads, p.kv.head_dim = headDim, p.kv.max_seq = maxSeq, p.kv.page_size = pageSize;
        bool paged = false;
        if (epilogue == 3) {
            const size_t expect = 2 + (prologue == 1) + 1 + 2;
            if (inputs.size() != expect && inputs.size() != expect + 1) return ans;
            paged = inputs.size() == expect + 1;
            auto const &kc = inputs[inputs.size() - 2].get();
            if (kc.shape.size() != 4) return ans;
            if (paged) {
                p.kv.max_blocks_per_seq = inputs[inputs.size() - 3].get().shape.back();
                p.kv.n_blocks = kc.shape[0];
                if (!p.kv.page_size) p.kv.page_size = kc.shape[2];
            } else if (!p.kv.max_seq) {
                p.kv.max_seq = kc.shape[2];
            }
        }
        ans.emplace_back(std::make_unique<FusedLinearB200>(p, paged));
        return ans;
    }

    // ---- flash-decoding ----------------------------------------------------------------------------------------------
    // The workspace carries arrival counters that must start at zero; the Stream zero-fills its stack once at
    // lower time and the kernel leaves the counters at zero after every call.
    struct AttentionDecodeB200 final : public Kernel {
        rg_attn_decode_params info;
        bool paged;
        AttentionDecodeB200(rg_attn_decode_params p, bool paged_) noexcept : info(p), paged(paged_) {}
        RG_KERNEL_IDS(AttentionDecodeB200, "Split-K flash-decoding over a (paged) KV cache on B200 (bulk-copy staged tiles)")
        RoutineWorkspace lower(Resources &res) const final {
            auto st = res.fetchOrStore<CudaStream>();
            return RoutineWorkspace(
                [info = info, paged = paged, st](Resources &, void *ws, void const *const *in, void *const *out) {
                    void const *in_[5] = {in[0], in[1], in[2], in[3], paged ? in[4] : nullptr};
                    check(rg_b200_attn_decode(&info, ws, in_, out, st->stream), "rg_b200_attn_decode");
                },
                rg_b200_attn_decode_workspace(&info));
        }
    };
    std::vector<KernelBox> AttentionDecodeCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &q = inputs[0].get();
        auto const &kc = inputs[1].get();
        if (_target != Target::Nvidia || !half(q.dataType) || q.shape.size() != 3 || kc.shape.size() != 4) return ans;
        rg_attn_decode_params p{};
        p.dtype = q.dataType;
        p.batch = q.shape[0], p.n_heads = q.shape[1];
        p.max_len = maxLen;
        p.kv.n_kv_heads = kc.shape[1], p.kv.head_dim = q.shape[2];
        const bool paged = inputs.size() == 5;
        if (paged) {
            p.kv.page_size = pageSize ? pageSize : kc.shape[2];
            p.kv.max_blocks_per_seq = inputs[4].get().shape.back();
            p.kv.n_blocks = kc.shape[0];
        } else {
            p.kv.max_seq = kc.shape[2];
        }
        ans.emplace_back(std::make_unique<AttentionDecodeB200>(p, paged));
        return ans;
    }

    struct QkvRopeAppendB200 final : public Kernel {
        rg_qkv_rope_append_params info;
        bool paged;
        QkvRopeAppendB200(rg_qkv_rope_append_params p, bool paged_) noexcept : info(p), paged(paged_) {}
        RG_KERNEL_IDS(QkvRopeAppendB200, "QKV split + RoPE + cache append on B200")
        RoutineWorkspace lower(Resources &res) const final {
            auto st = res.fetchOrStore<CudaStream>();
            return RoutineWorkspace([info = info, paged = paged, st](Resources &, void *ws, void const *const *in, void *const *out) {
                int i = 2;
                void const *in_[3] = {in[0], in[1], paged ? in[i++] : nullptr};
                void *out_[3] = {out[0], const_cast<void *>(in[i]), const_cast<void *>(in[i + 1])};
                check(rg_b200_qkv_rope_append(&info, ws, in_, out_, st->stream), "rg_b200_qkv_rope_append");
            });
        }
    };
    std::vector<KernelBox> QkvRopeAppendCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        if (_target != Target::Nvidia || !halfOrFloat(x.dataType) || x.shape.size() != 2) return ans;
        if (inputs.size() != 4 && inputs.size() != 5) return ans;
        const bool paged = inputs.size() == 5;
        auto const &kc = inputs[inputs.size() - 2].get();
        if (kc.shape.size() != 4 || x.shape[1] != (nHeads + 2 * nKVHeads) * headDim) return ans;
        rg_qkv_rope_append_params p{};
        p.dtype = x.dataType;
        p.tokens = x.shape[0], p.n_heads = nHeads, p.theta = theta;
        p.tokens_per_seq = tokensPerSeq;
        p.kv.n_kv_heads = nKVHeads, p.kv.head_dim = headDim;
        if (paged) {
            p.kv.page_size = pageSize ? pageSize : kc.shape[2];
            p.kv.max_blocks_per_seq = inputs[2].get().shape.back();
            p.kv.n_blocks = kc.shape[0];
        } else {
            p.kv.max_seq = kc.shape[2];
        }
        ans.emplace_back(std::make_unique<QkvRopeAppendB200>(p, paged));
        return ans;
    }

    struct AttentionPrefillB200 final : public Kernel {
        rg_attn_prefill_params info;
        bool hasPast;
        AttentionPrefillB200(rg_attn_prefill_params p, bool hasPast_) noexcept : info(p), hasPast(hasPast_) {}
        RG_KERNEL_IDS(AttentionPrefillB200, "Causal flash attention (prefill) on B200")
        RoutineWorkspace lower(Resources &res) const final {
            auto st = res.fetchOrStore<CudaStream>();
            return RoutineWorkspace([info = info, hasPast = hasPast, st](Resources &, void *ws, void const *const *in, void *const *out) {
                void const *in_[4] = {in[0], in[1], in[2], hasPast ? in[3] : nullptr};
                check(rg_b200_attn_prefill(&info, ws, in_, out, st->stream), "rg_b200_attn_prefill");
            });
        }
    };
    std::vector<KernelBox> AttentionPrefillCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &q = inputs[0].get();
        auto const &kc = inputs[1].get();
        if (_target != Target::Nvidia || !half(q.dataType) || q.shape.size() != 2 || kc.shape.size() != 4 || seqLen == 0) return ans;
        if (inputs.size() != 3 && inputs.size() != 4) return ans;
        const dim_t D = kc.shape[3], nKV = kc.shape[1], maxSeq = kc.shape[2], B = q.shape[0] / seqLen;
        if (D != 128 || q.shape[1] != nHeads * D || B * seqLen != q.shape[0] || kc.shape[0] != B) return ans;
        rg_attn_prefill_params p{};
        p.dtype = q.dataType;
        p.batch = B, p.n_heads = nHeads, p.n_kv_heads = nKV, p.seq_len = seqLen, p.head_dim = D, p.kv_capacity = maxSeq;
        const int64_t qrow = static_cast<int64_t>(nHeads) * D;
        const int64_t s[12] = {static_cast<int64_t>(seqLen) * qrow, D, qrow,
                               static_cast<int64_t>(nKV) * maxSeq * D, static_cast<int64_t>(maxSeq) * D, D,
                               static_cast<int64_t>(nKV) * maxSeq * D, static_cast<int64_t>(maxSeq) * D, D,
                               static_cast<int64_t>(seqLen) * qrow, D, qrow};
        for (int i = 0; i < 12; ++i) p.strides[i] = s[i];
        ans.emplace_back(std::make_unique<AttentionPrefillB200>(p, inputs.size() == 4));
        return ans;
    }

    RG_SIMPLE_KERNEL(SwigluB200, rg_swiglu_params, rg_b200_swiglu, "SiLU gate on B200");
    std::vector<KernelBox> SwigluCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        if (_target != Target::Nvidia || !halfOrFloat(x.dataType) || x.shape.empty() || x.shape.back() % 2 != 0) return ans;
        rg_swiglu_params p{};
        p.dtype = x.dataType;
        p.f = x.shape.back() / 2;
        p.rows = static_cast<uint32_t>(x.elementsSize() / x.shape.back());
        ans.emplace_back(std::make_unique<SwigluB200>(p));
        return ans;
    }

    RG_SIMPLE_KERNEL(DecodeStepB200, rg_decode_step_params, rg_b200_decode_step, "Whole batch-1 decode step as one persistent kernel on B200");
    std::vector<KernelBox> DecodeStepCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        if (_target != Target::Nvidia || inputs.size() < 5 || (inputs.size() - 5) % 8 != 0) return ans;
        auto const &embed = inputs[2].get();
        if (!half(embed.dataType) || embed.shape.size() != 2) return ans;
        rg_decode_step_params p{};
        p.dtype = embed.dataType;
        p.layers = static_cast<uint32_t>((inputs.size() - 5) / 8);
        p.vocab = embed.shape[0], p.hidden = embed.shape[1];
        p.n_heads = nHeads, p.n_kv_heads = nKVHeads, p.head_dim = headDim;
        p.epsilon = epsilon, p.theta = theta;
        if (p.layers) {
            auto const &wgu = inputs[5 + 4].get();
            auto const &kc = inputs[5 + 6].get();
            if (wgu.shape.size() != 2 || kc.shape.size() != 4 || kc.shape[0] != 1) return ans;
            p.ffn = wgu.shape[0] / 2;
            p.max_seq = kc.shape[2];
        }
        ans.emplace_back(std::make_unique<DecodeStepB200>(p));
        return ans;
    }

    // state (outputs[0] aliases inputs[0] in the graph) = (src ? src : state) + delta
    std::vector<KernelBox> StateUpdateCollector::filter(TensorRefs inputs, TensorRefs) const {
        std::vector<KernelBox> ans;
        auto const &s = inputs[0].get();
        if (_target != Target::Nvidia || s.dataType != DataType::I64) return ans;
        if (inputs.size() > 1 && (inputs[1].get().dataType != DataType::I64 || inputs[1].get().elementsSize() < s.elementsSize())) return ans;
        rg_state_update_params p{};
        p.n = static_cast<uint32_t>(s.elementsSize());
        p.delta = delta;
        ans.emplace_back(std::make_unique<StateUpdateB200>(p, inputs.size() > 1));
        return ans;
    }

    // ---- AllReduce (src/04kernel/src/kernels/all_reduce/nccl_kernel.cu:9-19) ------------------------------------------
    // The communicator lives in Resources, as NcclCommunicator does in the reference (nccl_kernel.cu:13); it is
    // stored there by whoever builds the Stream for this rank (graph.cc, from world/rank).
    struct CommResource final : public runtime::Resource {
        rg_comm *comm;
        bool owned;
        explicit CommResource(rg_comm *c, bool owned_ = false) : comm(c), owned(owned_) {}
        ~CommResource() override {
            if (comm && owned) rg_b200_comm_destroy(comm);
        }
        static size_t typeId() noexcept {
            static uint8_t ID = 1;
            return reinterpret_cast<size_t>(&ID);
        }
        size_t resourceTypeId() const noexcept override { return typeId(); }
        std::string_view description() const noexcept override { return "NVLink peer-memory communicator"; }
    };
    runtime::ResourceBox makeCommResource(void *comm) { return std::make_unique<CommResource>(static_cast<rg_comm *>(comm)); }

    struct AllReduceB200 final : public Kernel {
        rg_all_reduce_params info;
        bool hasResidual;
        AllReduceB200(rg_all_reduce_params p, bool r) noexcept : info(p), hasResidual(r) {}
        RG_KERNEL_IDS(AllReduceB200, "AllReduce over NVLink peer memory on B200 (flag-in-data push, one- or two-shot, rank-order combine)")
        RoutineWorkspace lower(Resources &res) const final {
            auto st = res.fetchOrStore<CudaStream>();
            return RoutineWorkspace([info = info, r = hasResidual, st](Resources &res, void *, void const *const *in, void *const *out) {
                auto comm = res.fetch<CommResource>();
                if (!comm) RUNTIME_ERROR("AllReduce: no communicator in Resources");
                void const *in_[2] = {in[0], r ? in[1] : nullptr};
                check(rg_b200_all_reduce(comm->comm, &info, in_, out, st->stream), "rg_b200_all_reduce");
            });
        }
    };
    std::vector<KernelBox> AllReduceCollector::filter(TensorRefs inputs, TensorRefs outputs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        auto const &y = outputs[0].get();
        if (_target != Target::Nvidia) return ans;
        switch (x.dataType) {// the set the reference's communicator maps to NCCL types
            case RG_F32: case RG_FP16: case RG_BF16: case RG_F64: case RG_U8: case RG_I8: case RG_I32: case RG_U32: case RG_I64: break;
            default: return ans;
        }
        if (x.elementsSize() != y.elementsSize() || x.dataType != y.dataType) return ans;// nccl_kernel.cc:14-17
        rg_all_reduce_params p{};
        p.dtype = x.dataType;
        p.op = static_cast<int>(type);
        p.count = x.elementsSize();
        ans.emplace_back(std::make_unique<AllReduceB200>(p, inputs.size() > 1));
        return ans;
    }

    // ---- Row-parallel product whose epilogue is the sending half of the all-reduce, then the receiving half ---------------
    struct MatMulAllReduceB200 final : public Kernel {
        rg_mat_mul_params mm;
        rg_all_reduce_params ar;
        bool hasResidual;
        MatMulAllReduceB200(rg_mat_mul_params m, rg_all_reduce_params a, bool r) noexcept : mm(m), ar(a), hasResidual(r) {}
        RG_KERNEL_IDS(MatMulAllReduceB200, "tcgen05 product that stores into the peers' all-reduce slots over NVLink, then the receiving half of the all-reduce, on B200")
        RoutineWorkspace lower(Resources &res) const final {
            auto st = res.fetchOrStore<CudaStream>();
            return RoutineWorkspace(
                [mm = mm, ar = ar, r = hasResidual, st](Resources &res, void *ws, void const *const *in, void *const *out) {
                    auto comm = res.fetch<CommResource>();
                    if (!comm) RUNTIME_ERROR("MatMulAllReduce: no communicator in Resources");
                    void const *in_[2] = {in[0], in[1]};
                    check(rg_b200_mat_mul_push(comm->comm, &mm, ws, in_, st->stream), "rg_b200_mat_mul_push");
                    void const *res_[1] = {r ? in[2] : nullptr};
                    check(rg_b200_all_reduce_recv(comm->comm, &ar, res_, out, st->stream), "rg_b200_all_reduce_recv");
                },
                rg_b200_mat_mul_workspace(&mm));
        }
    };
    std::vector<KernelBox> MatMulAllReduceCollector::filter(TensorRefs inputs, TensorRefs outputs) const {
        std::vector<KernelBox> ans;
        if (_target != Target::Nvidia || inputs.size() < 2 || inputs.size() > 3 || outputs.size() != 1) return ans;
        auto const &x = inputs[0].get();
        auto const &w = inputs[1].get();
        if ((x.dataType != RG_FP16 && x.dataType != RG_BF16) || w.dataType != x.dataType) return ans;
        if (x.shape.size() != 2 || w.shape.size() != 2 || x.shape[1] != w.shape[1]) return ans;
        // what rg_b200_mat_mul_push takes: up to 64 tokens, whole 16-byte chunks per output row
        if (x.shape[0] == 0 || x.shape[0] > 64 || w.shape[0] < 128 || w.shape[0] % 8 != 0 || x.shape[1] % 8 != 0 || x.shape[1] < 64) return ans;
        rg_mat_mul_params mm{};
        mm.dtype = x.dataType;
        mm.m = x.shape[0], mm.n = w.shape[0], mm.k = x.shape[1];
        mm.trans_b = 1, mm.alpha = alpha, mm.beta = 0.f, mm.batch = 1;
        mm.flags = RG_MM_B_STATIC;// the weight operand is a graph input or constant: nothing in the stream writes it
        rg_all_reduce_params ar{};
        ar.dtype = x.dataType, ar.op = 0, ar.count = static_cast<uint64_t>(mm.m) * mm.n;
        ans.emplace_back(std::make_unique<MatMulAllReduceB200>(mm, ar, inputs.size() == 3));
        return ans;
    }

    // ---- AllReduce(Sum) + residual + RmsNormalization in one launch (what the fusion pass makes of the three operators) ----
    struct AllReduceNormB200 final : public Kernel {
        rg_all_reduce_norm_params info;
        bool hasResidual;
        AllReduceNormB200(rg_all_reduce_norm_params p, bool r) noexcept : info(p), hasResidual(r) {}
        RG_KERNEL_IDS(AllReduceNormB200, "AllReduce + residual + RMS normalization over NVLink peer memory on B200 (one launch, one CTA per row)")
        RoutineWorkspace lower(Resources &res) const final {
            auto st = res.fetchOrStore<CudaStream>();
            return RoutineWorkspace([info = info, r = hasResidual, st](Resources &res, void *, void const *const *in, void *const *out) {
                auto comm = res.fetch<CommResource>();
                if (!comm) RUNTIME_ERROR("AllReduceNorm: no communicator in Resources");
                void const *in_[3] = {in[0], r ? in[1] : nullptr, r ? in[2] : in[1]};
                check(rg_b200_all_reduce_norm(comm->comm, &info, in_, out, st->stream), "rg_b200_all_reduce_norm");
            });
        }
    };
    std::vector<KernelBox> AllReduceNormCollector::filter(TensorRefs inputs, TensorRefs outputs) const {
        std::vector<KernelBox> ans;
        auto const &x = inputs[0].get();
        if (_target != Target::Nvidia || (x.dataType != RG_FP16 && x.dataType != RG_BF16) || x.shape.empty()) return ans;
        if (outputs.size() != 2 || inputs.size() < 2 || inputs.size() > 3) return ans;
        rg_all_reduce_norm_params p{};
        p.dtype = x.dataType;
        p.dim = x.shape.back();
        p.rows = p.dim ? static_cast<uint32_t>(x.elementsSize() / p.dim) : 0;
        p.epsilon = epsilon;
        if (p.dim % 8 != 0 || p.dim > 16384 || inputs.back().get().elementsSize() != p.dim) return ans;
        ans.emplace_back(std::make_unique<AllReduceNormB200>(p, inputs.size() == 3));
        return ans;
    }

}// namespace refactor::kernel
