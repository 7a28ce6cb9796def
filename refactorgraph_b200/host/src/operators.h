// Operator classes of the decoder path (private to the host layer: computation.cc builds them from names and
// attributes, fusion.cc rewrites graphs of them).
#pragma once
#include "rg/graph.h"
#include <algorithm>

namespace refactor::computation {
    using namespace kernel;

    inline int64_t getInt(Attributes const &a, char const *k, int64_t dflt) {
        auto it = a.find(k);
        if (it == a.end()) return dflt;
        if (auto p = std::get_if<int64_t>(&it->second)) return *p;
        if (auto p = std::get_if<double>(&it->second)) return static_cast<int64_t>(*p);
        RUNTIME_ERROR(std::string("attribute ") + k + " is not a number");
    }
    inline double getFloat(Attributes const &a, char const *k, double dflt) {
        auto it = a.find(k);
        if (it == a.end()) return dflt;
        if (auto p = std::get_if<double>(&it->second)) return *p;
        if (auto p = std::get_if<int64_t>(&it->second)) return static_cast<double>(*p);
        RUNTIME_ERROR(std::string("attribute ") + k + " is not a number");
    }
    inline std::vector<int64_t> getInts(Attributes const &a, char const *k) {
        auto it = a.find(k);
        if (it == a.end()) return {};
        if (auto p = std::get_if<std::vector<int64_t>>(&it->second)) return *p;
        RUNTIME_ERROR(std::string("attribute ") + k + " is not an int list");
    }
    inline Shape broadcastShape(Shape const &a, Shape const &b) {
        const size_t r = std::max(a.size(), b.size());
        Shape o(r, 1);
        for (size_t i = 0; i < r; ++i) {
            const dim_t da = i < r - a.size() ? 1 : a[i - (r - a.size())];
            const dim_t db = i < r - b.size() ? 1 : b[i - (r - b.size())];
            ASSERT(da == db || da == 1 || db == 1, "shapes cannot be broadcast");
            o[i] = std::max(da, db);
        }
        return o;
    }
    inline std::vector<Arc<Tensor>> one(DataType dt, Shape s) { return {Tensor::share(dt, std::move(s))}; }

#define RG_OP(TYPE, STR)                                 \
    std::string_view name() const final { return STR; }  \
    OpBox clone() const final { return std::make_unique<TYPE>(*this); }

    struct RmsNormalization final : Operator {
        float epsilon;
        explicit RmsNormalization(float e) : epsilon(e) {}
        RG_OP(RmsNormalization, "RmsNormalization")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<RmsNormalizationCollector>(t, epsilon); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            ASSERT(in.size() == 2, "RmsNormalization takes x and w");
            ASSERT(in[1].get().shape.size() == 1 && in[1].get().shape[0] == in[0].get().shape.back(), "RmsNormalization: w must be [D]");
            return one(in[0].get().dataType, in[0].get().shape);
        }
    };
    struct MatMul final : Operator {
        float alpha, beta;
        bool transA, transB;
        MatMul(float a, float b, bool ta, bool tb) : alpha(a), beta(b), transA(ta), transB(tb) {}
        RG_OP(MatMul, "MatMul")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<MatMulCollector>(t, alpha, beta, transA, transB); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            ASSERT(in.size() == 2 || in.size() == 3, "MatMul takes 2 or 3 inputs");
            auto const &a = in[0].get().shape;
            auto const &b = in[1].get().shape;
            ASSERT(a.size() >= 2 && b.size() >= 2, "MatMul: rank < 2");
            const dim_t m = transA ? a[a.size() - 1] : a[a.size() - 2], k = transA ? a[a.size() - 2] : a[a.size() - 1];
            const dim_t n = transB ? b[b.size() - 2] : b[b.size() - 1], kb = transB ? b[b.size() - 1] : b[b.size() - 2];
            ASSERT(k == kb, "MatMul: input shape not matched.");
            Shape o = broadcastShape(Shape(a.begin(), a.end() - 2), Shape(b.begin(), b.end() - 2));
            o.push_back(m), o.push_back(n);
            return one(in[0].get().dataType, o);
        }
    };
    struct Softmax final : Operator {
        int64_t axis;
        explicit Softmax(int64_t a) : axis(a) {}
        RG_OP(Softmax, "Softmax")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<SoftmaxCollector>(t, static_cast<dim_t>(axis)); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final { return one(in[0].get().dataType, in[0].get().shape); }
    };
    // src/08-01llm/src/operators/attention.cc:37-128: output shapes for the six input/attribute cases
    struct Attention final : Operator {
        dim_t maxSeqLen;
        explicit Attention(dim_t m) : maxSeqLen(m) {}
        RG_OP(Attention, "Attention")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<AttentionCollector>(t, maxSeqLen); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            ASSERT(in.size() == 3 || in.size() == 4 || in.size() == 6, "Attention takes 3, 4 or 6 inputs");
            auto const &q = in[0].get();
            auto const &k = in[1].get();
            ASSERT(q.shape.size() == 4 && k.shape.size() == 4 && in[2].get().shape == k.shape, "Attention: q/k/v must be rank 4");
            ASSERT(q.shape[0] == k.shape[0] && q.shape[2] == k.shape[2] && q.shape[3] == k.shape[3], "Attention: q/k shapes not matched");
            ASSERT(k.shape[1] > 0 && q.shape[1] % k.shape[1] == 0, "Attention: n_head must be a multiple of n_kv_head");
            std::vector<Arc<Tensor>> out = one(q.dataType, q.shape);
            if (in.size() == 3 && maxSeqLen == 0) return out;
            dim_t cache = maxSeqLen;
            if (cache == 0) {
                // past_seq_len must be a constant when max_seq_len is not given (README cases 3 and 5)
                auto const &p = in[3].get();
                ASSERT(p.data && p.dataType == DataType::I64, "Attention: past_seq_len must be a constant int64 when max_seq_len is 0");
                cache = static_cast<dim_t>(*reinterpret_cast<int64_t const *>(p.data->bytes.data())) + q.shape[2];
            }
            ASSERT(cache >= q.shape[2], "Attention: cache shorter than seq_len");
            Shape cs{k.shape[0], k.shape[1], cache, k.shape[3]};
            out.push_back(Tensor::share(q.dataType, cs));
            out.push_back(Tensor::share(q.dataType, cs));
            return out;
        }
    };
    struct AllReduce final : Operator {
        AllReduceType type;
        explicit AllReduce(AllReduceType t) : type(t) {}
        RG_OP(AllReduce, "AllReduce")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<AllReduceCollector>(t, type); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final { return one(in[0].get().dataType, in[0].get().shape); }
    };
    struct MatMulAllReduce final : Operator {
        float alpha;
        explicit MatMulAllReduce(float a) : alpha(a) {}
        RG_OP(MatMulAllReduce, "MatMulAllReduce")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<MatMulAllReduceCollector>(t, alpha); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            ASSERT((in.size() == 2 || in.size() == 3) && in[0].get().shape.size() == 2 && in[1].get().shape.size() == 2,
                   "MatMulAllReduce takes x[m, k], w[n, k] and an optional residual");
            return one(in[0].get().dataType, Shape{in[0].get().shape[0], in[1].get().shape[0]});
        }
    };
    struct AllReduceNorm final : Operator {
        float epsilon;
        explicit AllReduceNorm(float e) : epsilon(e) {}
        RG_OP(AllReduceNorm, "AllReduceNorm")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<AllReduceNormCollector>(t, epsilon); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            ASSERT(in.size() == 2 || in.size() == 3, "AllReduceNorm takes x, an optional residual and the norm weight");
            return {Tensor::share(in[0].get().dataType, in[0].get().shape), Tensor::share(in[0].get().dataType, in[0].get().shape)};
        }
    };
    struct Gather final : Operator {
        int64_t axis;
        explicit Gather(int64_t a) : axis(a) {}
        RG_OP(Gather, "Gather")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<GatherCollector>(t, static_cast<dim_t>(axis)); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            auto const &d = in[0].get().shape;
            auto const &i = in[1].get().shape;
            ASSERT(static_cast<size_t>(axis) < d.size(), "Gather: axis out of range");
            Shape o(d.begin(), d.begin() + axis);
            o.insert(o.end(), i.begin(), i.end());
            o.insert(o.end(), d.begin() + axis + 1, d.end());
            return one(in[0].get().dataType, o);
        }
    };
    struct SimpleBinary final : Operator {
        SimpleBinaryType type;
        explicit SimpleBinary(SimpleBinaryType t) : type(t) {}
        RG_OP(SimpleBinary, "SimpleBinary")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<SimpleBinaryCollector>(t, type); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            return one(in[0].get().dataType, broadcastShape(in[0].get().shape, in[1].get().shape));
        }
    };
    struct SimpleUnary final : Operator {
        SimpleUnaryType type;
        explicit SimpleUnary(SimpleUnaryType t) : type(t) {}
        RG_OP(SimpleUnary, "SimpleUnary")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<SimpleUnaryCollector>(t, type); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final { return one(in[0].get().dataType, in[0].get().shape); }
    };
    struct Transpose final : Operator {
        std::vector<dim_t> perm;
        explicit Transpose(std::vector<dim_t> p) : perm(std::move(p)) {}
        RG_OP(Transpose, "Transpose")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<TransposeCollector>(t, perm); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            auto const &s = in[0].get().shape;
            ASSERT(perm.size() == s.size(), "Transpose: perm rank mismatch");
            Shape o(s.size());
            for (size_t i = 0; i < s.size(); ++i) o[i] = s[perm[i]];
            return one(in[0].get().dataType, o);
        }
    };
    // ---- data movement (ONNX semantics; negative axes count from the end) ----
    inline dim_t normAxis(int64_t axis, size_t rank) {
        if (axis < 0) axis += static_cast<int64_t>(rank);
        ASSERT(axis >= 0 && static_cast<size_t>(axis) < rank, "axis out of range");
        return static_cast<dim_t>(axis);
    }
    struct Concat final : Operator {
        int64_t axis;
        explicit Concat(int64_t a) : axis(a) {}
        RG_OP(Concat, "Concat")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<ConcatCollector>(t, resolved); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            ASSERT(!in.empty(), "Concat needs an input");
            Shape o = in[0].get().shape;
            resolved = normAxis(axis, o.size());
            o[resolved] = 0;
            for (auto const &t : in) {
                auto const &s = t.get().shape;
                ASSERT(s.size() == o.size() && t.get().dataType == in[0].get().dataType, "Concat: rank or type mismatch");
                for (size_t i = 0; i < s.size(); ++i) {
                    ASSERT(i == resolved || s[i] == o[i], "Concat: shapes differ outside the axis");
                }
                o[resolved] += s[resolved];
            }
            return one(in[0].get().dataType, o);
        }
        mutable dim_t resolved = 0;// axis >= 0, known once the input rank is
    };
    struct Split final : Operator {
        int64_t axis;
        std::vector<int64_t> sizes;// empty: equal parts, one per output
        dim_t nOut;
        Split(int64_t a, std::vector<int64_t> s, dim_t n) : axis(a), sizes(std::move(s)), nOut(n) {}
        RG_OP(Split, "Split")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<SplitCollector>(t, resolved); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            auto const &x = in[0].get();
            resolved = normAxis(axis, x.shape.size());
            std::vector<int64_t> parts = sizes;
            if (parts.empty()) {
                ASSERT(nOut > 0 && x.shape[resolved] % nOut == 0, "Split: the axis does not divide into equal parts");
                parts.assign(nOut, x.shape[resolved] / nOut);
            }
            int64_t sum = 0;
            for (auto v : parts) {
                ASSERT(v >= 0, "Split: negative part");
                sum += v;
            }
            ASSERT(sum == static_cast<int64_t>(x.shape[resolved]), "Split: parts do not add up to the axis");
            std::vector<Arc<Tensor>> out;
            for (auto v : parts) {
                Shape o = x.shape;
                o[resolved] = static_cast<dim_t>(v);
                out.push_back(Tensor::share(x.dataType, o));
            }
            return out;
        }
        mutable dim_t resolved = 0;
    };
    // starts / ends / axes / steps as ONNX Slice defines them (clamped ends, negative indices, negative steps)
    struct Slice final : Operator {
        std::vector<int64_t> starts, ends, axes, steps;
        Slice(std::vector<int64_t> s, std::vector<int64_t> e, std::vector<int64_t> a, std::vector<int64_t> st)
            : starts(std::move(s)), ends(std::move(e)), axes(std::move(a)), steps(std::move(st)) {}
        RG_OP(Slice, "Slice")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<SliceCollector>(t, dims); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            auto const &x = in[0].get();
            const size_t rank = x.shape.size();
            ASSERT(starts.size() == ends.size() && (axes.empty() || axes.size() == starts.size()) && (steps.empty() || steps.size() == starts.size()),
                   "Slice: starts, ends, axes and steps must have one entry per sliced axis");
            dims.assign(rank, SliceDim{0, 1, 0});
            for (size_t d = 0; d < rank; ++d) dims[d].length = x.shape[d];
            for (size_t i = 0; i < starts.size(); ++i) {
                const dim_t d = normAxis(axes.empty() ? static_cast<int64_t>(i) : axes[i], rank);
                const int64_t n = x.shape[d], step = steps.empty() ? 1 : steps[i];
                ASSERT(step != 0, "Slice: step 0");
                int64_t s = starts[i] < 0 ? starts[i] + n : starts[i], e = ends[i] < 0 ? ends[i] + n : ends[i];
                if (step > 0) {
                    s = std::min(std::max<int64_t>(s, 0), n), e = std::min(std::max<int64_t>(e, 0), n);
                    dims[d] = SliceDim{s, step, e > s ? (e - s + step - 1) / step : 0};
                } else {
                    s = std::min(std::max<int64_t>(s, -1), n - 1), e = std::min(std::max<int64_t>(e, -1), n - 1);
                    dims[d] = SliceDim{s, step, s > e ? (s - e - step - 1) / (-step) : 0};
                }
            }
            Shape o(rank);
            for (size_t d = 0; d < rank; ++d) o[d] = static_cast<dim_t>(dims[d].length);
            return one(x.dataType, o);
        }
        mutable SliceDimensions dims;
    };
    struct Cast final : Operator {
        DataType to;
        explicit Cast(DataType t) : to(t) {}
        RG_OP(Cast, "Cast")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<CastCollector>(t); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final { return one(to, in[0].get().shape); }
    };
    struct Expand final : Operator {
        std::vector<int64_t> shape;
        explicit Expand(std::vector<int64_t> s) : shape(std::move(s)) {}
        RG_OP(Expand, "Expand")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<ExpandCollector>(t); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            Shape want(shape.size());
            for (size_t i = 0; i < shape.size(); ++i) {
                ASSERT(shape[i] >= 0, "Expand: negative dimension");
                want[i] = static_cast<dim_t>(shape[i]);
            }
            return one(in[0].get().dataType, broadcastShape(in[0].get().shape, want));
        }
    };
    struct Reshape final : Operator {
        std::vector<int64_t> shape;
        explicit Reshape(std::vector<int64_t> s) : shape(std::move(s)) {}
        RG_OP(Reshape, "Reshape")
        bool isIdentity() const final { return true; }
        CollectorBox candidateKernels(Target) const final { return nullptr; }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            const size_t total = in[0].get().elementsSize();
            Shape o(shape.size());
            size_t known = 1;
            int infer_at = -1;
            for (size_t i = 0; i < shape.size(); ++i) {
                if (shape[i] == -1) infer_at = static_cast<int>(i);
                else {
                    o[i] = shape[i] == 0 ? in[0].get().shape[i] : static_cast<dim_t>(shape[i]);
                    known *= o[i];
                }
            }
            if (infer_at >= 0) o[infer_at] = static_cast<dim_t>(total / (known ? known : 1));
            auto t = Tensor::share(in[0].get().dataType, o);
            ASSERT(t->elementsSize() == total, "Reshape: element count changed");
            return {t};
        }
    };
    struct Where final : Operator {
        RG_OP(Where, "Where")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<WhereCollector>(t); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            return one(in[1].get().dataType, broadcastShape(in[0].get().shape, broadcastShape(in[1].get().shape, in[2].get().shape)));
        }
    };
    struct RotaryPositionEmbedding final : Operator {
        float theta;
        explicit RotaryPositionEmbedding(float t) : theta(t) {}
        RG_OP(RotaryPositionEmbedding, "RotaryPositionEmbedding")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<RotaryPositionEmbeddingCollector>(t, theta); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            ASSERT(in.size() == 2 && in[0].get().shape.size() == 3, "RotaryPositionEmbedding takes x[tokens,heads,D] and positions");
            return one(in[0].get().dataType, in[0].get().shape);
        }
    };
    struct TopK final : Operator {
        dim_t k;
        bool softmax;
        TopK(dim_t k_, bool s) : k(k_), softmax(s) {}
        RG_OP(TopK, "TopK")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<TopKCollector>(t, k, softmax); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            Shape o = in[0].get().shape;
            ASSERT(!o.empty() && k <= o.back(), "TopK: k larger than the row");
            o.back() = k;
            return {Tensor::share(softmax ? DataType(DataType::F32) : in[0].get().dataType, o), Tensor::share(DataType::I64, o)};
        }
    };
    struct TopKSample final : Operator {
        dim_t k;
        float temperature;
        uint64_t seed;
        TopKSample(dim_t k_, float t, uint64_t s) : k(k_), temperature(t), seed(s) {}
        RG_OP(TopKSample, "TopKSample")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<TopKSampleCollector>(t, k, temperature, seed); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            Shape o(in[0].get().shape.begin(), in[0].get().shape.end() - 1);
            return one(DataType::I64, o);
        }
    };
    struct FusedLinear final : Operator {
        int prologue, epilogue;
        float epsilon, theta;
        dim_t nHeads, nKVHeads, headDim, maxSeq, pageSize, tokensPerSeq;
        explicit FusedLinear(Attributes const &a)
            : prologue(static_cast<int>(getInt(a, "prologue", 0))), epilogue(static_cast<int>(getInt(a, "epilogue", 0))),
              epsilon(static_cast<float>(getFloat(a, "epsilon", 1e-5))), theta(static_cast<float>(getFloat(a, "theta", 10000.0))),
              nHeads(static_cast<dim_t>(getInt(a, "n_heads", 0))), nKVHeads(static_cast<dim_t>(getInt(a, "n_kv_heads", 0))),
              headDim(static_cast<dim_t>(getInt(a, "head_dim", 0))), maxSeq(static_cast<dim_t>(getInt(a, "max_seq", 0))),
              pageSize(static_cast<dim_t>(getInt(a, "page_size", 0))), tokensPerSeq(static_cast<dim_t>(getInt(a, "tokens_per_seq", 0))) {}
        RG_OP(FusedLinear, "FusedLinear")
        CollectorBox candidateKernels(Target t) const final {
            return std::make_unique<FusedLinearCollector>(t, prologue, epilogue, epsilon, theta, nHeads, nKVHeads, headDim, maxSeq, pageSize, tokensPerSeq);
        }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            auto const &x = in[0].get();
            auto const &w = in[1].get();
            ASSERT(x.shape.size() == 2 && w.shape.size() == 2 && x.shape[1] == w.shape[1], "FusedLinear: X[m,k], W[n,k]");
            dim_t n = w.shape[0];
            if (epilogue == 2) n /= 2;
            if (epilogue == 3) n = nHeads * headDim;
            return one(x.dataType, Shape{x.shape[0], n});
        }
    };
    struct AttentionDecode final : Operator {
        dim_t maxLen, pageSize;
        AttentionDecode(dim_t m, dim_t p) : maxLen(m), pageSize(p) {}
        RG_OP(AttentionDecode, "AttentionDecode")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<AttentionDecodeCollector>(t, maxLen, pageSize); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final { return one(in[0].get().dataType, in[0].get().shape); }
    };
    struct QkvRopeAppend final : Operator {
        dim_t nHeads, nKVHeads, headDim, pageSize, tokensPerSeq;
        float theta;
        explicit QkvRopeAppend(Attributes const &a)
            : nHeads(static_cast<dim_t>(getInt(a, "n_heads", 0))), nKVHeads(static_cast<dim_t>(getInt(a, "n_kv_heads", 0))),
              headDim(static_cast<dim_t>(getInt(a, "head_dim", 0))), pageSize(static_cast<dim_t>(getInt(a, "page_size", 0))),
              tokensPerSeq(static_cast<dim_t>(getInt(a, "tokens_per_seq", 0))), theta(static_cast<float>(getFloat(a, "theta", 10000.0))) {}
        RG_OP(QkvRopeAppend, "QkvRopeAppend")
        CollectorBox candidateKernels(Target t) const final {
            return std::make_unique<QkvRopeAppendCollector>(t, nHeads, nKVHeads, headDim, pageSize, theta, tokensPerSeq);
        }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            ASSERT(in[0].get().shape.size() == 2, "QkvRopeAppend: qkv must be [tokens, (nH + 2 nKV) * D]");
            return one(in[0].get().dataType, Shape{in[0].get().shape[0], nHeads * headDim});
        }
    };
    struct AttentionPrefill final : Operator {
        dim_t nHeads, seqLen;
        AttentionPrefill(dim_t h, dim_t s) : nHeads(h), seqLen(s) {}
        RG_OP(AttentionPrefill, "AttentionPrefill")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<AttentionPrefillCollector>(t, nHeads, seqLen); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final { return one(in[0].get().dataType, in[0].get().shape); }
    };
    struct Swiglu final : Operator {
        RG_OP(Swiglu, "SwiGLU")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<SwigluCollector>(t); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            Shape o = in[0].get().shape;
            ASSERT(!o.empty() && o.back() % 2 == 0, "SwiGLU: last dimension must be even");
            o.back() /= 2;
            return one(in[0].get().dataType, o);
        }
    };
    struct DecodeStep final : Operator {
        dim_t nHeads, nKVHeads, headDim;
        float epsilon, theta;
        explicit DecodeStep(Attributes const &a)
            : nHeads(static_cast<dim_t>(getInt(a, "n_heads", 0))), nKVHeads(static_cast<dim_t>(getInt(a, "n_kv_heads", 0))),
              headDim(static_cast<dim_t>(getInt(a, "head_dim", 0))), epsilon(static_cast<float>(getFloat(a, "epsilon", 1e-5))),
              theta(static_cast<float>(getFloat(a, "theta", 10000.0))) {}
        RG_OP(DecodeStep, "DecodeStep")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<DecodeStepCollector>(t, nHeads, nKVHeads, headDim, epsilon, theta); }
        std::vector<Arc<Tensor>> infer(TensorRefs in) const final {
            ASSERT(in.size() >= 5 && (in.size() - 5) % 8 == 0, "DecodeStep: inputs are token, pos, embed, norm_f, lm_head + 8 per layer");
            auto const &embed = in[2].get();
            return {Tensor::share(DataType::I64, Shape{1}), Tensor::share(DataType::F32, Shape{1}),
                    Tensor::share(embed.dataType, Shape{1, embed.shape[0]})};
        }
    };
    struct StateUpdate final : Operator {
        int64_t delta;
        explicit StateUpdate(int64_t d) : delta(d) {}
        RG_OP(StateUpdate, "StateUpdate")
        CollectorBox candidateKernels(Target t) const final { return std::make_unique<StateUpdateCollector>(t, delta); }
        std::vector<Arc<Tensor>> infer(TensorRefs) const final { return {}; }
    };

}// namespace refactor::computation
