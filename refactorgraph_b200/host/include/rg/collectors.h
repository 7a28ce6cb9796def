// Collectors of the decoder path, same names and constructor arguments as the reference
// (src/04kernel/include/kernel/collectors/*.h).  filter() returns the B200 kernel for Target::Nvidia and nothing
// for any other target: there is no CPU fallback in this library.
#pragma once
#include "kernel.h"

namespace refactor::kernel {

    // src/04kernel/include/kernel/collectors/simple_unary.h:8-30
    enum class SimpleUnaryType : uint8_t {
        Abs, Acos, Acosh, Asin, Asinh, Atan, Atanh, Cos, Cosh, Sin, Sinh, Tan, Tanh, Relu, Sqrt, Sigmoid, Erf, Neg, Not,
        HardSwish, Exp,
        Silu = 100,// x*sigmoid(x): the fused pair of the decoder's FFN (not in the reference)
    };
    // src/04kernel/include/kernel/collectors/simple_binary.h:8-19
    enum class SimpleBinaryType : uint8_t { Add, Sub, Mul, Div, Pow, And, Or, Xor, Mod, Fmod };
    // src/04kernel/include/kernel/attributes/communication.h:5-11
    enum class AllReduceType : uint8_t { Sum, Avg, Min, Max, Prod };

#define RG_COLLECTOR(NAME, TYPE, FIELD)                                                           \
    struct NAME final : public InfoCollector {                                                    \
        TYPE FIELD;                                                                               \
        NAME(Target target, TYPE FIELD##_) noexcept : InfoCollector(target), FIELD(std::move(FIELD##_)) {} \
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;         \
    }

    // src/04kernel/include/kernel/collectors/rms_normalization.h:8-16
    RG_COLLECTOR(RmsNormalizationCollector, float, epsilon);
    // src/04kernel/include/kernel/collectors/softmax.h:8-16
    RG_COLLECTOR(SoftmaxCollector, dim_t, axis);
    // src/04kernel/include/kernel/collectors/mat_mul.h:8-17
    struct MatMulCollector final : public InfoCollector {
        float alpha, beta;
        bool transA, transB;
        MatMulCollector(Target target, float alpha_, float beta_, bool transA_, bool transB_) noexcept
            : InfoCollector(target), alpha(alpha_), beta(beta_), transA(transA_), transB(transB_) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };
    // src/04kernel/include/kernel/collectors/attention.h:8-15
    RG_COLLECTOR(AttentionCollector, dim_t, maxSeqLen);
    // src/04kernel/include/kernel/collectors/all_reduce.h:9-18
    RG_COLLECTOR(AllReduceCollector, AllReduceType, type);
    // src/04kernel/include/kernel/collectors/gather.h:8-16
    RG_COLLECTOR(GatherCollector, dim_t, axis);
    // src/04kernel/include/kernel/collectors/simple_binary.h:23-31
    RG_COLLECTOR(SimpleBinaryCollector, SimpleBinaryType, type);
    // src/04kernel/include/kernel/collectors/simple_unary.h:34-42
    RG_COLLECTOR(SimpleUnaryCollector, SimpleUnaryType, type);
    // src/04kernel/include/kernel/collectors/transpose.h
    RG_COLLECTOR(TransposeCollector, std::vector<dim_t>, perm);
    // src/04kernel/include/kernel/collectors/concat.h, split.h: the axis; part lengths come from the tensors
    RG_COLLECTOR(ConcatCollector, dim_t, axis);
    RG_COLLECTOR(SplitCollector, dim_t, axis);
    // src/04kernel/include/kernel/collectors/slice.h with the Dimensions of src/04kernel/include/kernel/attributes/slice_info.h:8-13
    struct SliceDim {
        int64_t start, step, length;
    };
    using SliceDimensions = std::vector<SliceDim>;
    RG_COLLECTOR(SliceCollector, SliceDimensions, dims);
    // src/04kernel/include/kernel/collectors/cast.h and the expand collector (src/04kernel/src/collectors/expand.cc): no attributes
    struct CastCollector final : public InfoCollector {
        explicit CastCollector(Target target) noexcept : InfoCollector(target) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };
    struct ExpandCollector final : public InfoCollector {
        explicit ExpandCollector(Target target) noexcept : InfoCollector(target) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };
    // src/04kernel/include/kernel/collectors/where.h
    struct WhereCollector final : public InfoCollector {
        explicit WhereCollector(Target target) noexcept : InfoCollector(target) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };

    // ---- operators the decoder needs that the reference does not have ------------------------------------------
    // x[tokens, heads, D], positions int64[tokens]
    RG_COLLECTOR(RotaryPositionEmbeddingCollector, float, theta);
    // x[rows, n] -> values[rows, k], indices int64[rows, k]; softmax: values are probabilities over the whole row
    struct TopKCollector final : public InfoCollector {
        dim_t k;
        bool softmax;
        TopKCollector(Target target, dim_t k_, bool softmax_) noexcept : InfoCollector(target), k(k_), softmax(softmax_) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };
    // logits[rows, n], step uint64[1] -> token int64[rows]
    struct TopKSampleCollector final : public InfoCollector {
        dim_t k;
        float temperature;
        uint64_t seed;
        TopKSampleCollector(Target target, dim_t k_, float t, uint64_t seed_) noexcept
            : InfoCollector(target), k(k_), temperature(t), seed(seed_) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };
    // Fused decode linear layer (rg_b200_linear): prologue 0|1 (RMSNorm), epilogue 0 none | 1 residual | 2 SiLU gate |
    // 3 QKV split + RoPE + cache append.  The operator passes exactly
    //   {X, W, [G], [R], [positions, (block_table), k_cache, v_cache]} and outputs {Y};
    // the caches are state edges that the kernel appends to in place.
    struct FusedLinearCollector final : public InfoCollector {
        int prologue, epilogue;
        float epsilon, theta;
        dim_t nHeads, nKVHeads, headDim, maxSeq, pageSize, tokensPerSeq;
        FusedLinearCollector(Target target, int prologue_, int epilogue_, float epsilon_, float theta_, dim_t nHeads_,
                             dim_t nKVHeads_, dim_t headDim_, dim_t maxSeq_, dim_t pageSize_, dim_t tokensPerSeq_ = 0) noexcept
            : InfoCollector(target), prologue(prologue_), epilogue(epilogue_), epsilon(epsilon_), theta(theta_),
              nHeads(nHeads_), nKVHeads(nKVHeads_), headDim(headDim_), maxSeq(maxSeq_), pageSize(pageSize_),
              tokensPerSeq(tokensPerSeq_) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };
    // Split-K flash-decoding (rg_b200_attn_decode): {q[B,nH,D], k_cache, v_cache, seq_lens int64[B], [block_table]} -> {o}
    struct AttentionDecodeCollector final : public InfoCollector {
        dim_t maxLen, pageSize;
        AttentionDecodeCollector(Target target, dim_t maxLen_, dim_t pageSize_) noexcept
            : InfoCollector(target), maxLen(maxLen_), pageSize(pageSize_) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };
    // qkv[tokens, (nH + 2 nKV) * D] -> q[tokens, nH * D]; k (rotated) and v appended to the cache state edges.
    // inputs {qkv, positions, [block_table], k_cache, v_cache}, outputs {q}
    struct QkvRopeAppendCollector final : public InfoCollector {
        dim_t nHeads, nKVHeads, headDim, pageSize, tokensPerSeq;
        float theta;
        QkvRopeAppendCollector(Target target, dim_t nHeads_, dim_t nKVHeads_, dim_t headDim_, dim_t pageSize_, float theta_,
                               dim_t tokensPerSeq_ = 0) noexcept
            : InfoCollector(target), nHeads(nHeads_), nKVHeads(nKVHeads_), headDim(headDim_), pageSize(pageSize_),
              tokensPerSeq(tokensPerSeq_), theta(theta_) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };
    // Causal flash attention over token-major activations: {q[B*S, nH*D], k_cache, v_cache [B, nKV, max_seq, D], [past]}
    // -> {o[B*S, nH*D]}; sequence b owns tokens [b*S, (b+1)*S)
    struct AttentionPrefillCollector final : public InfoCollector {
        dim_t nHeads, seqLen;
        AttentionPrefillCollector(Target target, dim_t nHeads_, dim_t seqLen_) noexcept : InfoCollector(target), nHeads(nHeads_), seqLen(seqLen_) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };
    // x[rows, 2f] -> silu(x[:, :f]) * x[:, f:]
    // Row-parallel product + AllReduce(Sum) (+ residual): x[m, k], w[n, k] (, residual[m, n]) -> y[m, n]; the product's epilogue is
    // the sending half of the all-reduce
    RG_COLLECTOR(MatMulAllReduceCollector, float, alpha);
    // AllReduce(Sum) + residual + RmsNormalization: x[rows, dim], (residual[rows, dim],) w[dim] -> y = sum(x) (+ residual), n = rmsnorm(y) * w
    RG_COLLECTOR(AllReduceNormCollector, float, epsilon);
    struct SwigluCollector final : public InfoCollector {
        explicit SwigluCollector(Target target) noexcept : InfoCollector(target) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };
    // One whole batch-1 decode step in a single persistent kernel (rg_b200_decode_step).
    // inputs {token, pos, embed, norm_f, lm_head, per layer: norm1, wqkv, wo, norm2, wgu, wd, k_cache, v_cache}
    // outputs {next int64[1], prob fp32[1], logits[1, vocab]}; token and pos are state edges updated in place
    struct DecodeStepCollector final : public InfoCollector {
        dim_t nHeads, nKVHeads, headDim;
        float epsilon, theta;
        DecodeStepCollector(Target target, dim_t nHeads_, dim_t nKVHeads_, dim_t headDim_, float epsilon_, float theta_) noexcept
            : InfoCollector(target), nHeads(nHeads_), nKVHeads(nKVHeads_), headDim(headDim_), epsilon(epsilon_), theta(theta_) {}
        std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const final;
    };
    // In-place int64 state update: inputs {state, [src]}; state = (src ? src : state) + delta.  The routine writes
    // through inputs[0] (a state edge of the graph); it has no outputs.
    RG_COLLECTOR(StateUpdateCollector, int64_t, delta);
#undef RG_COLLECTOR

}// namespace refactor::kernel
