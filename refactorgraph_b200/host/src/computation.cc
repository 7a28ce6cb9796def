// Semantic operators of the decoder path: attribute parsing, shape inference and the collector each one lowers
// to.  The reference splits this between its frontend operators (src/07onnx, src/08-01llm, src/08communication:
// infer + lower) and src/05computation/src/operators/*.cc (candidateKernels); here one class does both.
#include "operators.h"

namespace refactor::computation {

    OpBox makeOperator(std::string const &type, Attributes const &a) {
        auto is = [&](std::initializer_list<char const *> names) {
            return std::any_of(names.begin(), names.end(), [&](char const *n) { return type == n; });
        };
        if (is({"llm::RmsNormalization", "onnx::RmsNormalization"})) return std::make_unique<RmsNormalization>(static_cast<float>(getFloat(a, "epsilon", 1e-5)));
        if (is({"onnx::MatMul"})) return std::make_unique<MatMul>(1.f, 1.f, false, false);
        if (is({"llm::MatMul"})) return std::make_unique<MatMul>(1.f, 1.f, getInt(a, "transA", 0) != 0, getInt(a, "transB", 0) != 0);
        if (is({"onnx::Gemm"}))
            return std::make_unique<MatMul>(static_cast<float>(getFloat(a, "alpha", 1)), static_cast<float>(getFloat(a, "beta", 1)),
                                            getInt(a, "transA", 0) != 0, getInt(a, "transB", 0) != 0);
        if (is({"onnx::Softmax"})) return std::make_unique<Softmax>(getInt(a, "axis", -1));
        if (is({"llm::Attention"})) return std::make_unique<Attention>(static_cast<dim_t>(getInt(a, "max_seq_len", 0)));
        if (is({"onnx::Gather"})) return std::make_unique<Gather>(getInt(a, "axis", 0));
        if (is({"onnx::Add"})) return std::make_unique<SimpleBinary>(SimpleBinaryType::Add);
        if (is({"onnx::Sub"})) return std::make_unique<SimpleBinary>(SimpleBinaryType::Sub);
        if (is({"onnx::Mul"})) return std::make_unique<SimpleBinary>(SimpleBinaryType::Mul);
        if (is({"onnx::Div"})) return std::make_unique<SimpleBinary>(SimpleBinaryType::Div);
        if (is({"onnx::Pow"})) return std::make_unique<SimpleBinary>(SimpleBinaryType::Pow);
        if (is({"onnx::And"})) return std::make_unique<SimpleBinary>(SimpleBinaryType::And);
        if (is({"onnx::Or"})) return std::make_unique<SimpleBinary>(SimpleBinaryType::Or);
        if (is({"onnx::Xor"})) return std::make_unique<SimpleBinary>(SimpleBinaryType::Xor);
        if (is({"onnx::Mod"})) return std::make_unique<SimpleBinary>(getInt(a, "fmod", 0) ? SimpleBinaryType::Fmod : SimpleBinaryType::Mod);
        {
            static const std::pair<char const *, SimpleUnaryType> UNARY[] = {
                {"onnx::Abs", SimpleUnaryType::Abs}, {"onnx::Acos", SimpleUnaryType::Acos}, {"onnx::Acosh", SimpleUnaryType::Acosh},
                {"onnx::Asin", SimpleUnaryType::Asin}, {"onnx::Asinh", SimpleUnaryType::Asinh}, {"onnx::Atan", SimpleUnaryType::Atan},
                {"onnx::Atanh", SimpleUnaryType::Atanh}, {"onnx::Cos", SimpleUnaryType::Cos}, {"onnx::Cosh", SimpleUnaryType::Cosh},
                {"onnx::Sin", SimpleUnaryType::Sin}, {"onnx::Sinh", SimpleUnaryType::Sinh}, {"onnx::Tan", SimpleUnaryType::Tan},
                {"onnx::Erf", SimpleUnaryType::Erf}, {"onnx::Not", SimpleUnaryType::Not}, {"onnx::HardSwish", SimpleUnaryType::HardSwish}};
            for (auto const &[name, t] : UNARY)
                if (is({name})) return std::make_unique<SimpleUnary>(t);
        }
        if (is({"onnx::Sigmoid"})) return std::make_unique<SimpleUnary>(SimpleUnaryType::Sigmoid);
        if (is({"onnx::Tanh"})) return std::make_unique<SimpleUnary>(SimpleUnaryType::Tanh);
        if (is({"onnx::Relu"})) return std::make_unique<SimpleUnary>(SimpleUnaryType::Relu);
        if (is({"onnx::Sqrt"})) return std::make_unique<SimpleUnary>(SimpleUnaryType::Sqrt);
        if (is({"onnx::Neg"})) return std::make_unique<SimpleUnary>(SimpleUnaryType::Neg);
        if (is({"onnx::Exp"})) return std::make_unique<SimpleUnary>(SimpleUnaryType::Exp);
        if (is({"b200::Silu"})) return std::make_unique<SimpleUnary>(SimpleUnaryType::Silu);
        if (is({"onnx::Transpose"})) {
            auto p = getInts(a, "perm");
            return std::make_unique<Transpose>(std::vector<dim_t>(p.begin(), p.end()));
        }
        if (is({"onnx::Reshape"})) return std::make_unique<Reshape>(getInts(a, "shape"));
        if (is({"onnx::Concat"})) return std::make_unique<Concat>(getInt(a, "axis", 0));
        if (is({"onnx::Split"})) return std::make_unique<Split>(getInt(a, "axis", 0), getInts(a, "split"), static_cast<dim_t>(getInt(a, "num_outputs", 0)));
        if (is({"onnx::Slice"})) return std::make_unique<Slice>(getInts(a, "starts"), getInts(a, "ends"), getInts(a, "axes"), getInts(a, "steps"));
        if (is({"onnx::Expand"})) return std::make_unique<Expand>(getInts(a, "shape"));
        if (is({"onnx::Cast"})) {
            auto to = DataType::parse(static_cast<uint8_t>(getInt(a, "to", 0)));
            if (!to) RUNTIME_ERROR("onnx::Cast: unknown target type");
            return std::make_unique<Cast>(*to);
        }
        if (is({"onnx::Where"})) return std::make_unique<Where>();
        if (is({"onnx::AllReduceSum"})) return std::make_unique<AllReduce>(AllReduceType::Sum);
        if (is({"onnx::AllReduceAvg"})) return std::make_unique<AllReduce>(AllReduceType::Avg);
        if (is({"onnx::AllReduceMin"})) return std::make_unique<AllReduce>(AllReduceType::Min);
        if (is({"onnx::AllReduceMax"})) return std::make_unique<AllReduce>(AllReduceType::Max);
        if (is({"onnx::AllReduceProd"})) return std::make_unique<AllReduce>(AllReduceType::Prod);
        if (is({"llm::RotaryPositionEmbedding"})) return std::make_unique<RotaryPositionEmbedding>(static_cast<float>(getFloat(a, "theta", 10000.0)));
        if (is({"llm::TopK"})) return std::make_unique<TopK>(static_cast<dim_t>(getInt(a, "k", 1)), getInt(a, "softmax", 0) != 0);
        if (is({"b200::TopKSample"}))
            return std::make_unique<TopKSample>(static_cast<dim_t>(getInt(a, "k", 50)), static_cast<float>(getFloat(a, "temperature", 1.0)),
                                                static_cast<uint64_t>(getInt(a, "seed", 0)));
        if (is({"b200::Linear"})) return std::make_unique<FusedLinear>(a);
        if (is({"b200::AttentionDecode"}))
            return std::make_unique<AttentionDecode>(static_cast<dim_t>(getInt(a, "max_len", 0)), static_cast<dim_t>(getInt(a, "page_size", 0)));
        if (is({"b200::QkvRopeAppend"})) return std::make_unique<QkvRopeAppend>(a);
        if (is({"b200::SwiGLU"})) return std::make_unique<Swiglu>();
        if (is({"b200::MatMulAllReduce"})) return std::make_unique<MatMulAllReduce>(static_cast<float>(getFloat(a, "alpha", 1.0)));
        if (is({"b200::AllReduceNorm"})) return std::make_unique<AllReduceNorm>(static_cast<float>(getFloat(a, "epsilon", 1e-5)));
        if (is({"b200::AttentionPrefill"}))
            return std::make_unique<AttentionPrefill>(static_cast<dim_t>(getInt(a, "n_heads", 0)), static_cast<dim_t>(getInt(a, "seq_len", 0)));
        if (is({"b200::DecodeStep"})) return std::make_unique<DecodeStep>(a);
        if (is({"b200::StateUpdate"})) return std::make_unique<StateUpdate>(getInt(a, "delta", 0));
        TODO("Unsupported operator " + type);
    }

    // Normalises negative axes once input ranks are known, then infers every node's outputs in topological order.
    void Graph::inferShapes() {
        for (auto &n : nodes) {
            TensorRefs in;
            for (auto e : n.inputs) {
                ASSERT(edges[e].tensor, "edge " + edges[e].name + " has no tensor info before node " + n.name);
                in.emplace_back(*edges[e].tensor);
            }
            if (auto sm = dynamic_cast<Softmax *>(n.op.get()); sm && sm->axis < 0) sm->axis += in[0].get().rank();
            if (auto g = dynamic_cast<Gather *>(n.op.get()); g && g->axis < 0) g->axis += in[0].get().rank();
            auto out = n.op->infer(in);
            ASSERT(out.size() >= n.outputs.size(), "node " + n.name + " has more outputs than its operator produces");
            for (size_t i = 0; i < n.outputs.size(); ++i) edges[n.outputs[i]].tensor = out[i];
        }
    }

    // src/05computation/src/graph.cc:17-77: first candidate wins; nodes without a kernel are collected and
    // reported together as "No kernel selected for ...".
    kernel::Graph Graph::lower(Target target) const {
        kernel::Graph g;
        g.globalInputs = globalInputs;
        g.globalOutputs = globalOutputs;
        std::vector<size_t> alias(edges.size());
        for (size_t i = 0; i < edges.size(); ++i) {
            alias[i] = i;
            g.edges.push_back({edges[i].tensor, edges[i].name});
        }
        // A graph input that only matrix products read is a weight: nothing in the graph writes it (caches, states and
        // other inputs updated in place are consumed by at least one other kind of node).
        std::vector<char> isWeight(edges.size(), 0);
        for (auto e : globalInputs) isWeight[e] = 1;
        for (auto const &n : nodes) {
            const bool product = dynamic_cast<MatMul const *>(n.op.get()) != nullptr;
            for (auto e : n.inputs)
                if (!product) isWeight[e] = 0;
            for (auto e : n.outputs) isWeight[e] = 0;
        }
        std::string missing;
        for (auto const &n : nodes) {
            if (n.op->isIdentity()) {
                alias[n.outputs[0]] = alias[n.inputs[0]];
                continue;
            }
            TensorRefs in, out;
            for (auto e : n.inputs) in.emplace_back(*edges[e].tensor);
            for (auto e : n.outputs) out.emplace_back(*edges[e].tensor);
            auto candidates = n.op->candidateKernels(target)->filter(std::move(in), std::move(out));
            if (candidates.empty()) {
                missing += std::string(n.op->name()) + "(" + n.name + ") ";
                continue;
            }
            kernel::Graph::Node kn;
            kn.kernel = std::move(candidates.front());
            {
                std::vector<bool> isStatic;
                for (auto e : n.inputs) isStatic.push_back(isWeight[e] != 0);
                kn.kernel->hintStaticInputs(isStatic);
            }
            kn.name = n.name;
            for (auto e : n.inputs) kn.inputs.push_back(alias[e]);
            for (auto e : n.outputs) kn.outputs.push_back(alias[e]);
            g.nodes.push_back(std::move(kn));
        }
        if (!missing.empty()) RUNTIME_ERROR("No kernel selected for " + missing);
        for (auto &e : g.globalOutputs) {
            g.outputTensors.push_back(edges[e].tensor);
            e = alias[e];
        }
        return g;
    }
}// namespace refactor::computation
