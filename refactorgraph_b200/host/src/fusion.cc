// Kernel fusion on the operator graph, and graph serialisation.
//
// The reference rewrites its computation graph before lowering it (src/05computation/src/graph.cc:17-77 with
// layoutPermute, src/05computation/src/transfomation/layout_permutation.cpp:36, selected by the `passes` argument of
// Compiler.compile, src/09python_ffi/src/compiler.cc:68-83).  This file adds the rewrites that matter on B200: a decoder
// written operator by operator (RmsNormalization, MatMul, QkvRopeAppend, Add, SwiGLU, AllReduce ...) becomes the fused
// operators the kernels implement, so that `compile("cuda", allocator, ["fuse"])` of the plain graph runs the same
// launches as a graph whose author emitted the fused operators by hand.
#include "operators.h"
#include <cstdlib>
#include <functional>

namespace refactor::computation {

    namespace {
        constexpr size_t NONE = static_cast<size_t>(-1);

        struct Rewriter {
            Graph &g;
            std::vector<char> dead;// nodes removed by a rewrite
            size_t rewrites = 0;

            explicit Rewriter(Graph &g_) : g(g_), dead(g_.nodes.size(), 0) {}

            Tensor const &tensor(size_t e) const { return *g.edges[e].tensor; }
            bool isGlobalOutput(size_t e) const { return std::find(g.globalOutputs.begin(), g.globalOutputs.end(), e) != g.globalOutputs.end(); }
            bool isGlobalInput(size_t e) const { return std::find(g.globalInputs.begin(), g.globalInputs.end(), e) != g.globalInputs.end(); }
            size_t producer(size_t e) const {
                for (size_t n = 0; n < g.nodes.size(); ++n)
                    if (!dead[n] && std::find(g.nodes[n].outputs.begin(), g.nodes[n].outputs.end(), e) != g.nodes[n].outputs.end()) return n;
                return NONE;
            }
            std::vector<size_t> consumers(size_t e) const {
                std::vector<size_t> ans;
                for (size_t n = 0; n < g.nodes.size(); ++n)
                    if (!dead[n] && std::find(g.nodes[n].inputs.begin(), g.nodes[n].inputs.end(), e) != g.nodes[n].inputs.end()) ans.push_back(n);
                return ans;
            }
            // the one node that reads e, when e is read by exactly one node and is not a graph output
            size_t soleConsumer(size_t e) const {
                if (isGlobalOutput(e)) return NONE;
                auto c = consumers(e);
                return c.size() == 1 ? c[0] : NONE;
            }
            template<class Op> Op *as(size_t n) const { return n == NONE ? nullptr : dynamic_cast<Op *>(g.nodes[n].op.get()); }
            static bool half(DataType t) { return t == DataType::FP16 || t == DataType::BF16; }
            // NAME=0 in the environment switches one rewrite off, NAME=1 an optional one on (A/B timing of a fused kernel against its parts)
            static bool envOff(char const *name) {
                char const *e = std::getenv(name);
                return e && e[0] == '0';
            }
            static bool envOn(char const *name) {
                char const *e = std::getenv(name);
                return e && e[0] == '1';
            }

            static OpBox linear(int prologue, int epilogue, float epsilon, Attributes extra = {}) {
                extra["prologue"] = static_cast<int64_t>(prologue);
                extra["epilogue"] = static_cast<int64_t>(epilogue);
                extra["epsilon"] = static_cast<double>(epsilon);
                return makeOperator("b200::Linear", extra);
            }

            // MatMul(x[m,k], W[n,k], transB) on up to 4 tokens (or up to 16 with few rows of W) -> Linear; on up to 4 tokens an
            // RmsNormalization that only feeds it becomes its prologue; a third input (C of the product's shape, beta 1) becomes its
            // residual epilogue.
            bool matMulToLinear(size_t n) {
                auto mm = as<MatMul>(n);
                auto &node = g.nodes[n];
                if (!mm || mm->transA || !mm->transB || mm->alpha != 1.f) return false;
                if (node.inputs.size() != 2 && node.inputs.size() != 3) return false;
                auto const &x = tensor(node.inputs[0]);
                auto const &w = tensor(node.inputs[1]);
                if (!half(x.dataType) || x.shape.size() != 2 || w.shape.size() != 2 || x.shape[0] > 16) return false;
                const bool few = x.shape[0] <= 4;
                // 5..16 tokens: the streaming skinny kernel (no norm prologue), for the shape it is faster on than the tensor-core
                // GEMM: few rows of W and a long k (one rank's QKV projection of a tensor-parallel step)
                if (!few && !(x.shape[0] <= 16 && x.shape[1] % 128 == 0 && x.shape[1] >= 4096 && w.shape[0] <= 2560)) return false;
                int epilogue = 0;
                if (node.inputs.size() == 3) {
                    if (mm->beta != 1.f || tensor(node.inputs[2]).shape != tensor(node.outputs[0]).shape) return false;
                    epilogue = 1;
                }
                std::vector<size_t> in{node.inputs[0], node.inputs[1]};
                int prologue = 0;
                float eps = 1e-5f;
                const size_t pn = producer(node.inputs[0]);
                if (auto norm = as<RmsNormalization>(pn); few && norm && soleConsumer(node.inputs[0]) == n) {
                    prologue = 1, eps = norm->epsilon;
                    in = {g.nodes[pn].inputs[0], node.inputs[1], g.nodes[pn].inputs[1]};
                    dead[pn] = 1;
                }
                if (epilogue == 1) in.push_back(node.inputs[2]);
                node.op = linear(prologue, epilogue, eps);
                node.inputs = std::move(in);
                return true;
            }

            // Linear without an epilogue whose only reader is an Add with a tensor of the same shape, a SwiGLU, or a
            // QkvRopeAppend: the reader becomes the epilogue.
            bool linearEpilogue(size_t n) {
                auto lin = as<FusedLinear>(n);
                if (!lin || lin->epilogue != 0) return false;
                auto &node = g.nodes[n];
                const size_t y = node.outputs[0], c = soleConsumer(y);
                if (c == NONE) return false;
                auto &next = g.nodes[c];
                if (auto add = as<SimpleBinary>(c); add && add->type == SimpleBinaryType::Add && next.inputs.size() == 2) {
                    const size_t r = next.inputs[0] == y ? next.inputs[1] : next.inputs[0];
                    if (r == y || tensor(r).shape != tensor(y).shape) return false;
                    node.op = linear(lin->prologue, 1, lin->epsilon);
                    node.inputs.push_back(r);
                } else if (as<Swiglu>(c)) {
                    node.op = linear(lin->prologue, 2, lin->epsilon);
                } else if (auto qa = as<QkvRopeAppend>(c); qa && next.inputs[0] == y) {
                    auto const &kc = tensor(next.inputs[next.inputs.size() - 2]);
                    Attributes a;
                    a["n_heads"] = static_cast<int64_t>(qa->nHeads), a["n_kv_heads"] = static_cast<int64_t>(qa->nKVHeads);
                    a["head_dim"] = static_cast<int64_t>(qa->headDim), a["theta"] = static_cast<double>(qa->theta);
                    a["page_size"] = static_cast<int64_t>(qa->pageSize), a["tokens_per_seq"] = static_cast<int64_t>(qa->tokensPerSeq);
                    a["max_seq"] = static_cast<int64_t>(qa->pageSize ? 0 : kc.shape[2]);
                    node.op = linear(lin->prologue, 3, lin->epsilon, a);
                    node.inputs.insert(node.inputs.end(), next.inputs.begin() + 1, next.inputs.end());
                } else {
                    return false;
                }
                node.outputs = next.outputs;
                dead[c] = 1;
                return true;
            }

            // Products on more than 64 tokens run on the tensor cores; their SiLU-gate and QKV split / rotation / append
            // readers become the GEMM's epilogue (the forms the kernel library has: head_dim 128, gate rows a multiple of 128).
            // On 5..64 tokens the SiLU gate has such an epilogue too.
            bool gemmEpilogue(size_t n) {
                auto mm = as<MatMul>(n);
                auto &node = g.nodes[n];
                if (!mm || mm->transA || !mm->transB || mm->alpha != 1.f || node.inputs.size() != 2) return false;
                auto const &x = tensor(node.inputs[0]);
                auto const &w = tensor(node.inputs[1]);
                if (!half(x.dataType) || x.shape.size() != 2 || w.shape.size() != 2 || x.shape[0] <= 4) return false;
                const size_t y = node.outputs[0], c = soleConsumer(y);
                if (c == NONE) return false;
                auto &next = g.nodes[c];
                if (x.shape[0] <= 64) {
                    // 5..64 tokens (weights on the M side of the instruction): the SiLU gate (gate rows in 64s) and the QKV split +
                    // rotation + append (a 128-row tile = one head) have tensor-core epilogues
                    if (x.shape[1] % 8 != 0 || x.shape[1] < 64) return false;
                    auto qs = as<QkvRopeAppend>(c);
                    if (as<Swiglu>(c) && w.shape[0] % 128 == 0 && !envOff("RG_B200_FUSE_GATE_SMALL")) {
                        node.op = linear(0, 2, 1e-5f);
                    } else if (qs && next.inputs[0] == y && qs->headDim == 128 && w.shape[0] == (qs->nHeads + 2 * qs->nKVHeads) * 128 &&
                               envOn("RG_B200_FUSE_ROPE_SMALL")) {// off by default: measured slower than the product + rotation kernel
                        auto const &kc = tensor(next.inputs[next.inputs.size() - 2]);
                        Attributes a;
                        a["n_heads"] = static_cast<int64_t>(qs->nHeads), a["n_kv_heads"] = static_cast<int64_t>(qs->nKVHeads);
                        a["head_dim"] = static_cast<int64_t>(qs->headDim), a["theta"] = static_cast<double>(qs->theta);
                        a["page_size"] = static_cast<int64_t>(qs->pageSize), a["tokens_per_seq"] = static_cast<int64_t>(qs->tokensPerSeq);
                        a["max_seq"] = static_cast<int64_t>(qs->pageSize ? 0 : kc.shape[2]);
                        node.op = linear(0, 3, 1e-5f, a);
                        node.inputs.insert(node.inputs.end(), next.inputs.begin() + 1, next.inputs.end());
                    } else {
                        return false;
                    }
                } else if (as<Swiglu>(c) && w.shape[0] % 256 == 0) {
                    node.op = linear(0, 2, 1e-5f);
                } else if (auto qa = as<QkvRopeAppend>(c); qa && next.inputs[0] == y && qa->headDim == 128) {
                    auto const &kc = tensor(next.inputs[next.inputs.size() - 2]);
                    Attributes a;
                    a["n_heads"] = static_cast<int64_t>(qa->nHeads), a["n_kv_heads"] = static_cast<int64_t>(qa->nKVHeads);
                    a["head_dim"] = static_cast<int64_t>(qa->headDim), a["theta"] = static_cast<double>(qa->theta);
                    a["page_size"] = static_cast<int64_t>(qa->pageSize), a["tokens_per_seq"] = static_cast<int64_t>(qa->tokensPerSeq);
                    a["max_seq"] = static_cast<int64_t>(qa->pageSize ? 0 : kc.shape[2]);
                    node.op = linear(0, 3, 1e-5f, a);
                    node.inputs.insert(node.inputs.end(), next.inputs.begin() + 1, next.inputs.end());
                } else {
                    return false;
                }
                node.outputs = next.outputs;
                dead[c] = 1;
                return true;
            }

            // MatMul (two inputs) or AllReduceSum (one input) whose only reader adds a tensor of the same shape: the addend
            // becomes the product's C operand (beta 1) / the all-reduce's residual input.
            bool absorbAdd(size_t n) {
                auto &node = g.nodes[n];
                auto mm = as<MatMul>(n);
                auto ar = as<AllReduce>(n);
                if (!(mm && node.inputs.size() == 2) && !(ar && ar->type == AllReduceType::Sum && node.inputs.size() == 1)) return false;
                const size_t y = node.outputs[0], c = soleConsumer(y);
                auto add = as<SimpleBinary>(c);
                if (!add || add->type != SimpleBinaryType::Add) return false;
                auto &next = g.nodes[c];
                const size_t r = next.inputs[0] == y ? next.inputs[1] : next.inputs[0];
                if (r == y || tensor(r).shape != tensor(y).shape || tensor(r).dataType != tensor(y).dataType) return false;
                if (mm) node.op = std::make_unique<MatMul>(mm->alpha, 1.f, mm->transA, mm->transB);
                node.inputs.push_back(r);
                node.outputs = next.outputs;
                dead[c] = 1;
                return true;
            }

            // AllReduceSum (with or without an absorbed residual) one of whose readers is an RmsNormalization of rows that fit one
            // CTA's registers: one node with two outputs, the sum (still read by the next residual) and its normalisation.
            bool allReduceNorm(size_t n) {
                // Off unless RG_B200_FUSE_AR_NORM=1: on two GPUs the one-launch form measured 1.3 % slower per decode step than the
                // all-reduce (64 CTAs pushing) followed by the normalisation kernel (which starts early under programmatic
                // dependent launch): one CTA per row means 16 SMs issue all the NVLink stores.
                if (!envOn("RG_B200_FUSE_AR_NORM")) return false;
                auto ar = as<AllReduce>(n);
                auto &node = g.nodes[n];
                if (!ar || ar->type != AllReduceType::Sum || node.inputs.empty() || node.inputs.size() > 2) return false;
                const size_t y = node.outputs[0];
                auto const &ty = tensor(y);
                if (!half(ty.dataType) || ty.shape.empty() || ty.shape.back() % 8 != 0 || ty.shape.back() > 16384) return false;
                for (auto c : consumers(y)) {
                    auto norm = as<RmsNormalization>(c);
                    auto &next = g.nodes[c];
                    if (!norm || next.inputs.size() != 2 || next.inputs[0] != y || next.inputs[1] == y) continue;
                    if (tensor(next.inputs[1]).elementsSize() != ty.shape.back() || tensor(next.inputs[1]).dataType != ty.dataType) continue;
                    Attributes a;
                    a["epsilon"] = static_cast<double>(norm->epsilon);
                    node.op = makeOperator("b200::AllReduceNorm", a);
                    node.inputs.push_back(next.inputs[1]);
                    node.outputs = {y, next.outputs[0]};
                    dead[c] = 1;
                    return true;
                }
                return false;
            }

            // MatMul(x[m <= 64, k], W[n, k], transB, no C) whose only reader is an AllReduceSum (with or without an absorbed residual):
            // one node whose product writes into the peers' all-reduce slots from its epilogue.  Off unless RG_B200_FUSE_MM_AR=1:
            // bit-identical to the pair, but measured on two GPUs it costs 3-4.5 us more per product (16 tokens x 8192 outputs:
            // 32.6 vs 29.6 us for k = 4096, 24.4 vs 19.9 for k = 1024) — the product's last CTAs issue the NVLink stores and the
            // kernel cannot complete before they are acknowledged, while the stand-alone all-reduce hides its stores behind its
            // own polling and already starts under the product's tail.
            bool matMulAllReduce(size_t n) {
                if (!envOn("RG_B200_FUSE_MM_AR")) return false;
                auto mm = as<MatMul>(n);
                auto &node = g.nodes[n];
                if (!mm || mm->transA || !mm->transB || node.inputs.size() != 2) return false;
                auto const &x = tensor(node.inputs[0]);
                auto const &w = tensor(node.inputs[1]);
                if (!half(x.dataType) || x.shape.size() != 2 || w.shape.size() != 2) return false;
                if (x.shape[0] == 0 || x.shape[0] > 64 || w.shape[0] < 128 || w.shape[0] % 8 != 0 || x.shape[1] % 8 != 0 || x.shape[1] < 64) return false;
                const size_t y = node.outputs[0], c = soleConsumer(y);
                auto ar = as<AllReduce>(c);
                if (!ar || ar->type != AllReduceType::Sum) return false;
                auto &next = g.nodes[c];
                if (next.inputs.empty() || next.inputs[0] != y || next.inputs.size() > 2) return false;
                Attributes a;
                a["alpha"] = static_cast<double>(mm->alpha);
                node.op = makeOperator("b200::MatMulAllReduce", a);
                if (next.inputs.size() == 2) node.inputs.push_back(next.inputs[1]);
                node.outputs = next.outputs;
                dead[c] = 1;
                return true;
            }

            // follows identity operators (Reshape) from edge e to the node that really reads it
            size_t readerThroughIdentity(size_t e, size_t *edgeSeen = nullptr) {
                for (;;) {
                    const size_t c = soleConsumer(e);
                    if (c == NONE) return NONE;
                    if (!g.nodes[c].op->isIdentity()) {
                        if (edgeSeen) *edgeSeen = e;
                        return c;
                    }
                    e = g.nodes[c].outputs[0];
                }
            }

            // A completely fused batch-1 greedy decode step -> one DecodeStep node.
            bool wholeStep() {
                // entry: Gather(embed, token) with token a graph input of one element
                size_t gather = NONE;
                for (size_t n = 0; n < g.nodes.size() && gather == NONE; ++n)
                    if (!dead[n] && as<Gather>(n) && g.nodes[n].inputs.size() == 2 && isGlobalInput(g.nodes[n].inputs[0]) &&
                        isGlobalInput(g.nodes[n].inputs[1]) && tensor(g.nodes[n].inputs[1]).elementsSize() == 1)
                        gather = n;
                if (gather == NONE) return false;
                const size_t embed = g.nodes[gather].inputs[0], token = g.nodes[gather].inputs[1];
                if (!half(tensor(embed).dataType) || tensor(embed).shape.size() != 2) return false;
                std::vector<size_t> absorbed{gather};
                std::vector<size_t> layerInputs;// 8 per layer
                size_t x = g.nodes[gather].outputs[0], pos = NONE, lens = NONE;
                FusedLinear *first = nullptr;
                size_t head = NONE;
                for (;;) {
                    // x is read by the layer's QKV linear and by its O-projection residual (or by the LM head only)
                    auto readers = consumers(x);
                    if (isGlobalOutput(x)) return false;
                    size_t qkv = NONE, lm = NONE;
                    for (auto r : readers) {
                        auto l = as<FusedLinear>(r);
                        if (l && l->prologue == 1 && l->epilogue == 3 && g.nodes[r].inputs[0] == x) qkv = r;
                        if (l && l->prologue == 1 && l->epilogue == 0 && g.nodes[r].inputs[0] == x) lm = r;
                    }
                    if (qkv == NONE) {
                        if (lm == NONE || readers.size() != 1) return false;
                        head = lm;
                        break;
                    }
                    if (readers.size() != 2) return false;
                    auto lq = as<FusedLinear>(qkv);
                    auto &nq = g.nodes[qkv];
                    if (nq.inputs.size() != 6 || lq->pageSize != 0) return false;// x, wqkv, norm1, pos, kc, vc (contiguous cache)
                    if (!first) first = lq;
                    if (lq->nHeads != first->nHeads || lq->nKVHeads != first->nKVHeads || lq->headDim != first->headDim) return false;
                    if (pos == NONE) pos = nq.inputs[3];
                    if (nq.inputs[3] != pos || !isGlobalInput(pos)) return false;
                    const size_t kc = nq.inputs[4], vc = nq.inputs[5];
                    const size_t att = readerThroughIdentity(nq.outputs[0]);
                    auto ad = as<AttentionDecode>(att);
                    if (!ad || g.nodes[att].inputs.size() != 4 || g.nodes[att].inputs[1] != kc || g.nodes[att].inputs[2] != vc) return false;
                    if (lens == NONE) lens = g.nodes[att].inputs[3];
                    if (g.nodes[att].inputs[3] != lens) return false;
                    const size_t o = readerThroughIdentity(g.nodes[att].outputs[0]);
                    auto lo = as<FusedLinear>(o);
                    if (!lo || lo->prologue != 0 || lo->epilogue != 1 || g.nodes[o].inputs.size() != 3 || g.nodes[o].inputs[2] != x) return false;
                    const size_t h = g.nodes[o].outputs[0];
                    auto hr = consumers(h);
                    if (hr.size() != 2 || isGlobalOutput(h)) return false;
                    size_t gu = NONE, dn = NONE;
                    for (auto r : hr) {
                        auto l = as<FusedLinear>(r);
                        if (l && l->prologue == 1 && l->epilogue == 2 && g.nodes[r].inputs[0] == h) gu = r;
                        if (l && l->prologue == 0 && l->epilogue == 1 && g.nodes[r].inputs.size() == 3 && g.nodes[r].inputs[2] == h) dn = r;
                    }
                    if (gu == NONE || dn == NONE || soleConsumer(g.nodes[gu].outputs[0]) != dn || g.nodes[dn].inputs[0] != g.nodes[gu].outputs[0]) return false;
                    if (lq->epsilon != as<FusedLinear>(gu)->epsilon) return false;
                    for (size_t e : {nq.inputs[2], nq.inputs[1], g.nodes[o].inputs[1], g.nodes[gu].inputs[2], g.nodes[gu].inputs[1], g.nodes[dn].inputs[1], kc, vc}) {
                        if (!isGlobalInput(e)) return false;
                        layerInputs.push_back(e);
                    }
                    // identity nodes between the pieces die with them
                    for (size_t n = 0; n < g.nodes.size(); ++n)
                        if (!dead[n] && g.nodes[n].op->isIdentity()) {
                            const size_t p = producer(g.nodes[n].inputs[0]);
                            if (p == qkv || p == att) absorbed.push_back(n);
                        }
                    absorbed.insert(absorbed.end(), {qkv, att, o, gu, dn});
                    x = g.nodes[dn].outputs[0];
                }
                if (!first || layerInputs.empty()) return false;
                auto lh = as<FusedLinear>(head);
                auto &nh = g.nodes[head];
                if (nh.inputs.size() != 3 || lh->epsilon != first->epsilon) return false;// x, lm_head, norm_f
                const size_t logits = nh.outputs[0];
                // logits -> TopK(k = 1, softmax) -> (Reshape ->) StateUpdate(token <- index)
                size_t topk = NONE;
                for (auto r : consumers(logits))
                    if (auto t = as<TopK>(r); t && t->k == 1 && t->softmax) topk = r;
                if (topk == NONE || consumers(logits).size() != 1) return false;
                const size_t probs = g.nodes[topk].outputs[0], idx = g.nodes[topk].outputs[1];
                size_t tokUpdate = NONE, posUpdate = NONE;
                std::vector<size_t> idxIdentity;
                for (size_t n = 0; n < g.nodes.size(); ++n) {
                    auto su = dead[n] ? nullptr : as<StateUpdate>(n);
                    if (!su) continue;
                    auto &sn = g.nodes[n];
                    if (sn.inputs[0] == token && sn.inputs.size() == 2 && su->delta == 0) {
                        size_t src = sn.inputs[1];
                        for (size_t p = producer(src); p != NONE && g.nodes[p].op->isIdentity(); p = producer(src)) idxIdentity.push_back(p), src = g.nodes[p].inputs[0];
                        if (src == idx) tokUpdate = n;
                    }
                    if (sn.inputs[0] == pos && sn.inputs.size() == 1 && su->delta == 1) posUpdate = n;
                }
                if (tokUpdate == NONE || posUpdate == NONE) return false;
                // the kernel's limits (csrc/decode_mega.cu): one sequence, contiguous cache of the common head shape
                auto const &kc0 = tensor(layerInputs[6]);
                if (kc0.shape.size() != 4 || kc0.shape[0] != 1) return false;
                Attributes a;
                a["n_heads"] = static_cast<int64_t>(first->nHeads), a["n_kv_heads"] = static_cast<int64_t>(first->nKVHeads);
                a["head_dim"] = static_cast<int64_t>(first->headDim), a["epsilon"] = static_cast<double>(first->epsilon);
                a["theta"] = static_cast<double>(first->theta);
                Graph::Node step;
                step.op = makeOperator("b200::DecodeStep", a);
                step.name = g.nodes[gather].name + "_decode_step";
                step.inputs = {token, pos, embed, nh.inputs[2], nh.inputs[1]};
                step.inputs.insert(step.inputs.end(), layerInputs.begin(), layerInputs.end());
                step.outputs = {idx, probs, logits};// the edges keep their descriptors: [1,1] index and probability, [1,V] logits
                absorbed.insert(absorbed.end(), {head, topk, tokUpdate, posUpdate});
                absorbed.insert(absorbed.end(), idxIdentity.begin(), idxIdentity.end());
                // every other reader of an absorbed intermediate would be left dangling: refuse the rewrite in that case
                for (size_t n : absorbed)
                    for (size_t e : g.nodes[n].outputs) {
                        if (e == idx || e == probs || e == logits) continue;
                        for (size_t c : consumers(e))
                            if (std::find(absorbed.begin(), absorbed.end(), c) == absorbed.end()) return false;
                        if (isGlobalOutput(e)) return false;
                    }
                for (size_t n : absorbed) dead[n] = 1;
                // the step node takes the place of the Gather, ahead of every surviving node that depends on its outputs
                g.nodes[gather] = std::move(step);
                dead[gather] = 0;
                return true;
            }

            void compact() {
                std::vector<Graph::Node> kept;
                for (size_t n = 0; n < g.nodes.size(); ++n)
                    if (!dead[n]) kept.push_back(std::move(g.nodes[n]));
                g.nodes = std::move(kept);
                dead.assign(g.nodes.size(), 0);
            }
            // a rewrite may give a node an input that is produced later in the list (the residual of an absorbed Add): restore
            // a topological order, stable with respect to the current one
            void sortTopologically() {
                const size_t N = g.nodes.size();
                std::vector<size_t> producerOf(g.edges.size(), NONE);
                for (size_t n = 0; n < N; ++n)
                    for (auto e : g.nodes[n].outputs) producerOf[e] = n;
                std::vector<char> placed(N, 0);
                std::vector<Graph::Node> order;
                std::function<void(size_t)> place = [&](size_t n) {
                    if (placed[n]) return;
                    placed[n] = 1;
                    for (auto e : g.nodes[n].inputs)
                        if (producerOf[e] != NONE && producerOf[e] != n) place(producerOf[e]);
                    order.push_back(std::move(g.nodes[n]));
                };
                // in-place state updates must stay behind every reader of the state they overwrite: they come last, in order
                std::vector<size_t> late;
                for (size_t n = 0; n < N; ++n) {
                    if (dynamic_cast<StateUpdate *>(g.nodes[n].op.get())) late.push_back(n);
                    else
                        place(n);
                }
                for (auto n : late) place(n);
                g.nodes = std::move(order);
            }
        };
    }// namespace

    size_t Graph::fuse(bool wholeStep) {
        Rewriter rw(*this);
        bool changed = true;
        while (changed) {
            changed = false;
            for (size_t n = 0; n < nodes.size(); ++n) {
                if (rw.dead[n]) continue;
                if (rw.matMulToLinear(n) || rw.linearEpilogue(n) || rw.gemmEpilogue(n) || rw.absorbAdd(n)) changed = true, ++rw.rewrites;
            }
        }
        // after the residual adds have been absorbed: all-reduce + normalisation pairs
        for (size_t n = 0; n < nodes.size(); ++n)
            if (!rw.dead[n] && rw.allReduceNorm(n)) ++rw.rewrites;
        // then the row-parallel products in front of the all-reduces that are left
        for (size_t n = 0; n < nodes.size(); ++n)
            if (!rw.dead[n] && rw.matMulAllReduce(n)) ++rw.rewrites;
        if (wholeStep && rw.wholeStep()) ++rw.rewrites;
        rw.compact();
        rw.sortTopologically();
        return rw.rewrites;
    }

    std::pair<std::string, std::vector<uint8_t>> Graph::serialize() const {
        std::ostringstream os;
        std::vector<uint8_t> data;
        auto shapeText = [](Tensor const &t) {
            std::string s(t.dataType.name());
            s += '<';
            for (size_t i = 0; i < t.shape.size(); ++i) s += (i ? "x" : "") + std::to_string(t.shape[i]);
            return s + '>';
        };
        for (size_t n = 0; n < nodes.size(); ++n) {
            os << "node\t" << n << '\t' << nodes[n].name << '\t' << nodes[n].op->name() << "\tin";
            for (auto e : nodes[n].inputs) os << ' ' << edges[e].name;
            os << "\tout";
            for (auto e : nodes[n].outputs) os << ' ' << edges[e].name;
            os << '\n';
        }
        for (size_t e = 0; e < edges.size(); ++e) {
            os << "edge\t" << e << '\t' << edges[e].name << '\t' << (edges[e].tensor ? shapeText(*edges[e].tensor) : std::string("?"));
            if (edges[e].tensor && edges[e].tensor->data && !edges[e].tensor->data->bytes.empty()) {
                os << "\tdata@" << data.size() << '+' << edges[e].tensor->data->bytes.size();
                data.insert(data.end(), edges[e].tensor->data->bytes.begin(), edges[e].tensor->data->bytes.end());
                data.resize((data.size() + 63) / 64 * 64);
            }
            os << '\n';
        }
        os << "inputs";
        for (auto e : globalInputs) os << ' ' << edges[e].name;
        os << "\noutputs";
        for (auto e : globalOutputs) os << ' ' << edges[e].name;
        os << '\n';
        return {os.str(), std::move(data)};
    }

}// namespace refactor::computation
