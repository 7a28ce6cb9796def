"""Whole graphs through compiler.compile('cuda', ...) / executor.run() against the oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle_np as onp
from refactorgraph_b200.graph_builder import F32, FP16, I64, GraphBuilder
from refactorgraph_b200.llama import (LlamaConfig, decode_step_graph, decode_step_graph_single_kernel, prefill_graph_reference_ops,
                                      seeded_weights, weight_inputs)

from _decode_oracle import oracle_decode as _oracle_decode

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
TINY = dict(layers=2, hidden=256, heads=4, kv_heads=4, head_dim=64, ffn=688, vocab=1000, eps=1e-6, max_seq=32, dtype=F32)


def test_tiny_prefill_matches_the_reference_cpu_kernels():
    """Configuration 1: fp32 tiny decoder, 32-token prefill, logits + top-5, against the logits the reference's own
    CPU kernels produced (tests/golden/tiny_llama_c1.npz, intended-softmax variant).  The as-built variant (the
    reference SoftmaxCpu divides by an integer-truncated sum) is reported, not matched."""
    gold = np.load(os.path.join(GOLDEN, "tiny_llama_c1.npz"))
    cfg = LlamaConfig(**TINY)
    g, index = prefill_graph_reference_ops(cfg, seeded_weights(cfg, 0), seq=32, top_k=5)
    for allocator in ("flat", "reusable"):
        ex = g.compiler().compile("cuda", allocator, [])
        ex.set_input(0, gold["ids"])
        ex.run()
        logits = ex.get_output(index["logits"])
        np.testing.assert_allclose(logits, gold["logits_intended"], atol=2e-4, rtol=1e-4)
        top5 = ex.get_output(index["topk_idx"])
        np.testing.assert_array_equal(top5, onp.topk(logits, 5)[1])      # bit-exact on the logits the GPU produced
        assert (top5 == gold["top5_intended"]).mean() > 0.98            # fp32 near-ties may swap neighbours
        ex.run()                                                          # CUDA-graph replay gives the same bytes
        np.testing.assert_array_equal(ex.get_output(index["logits"]), logits)
    print("as-built softmax divergence (reported): max |dlogit| =",
          float(np.abs(gold["logits_asbuilt"] - logits).max()))


@pytest.mark.parametrize("batch", [1, 2])
def test_decode_step_graph(batch):
    cfg = LlamaConfig(layers=2, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, max_seq=256, batch=batch)
    w16 = seeded_weights(cfg, 0, np.float16)
    # a wider spread than N(0, 0.02) keeps the greedy argmax away from fp16 ties
    rng = np.random.default_rng(1)
    w16["lm_head"] = (0.2 * rng.standard_normal(w16["lm_head"].shape)).astype(np.float16)
    w = {k: v.astype(np.float32) for k, v in w16.items()}
    past = np.array([70, 131][:batch], np.int64)
    kc = [rng.standard_normal((batch, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    vc = [rng.standard_normal((batch, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    token = rng.integers(0, cfg.vocab, (batch,)).astype(np.int64)
    steps = 6
    want_tok, want_logits = _oracle_decode(cfg, w, kc, vc, token, past, steps)

    g, index = decode_step_graph(cfg)

    def fresh():
        ex = g.compiler().compile("cuda", "flat", [])
        for name, _ in weight_inputs(cfg):
            ex.set_input(index[name], w16[name])
        for l in range(cfg.layers):
            ex.set_input(index[f"l{l}.k_cache"], kc[l])
            ex.set_input(index[f"l{l}.v_cache"], vc[l])
        ex.set_input(index["token"], token)
        ex.set_input(index["pos"], past)
        ex.set_input(index["lens"], past + 1)
        return ex

    # (a) device-resident loop: the step advances its own state; replays 2.. are CUDA-graph launches
    ex = fresh()
    got_tok, got_logits = [], []
    for _ in range(steps):
        ex.run()
        got_tok.append(ex.get_output(index["next"])[:, 0].copy())
        got_logits.append(ex.get_output(index["logits"]).astype(np.float32))
    got_tok, got_logits = np.stack(got_tok), np.stack(got_logits)
    np.testing.assert_allclose(got_logits, want_logits, atol=2e-2, rtol=1e-2)
    np.testing.assert_array_equal(got_tok, want_tok)
    probs = ex.get_output(index["probs"])
    assert ((probs > 0) & (probs <= 1)).all()
    # (b) host-fed loop, eager mode: the same tokens
    ex2 = fresh()
    ex2.set_graph_mode(False)
    tok, pos = token.copy(), past.copy()
    for s in range(steps):
        ex2.set_input(index["token"], tok)
        ex2.set_input(index["pos"], pos)
        ex2.set_input(index["lens"], pos + 1)
        ex2.run()
        tok = ex2.get_output(index["next"])[:, 0].copy()
        pos = pos + 1
        np.testing.assert_array_equal(tok, got_tok[s])


def test_reference_attention_operator_with_inplace_cache():
    """llm::Attention with 4 inputs and max_seq_len > 0 (README case 4): the cache lives in the output edges and
    past_seq_len is read on the device, so the same lowered kernel serves successive steps."""
    rng = np.random.default_rng(5)
    N, nH, nKV, D, S0, maxseq = 1, 4, 2, 64, 5, 16
    g = GraphBuilder()
    q = g.input("q", F32, (N, nH, 1, D))
    k = g.input("k", F32, (N, nKV, 1, D))
    v = g.input("v", F32, (N, nKV, 1, D))
    past = g.input("past", I64, (1,))
    o, kc, vc = g.op("llm::Attention", [q, k, v, past], n_out=3, max_seq_len=maxseq)
    for e in (o, kc, vc):
        g.output(e)
    ex = g.compiler().compile("cuda", "flat", [])
    kc_ref = np.zeros((N, nKV, maxseq, D), np.float32)
    vc_ref = np.zeros_like(kc_ref)
    for step in range(S0):
        qn, kn, vn = (rng.standard_normal(s).astype(np.float32) for s in ((N, nH, 1, D), (N, nKV, 1, D), (N, nKV, 1, D)))
        for i, a in enumerate((qn, kn, vn, np.array([step], np.int64))):
            ex.set_input(i, a)
        ex.run()
        want, kc_ref, vc_ref = onp.attention(qn, kn, vn, past=step, k_cache=kc_ref, v_cache=vc_ref)
        np.testing.assert_allclose(ex.get_output(0), want, rtol=1e-4, atol=1e-5)
        np.testing.assert_array_equal(ex.get_output(1), kc_ref)


@pytest.mark.parametrize("shape", [dict(heads=4, kv_heads=2, head_dim=128, hidden=512, ffn=1024, vocab=2000, past=70),
                                   dict(heads=8, kv_heads=8, head_dim=128, hidden=1024, ffn=2752, vocab=32000, past=700),
                                   dict(heads=4, kv_heads=4, head_dim=64, hidden=256, ffn=688, vocab=1000, past=0),
                                   dict(heads=4, kv_heads=1, head_dim=128, hidden=512, ffn=1024, vocab=777, past=64),
                                   # three cached tiles per CTA: one pair and one single tile per attention pass
                                   dict(heads=4, kv_heads=2, head_dim=128, hidden=512, ffn=1024, vocab=2000, past=1500, max_seq=2048),
                                   dict(heads=4, kv_heads=2, head_dim=64, hidden=256, ffn=688, vocab=1000, past=1100, max_seq=2048)])
def test_single_kernel_decode_step(shape):
    """b200::DecodeStep (the whole step in one persistent kernel) against the numpy oracle and the multi-kernel graph."""
    from refactorgraph_b200 import capi
    shape = dict(shape)
    past0 = shape.pop("past")
    cfg = LlamaConfig(layers=3, max_seq=shape.pop("max_seq", 1024), batch=1, **shape)
    w16 = seeded_weights(cfg, 0, np.float16)
    rng = np.random.default_rng(1)
    w16["lm_head"] = (0.1 * rng.standard_normal(w16["lm_head"].shape)).astype(np.float16)   # spread enough to avoid fp16 arg-max ties
    w = {k: v.astype(np.float32) for k, v in w16.items()}
    past = np.array([past0], np.int64)
    kc = [rng.standard_normal((1, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    vc = [rng.standard_normal((1, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    token = rng.integers(0, cfg.vocab, (1,)).astype(np.int64)
    steps = 5
    want_tok, want_logits = _oracle_decode(cfg, w, kc, vc, token, past, steps)
    g, index = decode_step_graph_single_kernel(cfg)
    ex = g.compiler().compile("cuda", "flat", [])
    assert ex.node_count() == 1
    for name, _ in weight_inputs(cfg):
        ex.set_input(index[name], w16[name])
    for l in range(cfg.layers):
        ex.set_input(index[f"l{l}.k_cache"], kc[l])
        ex.set_input(index[f"l{l}.v_cache"], vc[l])
    ex.set_input(index["token"], token)
    ex.set_input(index["pos"], past)
    for s in range(steps):
        ex.run()
        assert capi.load().rg_b200_error_state() == 0, "a bounded wait expired inside the decode-step kernel"
        logits = ex.get_output(index["logits"]).astype(np.float32)
        np.testing.assert_allclose(logits, want_logits[s], atol=2e-2, rtol=1e-2)
        tok = ex.get_output(index["next"])
        np.testing.assert_array_equal(tok, onp.topk(logits, 1)[1][0])          # arg-max of its own logits, bit-exact
        np.testing.assert_array_equal(tok, want_tok[s])
        p = ex.get_output(index["probs"])
        np.testing.assert_allclose(p, onp.topk_softmax(logits, 1)[0][0], rtol=1e-4)
