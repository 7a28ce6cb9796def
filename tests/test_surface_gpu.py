"""The Python surface beyond compile / run on a GPU: the fusion pass gives the bytes of the hand-fused graphs, trace dumps
every tensor of every node, outputs can stay on the device as blobs and feed another executor, compile_on / dispatch lower
for a device object, and the paged-KV block allocator drives a paged decode step."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle_np as onp
from refactorgraph_b200 import capi
from refactorgraph_b200 import python_ffi as ffi
from refactorgraph_b200.graph_builder import F32, FP16, I64, GraphBuilder
from refactorgraph_b200.llama import (LlamaConfig, decode_step_graph, decode_step_graph_batched, decode_step_graph_single_kernel,
                                      seeded_weights, weight_inputs)

pytestmark = pytest.mark.gpu


def _fill(ex, index, cfg, w16, kc, vc, token, past):
    for name, _ in weight_inputs(cfg):
        ex.set_input(index[name], w16[name])
    for l in range(cfg.layers):
        ex.set_input(index[f"l{l}.k_cache"], kc[l])
        ex.set_input(index[f"l{l}.v_cache"], vc[l])
    ex.set_input(index["token"], token)
    ex.set_input(index["pos"], past)
    if "lens" in index:
        ex.set_input(index["lens"], past + 1)


def test_fusion_pass_gives_the_bytes_of_the_hand_fused_graphs():
    cfg = LlamaConfig(layers=3, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, max_seq=256, batch=1)
    rng = np.random.default_rng(1)
    w16 = seeded_weights(cfg, 0, np.float16)
    w16["lm_head"] = (0.2 * rng.standard_normal(w16["lm_head"].shape)).astype(np.float16)
    kc = [rng.standard_normal((1, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    vc = [rng.standard_normal((1, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    token, past = np.array([17], np.int64), np.array([70], np.int64)
    plain, pidx = decode_step_graph_batched(cfg)          # operator by operator
    hand, hidx = decode_step_graph(cfg)                   # b200::Linear emitted by hand
    single, sidx = decode_step_graph_single_kernel(cfg)   # b200::DecodeStep emitted by hand
    runs = {}
    for tag, (g, idx, passes) in {"unfused": (plain, pidx, []), "pass": (plain, pidx, ["fuse"]), "hand": (hand, hidx, []),
                                  "pass-step": (plain, pidx, ["fuse-step"]), "hand-step": (single, sidx, [])}.items():
        ex = g.compiler().compile("cuda", "flat", passes)
        _fill(ex, idx, cfg, w16, kc, vc, token, past)
        outs = []
        for _ in range(3):                                 # the state advances on the device
            ex.run()
            outs.append((ex.get_output(idx["logits"]).copy(), ex.get_output(idx["next"]).ravel().copy()))
        runs[tag] = (ex.node_count(), outs)
    assert runs["pass"][0] == runs["hand"][0] < runs["unfused"][0]
    assert runs["pass-step"][0] == 2 and runs["hand-step"][0] == 1     # the sequence-length state keeps its own update node
    for a, b in (("pass", "hand"), ("pass-step", "hand-step")):
        for (la, ta), (lb, tb) in zip(runs[a][1], runs[b][1]):
            np.testing.assert_array_equal(la, lb)                       # same kernels, same bytes
            np.testing.assert_array_equal(ta, tb)
    # the unfused graph rounds the normalised activations and the products once more: close, not identical
    np.testing.assert_allclose(runs["unfused"][1][0][0].astype(np.float32), runs["hand"][1][0][0].astype(np.float32), atol=2e-2, rtol=1e-2)
    assert capi.load().rg_b200_error_state() == 0


def test_trace_dumps_every_tensor_as_npy(tmp_path):
    rng = np.random.default_rng(2)
    g = GraphBuilder()
    x = g.input("x", F32, (4, 8))
    g.constant("w", (1 + 0.1 * rng.standard_normal(8)).astype(np.float32))
    g.constant("m", rng.standard_normal((8, 6)).astype(np.float32))
    n = g.op("llm::RmsNormalization", [x, "w"], epsilon=1e-6, name="norm")
    y = g.op("onnx::MatMul", [n, "m"], name="proj")
    g.output(y)
    c = g.compiler()
    ex = c.compile("cuda", "flat", [])
    xv = rng.standard_normal((4, 8)).astype(np.float32)
    ex.set_input(0, xv)
    ex.trace(str(tmp_path / "t"), "npy")
    meta0 = (tmp_path / "t" / "node000000.meta").read_text().splitlines()
    meta1 = (tmp_path / "t" / "node000001.meta").read_text().splitlines()
    assert meta0[0] == "node\t0\tnorm" and meta1[0] == "node\t1\tproj"
    files = {}
    for line in meta0[1:] + meta1[1:]:
        kind, k, edge, path = line.split("\t")
        files[(kind, edge)] = np.load(path)
    np.testing.assert_array_equal(files[("input", "x")], xv)
    np.testing.assert_array_equal(files[("input", "w")], c.get_tensor("w"))
    want_n = onp.rms_norm(xv, c.get_tensor("w"), 1e-6)
    np.testing.assert_allclose(files[("output", "norm:0")], want_n, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(files[("output", "proj:0")], want_n @ c.get_tensor("m"), rtol=1e-4, atol=1e-5)
    ex.trace(str(tmp_path / "txt"), "text")
    first = (tmp_path / "txt" / "data000000.text").read_text().splitlines()
    assert first[0] == "F32<4x8>" and len(first[1].split("\t")) >= 32


def test_outputs_stay_on_the_device_as_blobs_and_compile_on_a_device_object():
    rng = np.random.default_rng(3)
    dev = ffi.find_device("nvidia", torch.cuda.current_device())
    assert dev.kind == "nvidia"

    def stage(scale):
        g = GraphBuilder()
        x = g.input("x", F32, (16, 32))
        g.constant("s", np.full((1,), scale, np.float32))
        g.output(g.op("onnx::Mul", [x, "s"]))
        return g.compiler().compile_on(dev, "flat", [])
    a, b = stage(2.0), stage(3.0)
    xv = rng.standard_normal((16, 32)).astype(np.float32)
    a.set_input(0, xv)
    a.run()
    blob = a.get_output_blob(0)                     # never leaves the GPU
    assert blob.size == xv.nbytes and blob.address == a.output_address(0) and blob.device == torch.cuda.current_device()
    b.set_input_blob(0, blob)
    b.run()
    np.testing.assert_allclose(b.get_output(0), xv * 6.0, rtol=1e-6)
    # dispatch: lower again for a device, inputs carried over (src/09python_ffi/src/executor.cc:16-33)
    b.dispatch(dev, "reusable")
    b.run()
    np.testing.assert_allclose(b.get_output(0), xv * 6.0, rtol=1e-6)
    with pytest.raises(RuntimeError, match="no Nvidia card"):
        ffi.find_device("nvidia", 4096)


def test_block_allocator_drives_a_paged_decode_step():
    """Two sequences of different lengths in a paged cache whose blocks come from KvBlockAllocator; a third sequence is
    released and its blocks are reused.  The logits must equal those of the contiguous-cache graph on the same data."""
    cfg = LlamaConfig(layers=2, hidden=512, heads=8, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, max_seq=128, batch=2)
    page, max_blocks, n_blocks = 16, cfg.max_seq // 16, 24
    rng = np.random.default_rng(4)
    w16 = seeded_weights(cfg, 0, np.float16)
    past = np.array([37, 64], np.int64)
    kc = [rng.standard_normal((2, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    vc = [rng.standard_normal((2, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    token = rng.integers(0, cfg.vocab, (2,)).astype(np.int64)
    alloc = ffi.KvBlockAllocator(n_blocks, page, 2, max_blocks)
    alloc.add_sequence(7, 90)                                  # a finished request: its blocks go back and get reused
    alloc.release(7)
    rows = [alloc.add_sequence(100 + b, int(past[b])) for b in range(2)]
    assert rows == [0, 1]
    for b in range(2):
        alloc.append(100 + b)                                  # room for the token this step appends (64 -> a new block)
    table = alloc.table()
    np.testing.assert_array_equal(alloc.lengths(), past + 1)
    gp, pidx = decode_step_graph_batched(cfg, paged=True, page=page, max_blocks=max_blocks, n_blocks=n_blocks)
    gc, cidx = decode_step_graph_batched(cfg)
    exp, exc = gp.compiler().compile("cuda", "flat", []), gc.compiler().compile("cuda", "flat", [])
    _fill(exc, cidx, cfg, w16, kc, vc, token, past)
    for name, _ in weight_inputs(cfg):
        exp.set_input(pidx[name], w16[name])
    for l in range(cfg.layers):
        for nm, src in (("k_cache", kc[l]), ("v_cache", vc[l])):
            pages = np.zeros((n_blocks, cfg.kv_heads, page, cfg.head_dim), np.float16)
            for b in range(2):
                for j, blk in enumerate(alloc.blocks(100 + b)):
                    pages[blk] = src[b, :, j * page:(j + 1) * page]
            exp.set_input(pidx[f"l{l}.{nm}"], pages)
    exp.set_input(pidx["block_table"], table)
    exp.set_input(pidx["token"], token)
    exp.set_input(pidx["pos"], past)
    exp.set_input(pidx["lens"], alloc.lengths())
    exp.run(), exc.run()
    np.testing.assert_array_equal(exp.get_output(pidx["logits"]), exc.get_output(cidx["logits"]))
    assert capi.load().rg_b200_error_state() == 0
