"""Host layer without a GPU: graph assembly, shape inference and the reference's error behaviour."""
import os

import numpy as np
import pytest

from refactorgraph_b200 import python_ffi as ffi
from refactorgraph_b200.graph_builder import F32, FP16, I64, GraphBuilder
from refactorgraph_b200.llama import LlamaConfig, decode_step_graph, prefill_graph, prefill_graph_reference_ops, seeded_weights


def test_module_surface_matches_the_reference_names():
    for name in ("_make_operator", "_make_tensor", "_make_data", "_make_compiler", "Compiler", "Executor"):
        assert hasattr(ffi, name)
    for name in ("set_input", "get_output", "run", "bench", "trace", "dbg"):
        assert hasattr(ffi.Executor, name)
    for name in ("compile", "set_input", "set_input_info", "substitute"):
        assert hasattr(ffi.Compiler, name)


def test_unknown_operator_is_rejected_at_construction():
    with pytest.raises(Exception, match="Unsupported operator"):
        ffi._make_operator({}, "onnx::Conv", {})


def test_compile_on_cpu_has_no_kernel():
    # there is no CPU fallback: lowering for any other target fails the way computation::Graph::lower does
    g = GraphBuilder()
    x = g.input("x", F32, (4, 8))
    g.constant("w", np.ones(8, np.float32))
    g.output(g.op("llm::RmsNormalization", [x, "w"], epsilon=1e-6))
    with pytest.raises(RuntimeError, match="No kernel selected"):
        g.compiler().compile("cpu", "flat", [])
    with pytest.raises(RuntimeError, match="Unknown target"):
        g.compiler().compile("tpu", "flat", [])


def test_shape_errors_surface_as_runtime_errors():
    g = GraphBuilder()
    a = g.input("a", F32, (4, 8))
    b = g.input("b", F32, (9, 3))
    g.output(g.op("onnx::MatMul", [a, b]))
    with pytest.raises(RuntimeError, match="not matched"):
        g.compiler().compile("cpu", "flat", [])
    g = GraphBuilder()
    q = g.input("q", F32, (1, 6, 4, 16))
    k = g.input("k", F32, (1, 4, 4, 16))
    v = g.input("v", F32, (1, 4, 4, 16))
    g.output(g.op("llm::Attention", [q, k, v]))
    with pytest.raises(RuntimeError, match="multiple of n_kv_head"):
        g.compiler().compile("cpu", "flat", [])


def test_cycle_and_dangling_edges():
    g = GraphBuilder()
    x = g.input("x", F32, (2, 2))
    g.topology["n1"] = (["x", "n2:0"], ["n1:0"])
    g.topology["n2"] = (["n1:0"], ["n2:0"])
    g.nodes["n1"] = ffi._make_operator({}, "onnx::Add", {})
    g.nodes["n2"] = ffi._make_operator({}, "onnx::Sigmoid", {})
    g.outputs = ["n2:0"]
    with pytest.raises(RuntimeError, match="cycle"):
        g.compiler()


def test_decoder_graphs_assemble():
    cfg = LlamaConfig(layers=2, hidden=256, heads=2, kv_heads=2, head_dim=128, ffn=512, vocab=1000, max_seq=128, batch=2)
    g, index = decode_step_graph(cfg)
    assert index["token"] == 0 and index["pos"] == 1 and index["lens"] == 2
    assert len(g.inputs) == 3 + (2 + 6 * cfg.layers + 1) + 2 * cfg.layers
    g.compiler()  # topological sort and operator construction succeed
    tiny = LlamaConfig(layers=1, hidden=64, heads=2, kv_heads=2, head_dim=32, ffn=96, vocab=50, max_seq=8, dtype=F32)
    g2, idx2 = prefill_graph_reference_ops(tiny, seeded_weights(tiny, 0), seq=8)
    assert set(idx2) == {"logits", "topk_idx", "topk_val"}
    with pytest.raises(RuntimeError, match="No kernel selected"):
        g2.compiler().compile("cpu", "flat", [])  # shape inference over the whole graph ran before this error


def test_prefill_graph_with_fused_epilogues_assembles():
    """More than 64 tokens and head_dim 128: the QKV and gate/up products are b200::Linear nodes (GEMM epilogues do the
    RoPE + cache append and the SiLU gate); otherwise MatMul + QkvRopeAppend / SwiGLU.  Shape inference runs for both."""
    cfg = LlamaConfig(layers=2, hidden=256, heads=2, kv_heads=1, head_dim=128, ffn=512, vocab=1000, max_seq=128, batch=2)
    for fused, seq in ((True, 64), (False, 64), (True, 16)):
        g, index = prefill_graph(cfg, seq, fused_rope=fused)
        assert {"next", "probs", "logits", "ids", "positions", "last"} <= set(index)
        kinds = {name.split("_", 1)[1] for name in g.nodes}          # node names are "<number>_<operator>"
        assert ("Linear" in kinds) == (fused and cfg.batch * seq > 64)
        assert ("QkvRopeAppend" in kinds) != ("Linear" in kinds)
        with pytest.raises(RuntimeError, match="No kernel selected"):
            g.compiler().compile("cpu", "flat", [])


# ---- the rest of the reference's Python surface (src/09python_ffi/src/main.cpp:23-56) ------------------------------------
def test_module_surface_has_every_reference_entry_point():
    for name in ("config_log", "find_device", "_make_operator", "_make_tensor", "_make_data", "_make_data_ex", "_make_compiler",
                 "Tensor", "Operator", "Device", "Pinned", "Compiler", "Executor"):
        assert hasattr(ffi, name), name
    for name in ("substitute", "set_input", "set_input_info", "check_variables", "zero_inputs", "get_tensor", "compile", "compile_on", "serialize"):
        assert hasattr(ffi.Compiler, name), name
    for name in ("dispatch", "set_input", "set_input_blob", "get_output", "get_output_blob", "run", "bench", "trace", "dbg"):
        assert hasattr(ffi.Executor, name), name


def test_find_device_and_external_data(tmp_path):
    cpu = ffi.find_device("CPU", 0)
    assert cpu.kind == "cpu" and cpu.card == 0
    with pytest.raises(RuntimeError, match="Unknown device type"):
        ffi.find_device("tpu", 0)
    # _make_data_ex reads a constant from a file at an offset (ONNX external data, src/09python_ffi/src/import.cpp:40-55)
    w = np.arange(24, dtype=np.float32).reshape(4, 6)
    f = tmp_path / "weights.bin"
    f.write_bytes(b"\0" * 16 + w.tobytes())
    t = ffi._make_data_ex(F32, [4, 6], str(f), 16)
    assert t.shape == [4, 6] and t.dtype == F32
    with pytest.raises(RuntimeError, match="No such file"):
        ffi._make_data_ex(F32, [4, 6], str(tmp_path / "missing.bin"), 0)
    with pytest.raises(RuntimeError, match="shorter"):
        ffi._make_data_ex(F32, [4, 7], str(f), 16)
    g = GraphBuilder()
    x = g.input("x", F32, (2, 6))
    g.edges["w"] = t
    g.output(g.op("llm::MatMul", [x, "w"], transB=1))
    c = g.compiler()
    np.testing.assert_array_equal(c.get_tensor("w"), w)
    assert c.get_tensor("nope") is None
    zeros = c.zero_inputs()
    assert len(zeros) == 1 and zeros[0].shape == (2, 6) and zeros[0].dtype == np.float32 and not zeros[0].any()
    assert c.check_variables(False) == []
    # compile_on with a CPU device fails the way compile("cpu") does: this library has kernels for one target only
    with pytest.raises(RuntimeError, match="No kernel selected"):
        c.compile_on(cpu, "flat", [])


def test_serialize_writes_graph_info_and_data(tmp_path):
    g = GraphBuilder()
    x = g.input("x", F32, (4, 8))
    g.constant("w", np.arange(8, dtype=np.float32))
    g.output(g.op("llm::RmsNormalization", [x, "w"], epsilon=1e-6, name="norm"))
    g.compiler().serialize(str(tmp_path / "dump"))
    info = (tmp_path / "dump" / "graph.info").read_text()
    assert "node\t0\tnorm\tRmsNormalization\tin x w\tout norm:0" in info
    assert "F32<4x8>" in info and "F32<8>\tdata@0+32" in info
    data = (tmp_path / "dump" / "graph.data").read_bytes()
    np.testing.assert_array_equal(np.frombuffer(data[:32], np.float32), np.arange(8, dtype=np.float32))


def test_data_movement_operators_infer_onnx_shapes(tmp_path):
    """Concat / Split / Slice / Expand / Cast with the attributes ONNX gives them: negative axes, a negative-step slice with a
    negative end, broadcast to a higher rank.  Shapes are read back from the serialised graph."""
    from refactorgraph_b200.graph_builder import FP16 as F16
    g = GraphBuilder()
    a = g.input("a", F32, (2, 3, 8))
    b = g.input("b", F32, (2, 5, 8))
    c = g.op("onnx::Concat", [a, b], axis=1, name="cat")
    s0, s1 = g.op("onnx::Split", [c], n_out=2, axis=-1, split=[6, 2], name="sp")
    sl = g.op("onnx::Slice", [s0], starts=[7, 1], ends=[-9, 6], axes=[1, 2], steps=[-2, 2], name="sl")
    e = g.op("onnx::Expand", [s1], shape=[3, 2, 8, 2], name="ex")
    h = g.op("onnx::Cast", [sl], to=int(F16), name="ca")
    g.output(h)
    g.output(e)
    comp = g.compiler()
    assert sorted(comp.plan([])) == ["Cast", "Concat", "Expand", "Slice", "Split"]
    comp.serialize(str(tmp_path / "dump"))
    info = (tmp_path / "dump" / "graph.info").read_text()
    for line in ("cat:0\tF32<2x8x8>", "sp:0\tF32<2x8x6>", "sp:1\tF32<2x8x2>", "sl:0\tF32<2x4x3>", "ex:0\tF32<3x2x8x2>", "ca:0\tFP16<2x4x3>"):
        assert line in info, (line, info)
    # equal parts when no sizes are given; parts that do not add up are refused
    g2 = GraphBuilder()
    x = g2.input("x", F32, (4, 9))
    parts = g2.op("onnx::Split", [x], n_out=3, axis=1, num_outputs=3, name="eq")
    for p_ in parts:
        g2.output(p_)
    g2.compiler().serialize(str(tmp_path / "dump2"))
    assert (tmp_path / "dump2" / "graph.info").read_text().count("F32<4x3>") == 3
    g3 = GraphBuilder()
    x = g3.input("x", F32, (4, 9))
    with pytest.raises(RuntimeError):
        g3.op("onnx::Split", [x], n_out=2, axis=1, split=[4, 4])
        g3.compiler().plan([])


# ---- fusion pass: a decoder written operator by operator becomes the hand-fused graph ------------------------------------
def test_fusion_pass_reproduces_the_hand_fused_decode_graph():
    from refactorgraph_b200.llama import decode_step_graph_batched, decode_step_graph_single_kernel
    cfg = LlamaConfig(layers=3, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, max_seq=256, batch=1)
    plain, _ = decode_step_graph_batched(cfg)            # RmsNormalization, MatMul, QkvRopeAppend, AttentionDecode, SwiGLU ... per layer
    fused, _ = decode_step_graph(cfg)                    # the same step with b200::Linear written by hand
    c = plain.compiler()
    unfused_plan = c.plan([])
    assert unfused_plan.count("MatMul") == 4 * cfg.layers + 1 and "FusedLinear" not in unfused_plan
    assert c.plan(["ce", "lp"]) == unfused_plan          # the reference's pass names are accepted and change nothing here
    assert c.plan(["fuse"]) == fused.compiler().plan([])
    assert c.plan(["fuse"]).count("FusedLinear") == 4 * cfg.layers + 1
    # ... and the whole step becomes the single persistent kernel (the sequence-length state keeps its own update)
    assert c.plan(["fuse-step"]) == ["DecodeStep", "StateUpdate"]
    assert fused.compiler().plan(["fuse-step"]) == ["DecodeStep", "StateUpdate"]
    single, _ = decode_step_graph_single_kernel(cfg)
    assert single.compiler().plan([]) == ["DecodeStep"]
    # two sequences: fused linear layers, but no single-kernel step
    cfg2 = LlamaConfig(layers=2, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, max_seq=256, batch=2)
    p2 = decode_step_graph_batched(cfg2)[0].compiler().plan(["fuse-step"])
    assert "DecodeStep" not in p2 and p2.count("FusedLinear") == 4 * cfg2.layers + 1


def test_fusion_pass_on_batched_tensor_parallel_and_prefill_graphs():
    from refactorgraph_b200.llama import decode_step_graph_batched
    cfg = LlamaConfig(layers=1, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, max_seq=256, batch=16)
    # residual adds written as separate Add nodes are absorbed by the product (C operand) and by the all-reduce
    g = GraphBuilder()
    x = g.input("x", FP16, (16, 512))
    r = g.input("r", FP16, (16, 512))
    g.input("w", FP16, (512, 512))
    y = g.op("llm::MatMul", [x, "w"], transB=1)
    s = g.op("onnx::AllReduceSum", [y])
    h = g.op("onnx::Add", [s, r])
    y2 = g.op("llm::MatMul", [h, "w"], transB=1)
    g.output(g.op("onnx::Add", [r, y2]))
    c = g.compiler()
    assert c.plan([]) == ["MatMul", "AllReduce", "SimpleBinary", "MatMul", "SimpleBinary"]
    # the addends become the C operand / the residual input
    assert c.plan(["fuse"]) == ["MatMul", "AllReduce", "MatMul"]
    # opt-in: the product in front of the all-reduce becomes its sending half
    os.environ["RG_B200_FUSE_MM_AR"] = "1"
    try:
        assert c.plan(["fuse"]) == ["MatMulAllReduce", "MatMul"]
    finally:
        del os.environ["RG_B200_FUSE_MM_AR"]
    # 16 tokens against few weight rows with a long k (one rank's QKV projection): the streaming skinny kernel takes the
    # product together with the RoPE / cache-append reader
    cq = LlamaConfig(layers=1, hidden=8192, heads=8, kv_heads=1, head_dim=128, ffn=3584, vocab=2000, max_seq=256, batch=16)
    pq = decode_step_graph_batched(cq, world=8)[0].compiler().plan(["fuse"])
    assert pq[:3] == ["Gather", "RmsNormalization", "FusedLinear"] and pq.count("QkvRopeAppend") == 0
    # O and down stay plain tensor-core products; gate/up takes its SiLU gate as the epilogue; the 2000-row LM head qualifies for
    # the skinny kernel too
    assert pq == ["Gather", "RmsNormalization", "FusedLinear", "AttentionDecode", "MatMul", "AllReduce", "RmsNormalization", "FusedLinear",
                  "MatMul", "AllReduce", "RmsNormalization", "FusedLinear", "TopK", "StateUpdate", "StateUpdate", "StateUpdate"], pq
    # opt-in: O and down become products that write into the peers' all-reduce slots, with the receiving half behind them
    os.environ["RG_B200_FUSE_MM_AR"] = "1"
    try:
        pm = decode_step_graph_batched(cq, world=8)[0].compiler().plan(["fuse"])
    finally:
        del os.environ["RG_B200_FUSE_MM_AR"]
    assert pm == ["Gather", "RmsNormalization", "FusedLinear", "AttentionDecode", "MatMulAllReduce", "RmsNormalization", "FusedLinear",
                  "MatMulAllReduce", "RmsNormalization", "FusedLinear", "TopK", "StateUpdate", "StateUpdate", "StateUpdate"], pm
    # opt-in: every all-reduce of the layer is followed by a normalisation (the layer's second, or the final one): one launch each
    os.environ["RG_B200_FUSE_AR_NORM"] = "1"
    try:
        pn = decode_step_graph_batched(cq, world=8)[0].compiler().plan(["fuse"])
    finally:
        del os.environ["RG_B200_FUSE_AR_NORM"]
    assert pn == ["Gather", "RmsNormalization", "FusedLinear", "AttentionDecode", "MatMul", "AllReduceNorm", "FusedLinear", "MatMul",
                  "AllReduceNorm", "FusedLinear", "TopK", "StateUpdate", "StateUpdate", "StateUpdate"], pn
    # prefill (more than 64 tokens): SwiGLU and QkvRopeAppend become epilogues of the tensor-core product
    pcfg = LlamaConfig(layers=1, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, max_seq=128, batch=2)
    hand = prefill_graph(pcfg, 80, fused_rope=True)[0].compiler().plan([])
    auto = prefill_graph(pcfg, 80, fused_rope=False)[0].compiler()
    assert auto.plan([]).count("QkvRopeAppend") == 1 and auto.plan([]).count("SwiGLU") == 1
    got = auto.plan(["fuse"])
    # identical up to the LM head, where the pass goes one step further than the hand-written graph: two rows are few enough
    # for the streaming linear kernel, so the final norm is folded into it
    assert hand[-4:] == ["Gather", "RmsNormalization", "MatMul", "TopK"] and got[-3:] == ["Gather", "FusedLinear", "TopK"]
    assert got[:-3] == hand[:-4] and got.count("QkvRopeAppend") == 0 and got.count("SwiGLU") == 0


# ---- paged-KV block allocator -----------------------------------------------------------------------------------------------
def test_kv_block_allocator_grows_on_append_and_recycles_on_release():
    a = ffi.KvBlockAllocator(n_blocks=10, page_size=16, max_seqs=3, max_blocks_per_seq=4)
    assert a.free_blocks == 10
    r0 = a.add_sequence(100, 17)                 # two blocks
    r1 = a.add_sequence(200, 16)                 # exactly one block
    assert (r0, r1) == (0, 1) and a.free_blocks == 7
    assert a.blocks(100) == [0, 1] and a.blocks(200) == [2]
    t = a.table()
    assert t.shape == (3, 4) and t.dtype == np.int32
    np.testing.assert_array_equal(t, [[0, 1, -1, -1], [2, -1, -1, -1], [-1, -1, -1, -1]])
    np.testing.assert_array_equal(a.lengths(), [17, 16, 0])
    assert a.append(200) == 1                    # token 17 of sequence 200 opens a new block
    assert a.append(100, 15) == 0                # 32 tokens still fit two blocks
    assert a.append(100) == 1
    assert a.blocks(100) == [0, 1, 4] and a.blocks(200) == [2, 3] and a.length(100) == 33
    a.release(100)                               # blocks return to the free list, the row is reusable
    assert a.free_blocks == 8
    assert a.add_sequence(300, 1) == 0 and a.blocks(300) == [0]
    # failures leave the state untouched
    with pytest.raises(RuntimeError, match="outgrow"):
        a.append(200, 16 * 4)
    small = ffi.KvBlockAllocator(n_blocks=3, page_size=16, max_seqs=2, max_blocks_per_seq=4)
    small.add_sequence(1, 32)
    with pytest.raises(RuntimeError, match="out of blocks"):
        small.add_sequence(2, 33)
    small.add_sequence(2, 16)
    with pytest.raises(RuntimeError, match="out of blocks"):
        small.append(1)
    with pytest.raises(RuntimeError, match="no free table row"):
        small.add_sequence(3, 0)
    assert small.free_blocks == 0 and small.length(1) == 32
    with pytest.raises(RuntimeError, match="unknown sequence"):
        a.release(12345)
    with pytest.raises(RuntimeError, match="already exists"):
        a.add_sequence(200, 1)
    assert a.blocks(200) == [2, 3]
    # every block is owned by at most one sequence, and free + owned = all
    owned = [b for row in a.table().tolist() for b in row if b >= 0]
    assert len(owned) == len(set(owned)) and len(owned) + a.free_blocks == 10
