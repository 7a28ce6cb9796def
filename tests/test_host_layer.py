"""Host layer without a GPU: graph assembly, shape inference and the reference's error behaviour."""
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
