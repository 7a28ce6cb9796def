"""Llama-style decoder graphs for compiler.compile('cuda', ...) / executor.run().

Two builders:
  * `decode_step_graph`  — one generation step with the fused B200 operators (5 launches per layer): the graph the
    benchmark runs.  Token, position and length live in device state edges that the step itself advances, so a
    captured step replays with no host involvement; the host may also overwrite them before each run.
  * `prefill_graph_reference_ops` — a causal prefill written with the reference's own operator set only (Gather,
    RmsNormalization, MatMul, Transpose, Div, Where, Softmax, Add, Sigmoid, Mul — the operators the reference has
    CPU kernels for), used to compare a whole graph with the reference's CPU path.
"""
from __future__ import annotations

import numpy as np

from .config import LlamaConfig
from .graph_builder import BF16, BOOL, F32, FP16, I32, I64, GraphBuilder


LLAMA_7B = LlamaConfig()


def weight_inputs(cfg: LlamaConfig):
    """(name, shape) of every weight edge, in the order the graph declares them."""
    H, D = cfg.hidden, cfg.head_dim
    out = [("embed", (cfg.vocab, H))]
    for l in range(cfg.layers):
        out += [(f"l{l}.norm1", (H,)), (f"l{l}.wqkv", ((cfg.heads + 2 * cfg.kv_heads) * D, H)),
                (f"l{l}.wo", (H, cfg.heads * D)), (f"l{l}.norm2", (H,)), (f"l{l}.wgu", (2 * cfg.ffn, H)),
                (f"l{l}.wd", (H, cfg.ffn))]
    out += [("norm_f", (H,)), ("lm_head", (cfg.vocab, H))]
    return out


def decode_step_graph(cfg: LlamaConfig, top_k: int = 1, sample: bool = False, temperature: float = 1.0, seed: int = 0):
    """Builds the decode-step graph.  Returns (builder, index) where index maps edge names to global input /
    output numbers.  Inputs: token[B], pos[B], lens[B] (int64 state; lens = pos + 1), [step (uint64[1]) when
    sampling], weights, k/v caches [B, kv_heads, max_seq, D] per layer.  Outputs: next token ids and, for greedy
    decoding, their probabilities."""
    g = GraphBuilder()
    B, H, D = cfg.batch, cfg.hidden, cfg.head_dim
    token = g.input("token", I64, (B,))
    pos = g.input("pos", I64, (B,))
    lens = g.input("lens", I64, (B,))
    step = g.input("step", I64, (1,)) if sample else None
    for name, shape in weight_inputs(cfg):
        g.input(name, cfg.dtype, shape)
    for l in range(cfg.layers):
        g.input(f"l{l}.k_cache", cfg.dtype, (B, cfg.kv_heads, cfg.max_seq, D))
        g.input(f"l{l}.v_cache", cfg.dtype, (B, cfg.kv_heads, cfg.max_seq, D))
    kv_attrs = dict(n_heads=cfg.heads, n_kv_heads=cfg.kv_heads, head_dim=D, max_seq=cfg.max_seq, theta=cfg.theta)
    x = g.op("onnx::Gather", ["embed", token], axis=0)
    for l in range(cfg.layers):
        kc, vc = f"l{l}.k_cache", f"l{l}.v_cache"
        q = g.op("b200::Linear", [x, f"l{l}.wqkv", f"l{l}.norm1", pos, kc, vc], prologue=1, epilogue=3, epsilon=cfg.eps, **kv_attrs)
        q3 = g.op("onnx::Reshape", [q], shape=[B, cfg.heads, D])
        a = g.op("b200::AttentionDecode", [q3, kc, vc, lens], max_len=cfg.max_seq)
        a2 = g.op("onnx::Reshape", [a], shape=[B, cfg.heads * D])
        h = g.op("b200::Linear", [a2, f"l{l}.wo", x], epilogue=1)
        u = g.op("b200::Linear", [h, f"l{l}.wgu", f"l{l}.norm2"], prologue=1, epilogue=2, epsilon=cfg.eps)
        x = g.op("b200::Linear", [u, f"l{l}.wd", h], epilogue=1)
    logits = g.op("b200::Linear", [x, "lm_head", "norm_f"], prologue=1, epsilon=cfg.eps)
    index = {}
    if sample:
        nxt = g.op("b200::TopKSample", [logits, step], k=top_k, temperature=temperature, seed=seed)
        g.op("b200::StateUpdate", [step], n_out=0, delta=1)
        index["next"] = g.output(nxt)
    else:
        probs, idx = g.op("llm::TopK", [logits], n_out=2, k=top_k, softmax=1)
        nxt = g.op("onnx::Reshape", [idx], shape=[B]) if top_k == 1 else None
        index["next"] = g.output(idx)
        index["probs"] = g.output(probs)
    index["logits"] = g.output(logits)
    # carry the state to the next replay: token <- argmax / sample, pos += 1, lens += 1
    if nxt is not None:
        g.op("b200::StateUpdate", [token, nxt], n_out=0, delta=0)
    g.op("b200::StateUpdate", [pos], n_out=0, delta=1)
    g.op("b200::StateUpdate", [lens], n_out=0, delta=1)
    index.update({name: i for i, name in enumerate(g.inputs)})
    return g, index


def decode_step_graph_single_kernel(cfg: LlamaConfig):
    """The batch-1 greedy decode step as ONE node (b200::DecodeStep, a persistent cooperative kernel).  Inputs: token[1],
    pos[1] (int64 state: id of the token to feed and the number of cached tokens; both advanced by the kernel),
    weights, caches.  Outputs: next token, its probability, logits — the same values as `decode_step_graph`."""
    assert cfg.batch == 1
    g = GraphBuilder()
    token = g.input("token", I64, (1,))
    pos = g.input("pos", I64, (1,))
    for name, shape in weight_inputs(cfg):
        g.input(name, cfg.dtype, shape)
    for l in range(cfg.layers):
        g.input(f"l{l}.k_cache", cfg.dtype, (1, cfg.kv_heads, cfg.max_seq, cfg.head_dim))
        g.input(f"l{l}.v_cache", cfg.dtype, (1, cfg.kv_heads, cfg.max_seq, cfg.head_dim))
    ins = [token, pos, "embed", "norm_f", "lm_head"]
    for l in range(cfg.layers):
        ins += [f"l{l}.norm1", f"l{l}.wqkv", f"l{l}.wo", f"l{l}.norm2", f"l{l}.wgu", f"l{l}.wd", f"l{l}.k_cache", f"l{l}.v_cache"]
    nxt, prob, logits = g.op("b200::DecodeStep", ins, n_out=3, n_heads=cfg.heads, n_kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
                             epsilon=cfg.eps, theta=cfg.theta)
    index = {"next": g.output(nxt), "probs": g.output(prob), "logits": g.output(logits)}
    index.update({name: i for i, name in enumerate(g.inputs)})
    return g, index


def prefill_graph(cfg: LlamaConfig, seq: int, top_k: int = 1, fused_rope: bool = True):   # fused_rope: GEMM-epilogue fusions on
    """Causal prefill of `cfg.batch` sequences of `seq` tokens (token-major activations [B*S, hidden]): per layer
    RmsNormalization, Linear (tcgen05 QKV product whose epilogue splits the heads, rotates q and k and writes the K/V
    caches; with `fused_rope=False`, head_dim != 128 or fewer than 65 tokens: MatMul + QkvRopeAppend), AttentionPrefill, MatMul(+residual),
    RmsNormalization, MatMul, SwiGLU, MatMul(+residual); then the LM head on the last token of every sequence + TopK.
    Inputs: ids[B*S], positions[B*S], last[B] (row index of each sequence's last token), weights, caches."""
    g = GraphBuilder()
    B, H, D, n = cfg.batch, cfg.hidden, cfg.head_dim, cfg.batch * seq
    ids = g.input("ids", I64, (n,))
    pos = g.input("positions", I64, (n,))
    last = g.input("last", I64, (B,))
    for name, shape in weight_inputs(cfg):
        g.input(name, cfg.dtype, shape)
    for l in range(cfg.layers):
        g.input(f"l{l}.k_cache", cfg.dtype, (B, cfg.kv_heads, cfg.max_seq, D))
        g.input(f"l{l}.v_cache", cfg.dtype, (B, cfg.kv_heads, cfg.max_seq, D))
    x = g.op("onnx::Gather", ["embed", ids], axis=0)
    for l in range(cfg.layers):
        kc, vc = f"l{l}.k_cache", f"l{l}.v_cache"
        n1 = g.op("llm::RmsNormalization", [x, f"l{l}.norm1"], epsilon=cfg.eps)
        if fused_rope and D == 128 and n > 64:
            # QKV projection on the tcgen05 GEMM with the head split, rotation and cache append as its epilogue
            q = g.op("b200::Linear", [n1, f"l{l}.wqkv", pos, kc, vc], prologue=0, epilogue=3, n_heads=cfg.heads, n_kv_heads=cfg.kv_heads,
                     head_dim=D, theta=cfg.theta, max_seq=cfg.max_seq, tokens_per_seq=seq)
        else:
            qkv = g.op("llm::MatMul", [n1, f"l{l}.wqkv"], transB=1)
            q = g.op("b200::QkvRopeAppend", [qkv, pos, kc, vc], n_heads=cfg.heads, n_kv_heads=cfg.kv_heads, head_dim=D, theta=cfg.theta,
                     tokens_per_seq=seq)
        a = g.op("b200::AttentionPrefill", [q, kc, vc], n_heads=cfg.heads, seq_len=seq)
        h = g.op("llm::MatMul", [a, f"l{l}.wo", x], transB=1)           # Y = A W^T + 1 * C: the residual add rides in the epilogue
        n2 = g.op("llm::RmsNormalization", [h, f"l{l}.norm2"], epsilon=cfg.eps)
        if fused_rope and cfg.ffn % 128 == 0 and n > 64:
            u = g.op("b200::Linear", [n2, f"l{l}.wgu"], prologue=0, epilogue=2)     # silu(gate) * up in the GEMM epilogue
        else:
            gu = g.op("llm::MatMul", [n2, f"l{l}.wgu"], transB=1)
            u = g.op("b200::SwiGLU", [gu])
        x = g.op("llm::MatMul", [u, f"l{l}.wd", h], transB=1)
    xl = g.op("onnx::Gather", [x, last], axis=0)
    xf = g.op("llm::RmsNormalization", [xl, "norm_f"], epsilon=cfg.eps)
    logits = g.op("llm::MatMul", [xf, "lm_head"], transB=1)
    probs, idx = g.op("llm::TopK", [logits], n_out=2, k=top_k, softmax=1)
    index = {"next": g.output(idx), "probs": g.output(probs), "logits": g.output(logits)}
    index.update({name: i for i, name in enumerate(g.inputs)})
    return g, index


def shard_config(cfg: LlamaConfig, world: int) -> LlamaConfig:
    """Per-rank shape of a tensor-parallel model: heads, kv heads and FFN columns split `world` ways."""
    assert cfg.heads % world == 0 and cfg.kv_heads % world == 0 and cfg.ffn % world == 0
    from dataclasses import replace
    return replace(cfg, heads=cfg.heads // world, kv_heads=cfg.kv_heads // world, ffn=cfg.ffn // world)


def shard_weights(cfg: LlamaConfig, weights: dict, world: int, rank: int) -> dict:
    """Megatron-style split of full weights for rank `rank` of `world`: column-parallel QKV (whole heads per rank)
    and gate/up, row-parallel O and down; norms, embedding and LM head replicated."""
    D, nH, nKV, F = cfg.head_dim, cfg.heads, cfg.kv_heads, cfg.ffn
    hr, kr, fr = nH // world, nKV // world, F // world
    out = {}
    for name, w in weights.items():
        if name.endswith(".wqkv"):
            q, k, v = w[: nH * D], w[nH * D: (nH + nKV) * D], w[(nH + nKV) * D:]
            out[name] = np.concatenate([q[rank * hr * D: (rank + 1) * hr * D], k[rank * kr * D: (rank + 1) * kr * D],
                                        v[rank * kr * D: (rank + 1) * kr * D]])
        elif name.endswith(".wo"):
            out[name] = np.ascontiguousarray(w[:, rank * hr * D: (rank + 1) * hr * D])
        elif name.endswith(".wgu"):
            out[name] = np.concatenate([w[rank * fr: (rank + 1) * fr], w[F + rank * fr: F + (rank + 1) * fr]])
        elif name.endswith(".wd"):
            out[name] = np.ascontiguousarray(w[:, rank * fr: (rank + 1) * fr])
        else:
            out[name] = w
    return out


def decode_step_graph_batched(cfg: LlamaConfig, world: int = 1, paged: bool = False, page: int = 16, max_blocks: int = 0,
                              n_blocks: int = 0, top_k: int = 1, sample: bool = False, temperature: float = 1.0, seed: int = 0):
    """Decode step for any batch size, optionally one rank of a tensor-parallel group and/or a paged KV cache.
    `cfg` holds the PER-RANK shape (see shard_config).  Per layer: RmsNormalization, MatMul (tensor cores for
    batch > 4), QkvRopeAppend, AttentionDecode, MatMul, AllReduceSum(+residual) or Add, RmsNormalization, MatMul,
    SwiGLU, MatMul, AllReduceSum(+residual) or Add."""
    g = GraphBuilder()
    B, H, D = cfg.batch, cfg.hidden, cfg.head_dim
    token = g.input("token", I64, (B,))
    pos = g.input("pos", I64, (B,))
    lens = g.input("lens", I64, (B,))
    step = g.input("step", I64, (1,)) if sample else None
    table = g.input("block_table", I32, (B, max_blocks)) if paged else None
    for name, shape in weight_inputs(cfg):
        g.input(name, cfg.dtype, shape)
    cache_shape = (n_blocks, cfg.kv_heads, page, D) if paged else (B, cfg.kv_heads, cfg.max_seq, D)
    for l in range(cfg.layers):
        g.input(f"l{l}.k_cache", cfg.dtype, cache_shape)
        g.input(f"l{l}.v_cache", cfg.dtype, cache_shape)
    x = g.op("onnx::Gather", ["embed", token], axis=0)
    for l in range(cfg.layers):
        kc, vc = f"l{l}.k_cache", f"l{l}.v_cache"
        n1 = g.op("llm::RmsNormalization", [x, f"l{l}.norm1"], epsilon=cfg.eps)
        qkv = g.op("llm::MatMul", [n1, f"l{l}.wqkv"], transB=1)
        q = g.op("b200::QkvRopeAppend", [qkv, pos] + ([table] if paged else []) + [kc, vc], n_heads=cfg.heads,
                 n_kv_heads=cfg.kv_heads, head_dim=D, page_size=page if paged else 0, theta=cfg.theta)
        q3 = g.op("onnx::Reshape", [q], shape=[B, cfg.heads, D])
        a = g.op("b200::AttentionDecode", [q3, kc, vc, lens] + ([table] if paged else []), max_len=cfg.max_seq, page_size=page if paged else 0)
        a2 = g.op("onnx::Reshape", [a], shape=[B, cfg.heads * D])
        if world > 1:
            o = g.op("llm::MatMul", [a2, f"l{l}.wo"], transB=1)
            h = g.op("onnx::AllReduceSum", [o, x])
        else:
            h = g.op("llm::MatMul", [a2, f"l{l}.wo", x], transB=1)      # residual add in the GEMM epilogue
        n2 = g.op("llm::RmsNormalization", [h, f"l{l}.norm2"], epsilon=cfg.eps)
        gu = g.op("llm::MatMul", [n2, f"l{l}.wgu"], transB=1)
        u = g.op("b200::SwiGLU", [gu])
        if world > 1:
            d = g.op("llm::MatMul", [u, f"l{l}.wd"], transB=1)
            x = g.op("onnx::AllReduceSum", [d, h])
        else:
            x = g.op("llm::MatMul", [u, f"l{l}.wd", h], transB=1)
    xf = g.op("llm::RmsNormalization", [x, "norm_f"], epsilon=cfg.eps)
    logits = g.op("llm::MatMul", [xf, "lm_head"], transB=1)
    index = {}
    if sample:
        nxt = g.op("b200::TopKSample", [logits, step], k=top_k, temperature=temperature, seed=seed)
        g.op("b200::StateUpdate", [step], n_out=0, delta=1)
        index["next"] = g.output(nxt)
    else:
        probs, idx = g.op("llm::TopK", [logits], n_out=2, k=top_k, softmax=1)
        nxt = g.op("onnx::Reshape", [idx], shape=[B]) if top_k == 1 else None
        index["next"] = g.output(idx)
        index["probs"] = g.output(probs)
    index["logits"] = g.output(logits)
    if nxt is not None:
        g.op("b200::StateUpdate", [token, nxt], n_out=0, delta=0)
    g.op("b200::StateUpdate", [pos], n_out=0, delta=1)
    g.op("b200::StateUpdate", [lens], n_out=0, delta=1)
    index.update({name: i for i, name in enumerate(g.inputs)})
    return g, index


def prefill_graph_reference_ops(cfg: LlamaConfig, weights: dict, seq: int, top_k: int = 5):
    """Causal prefill of `seq` tokens (batch 1) using only operators the reference has kernels for; fp32.
    `weights` maps the names of `weight_inputs` to numpy arrays (wqkv/wgu are split here into the separate
    projections a reference graph would hold).  Outputs: logits [seq, vocab] and the top-k indices / values."""
    g = GraphBuilder()
    H, D, nH, nKV, F = cfg.hidden, cfg.head_dim, cfg.heads, cfg.kv_heads, cfg.ffn
    assert nH == nKV, "the reference-op graph spells attention with batched MatMul: MHA only"
    ids = g.input("ids", I64, (1, seq))
    g.constant("embed", weights["embed"])
    mask = np.tril(np.ones((seq, seq), np.bool_))[None, None]
    g.constant("mask", mask)
    g.constant("neg", np.float32([-3.0e38]))
    g.constant("scale", np.float32([np.sqrt(D)]))
    x = g.op("onnx::Gather", ["embed", ids], axis=0)                       # [1, S, H]
    for l in range(cfg.layers):
        wqkv = weights[f"l{l}.wqkv"]
        wq, wk, wv = wqkv[: nH * D], wqkv[nH * D: (nH + nKV) * D], wqkv[(nH + nKV) * D:]
        wgu = weights[f"l{l}.wgu"]
        for nm, w in (("wq", wq), ("wk", wk), ("wv", wv), ("wo", weights[f"l{l}.wo"]), ("wg", wgu[:F]), ("wu", wgu[F:]),
                      ("wd", weights[f"l{l}.wd"])):
            g.constant(f"l{l}.{nm}", np.ascontiguousarray(w.T))             # stored [in, out]: plain MatMul
        g.constant(f"l{l}.norm1", weights[f"l{l}.norm1"])
        g.constant(f"l{l}.norm2", weights[f"l{l}.norm2"])
        n1 = g.op("llm::RmsNormalization", [x, f"l{l}.norm1"], epsilon=cfg.eps)
        heads = []
        for nm in ("wq", "wk", "wv"):
            p = g.op("onnx::MatMul", [n1, f"l{l}.{nm}"])                    # [1, S, nH*D]
            p = g.op("onnx::Reshape", [p], shape=[1, seq, nH, D])
            heads.append(g.op("onnx::Transpose", [p], perm=[0, 2, 1, 3]))   # [1, nH, S, D]
        q, k, v = heads
        kt = g.op("onnx::Transpose", [k], perm=[0, 1, 3, 2])
        s = g.op("onnx::MatMul", [q, kt])                                   # [1, nH, S, S]
        s = g.op("onnx::Div", [s, "scale"])
        s = g.op("onnx::Where", ["mask", s, "neg"])
        p = g.op("onnx::Softmax", [s], axis=3)
        a = g.op("onnx::MatMul", [p, v])                                    # [1, nH, S, D]
        a = g.op("onnx::Transpose", [a], perm=[0, 2, 1, 3])
        a = g.op("onnx::Reshape", [a], shape=[1, seq, nH * D])
        o = g.op("onnx::MatMul", [a, f"l{l}.wo"])
        x = g.op("onnx::Add", [x, o])
        n2 = g.op("llm::RmsNormalization", [x, f"l{l}.norm2"], epsilon=cfg.eps)
        gt = g.op("onnx::MatMul", [n2, f"l{l}.wg"])
        up = g.op("onnx::MatMul", [n2, f"l{l}.wu"])
        sg = g.op("onnx::Sigmoid", [gt])
        act = g.op("onnx::Mul", [gt, sg])
        act = g.op("onnx::Mul", [act, up])
        dn = g.op("onnx::MatMul", [act, f"l{l}.wd"])
        x = g.op("onnx::Add", [x, dn])
    g.constant("norm_f", weights["norm_f"])
    g.constant("lm_head", np.ascontiguousarray(weights["lm_head"].T))
    xf = g.op("llm::RmsNormalization", [x, "norm_f"], epsilon=cfg.eps)
    logits = g.op("onnx::MatMul", [xf, "lm_head"])                          # [1, S, V]
    logits2 = g.op("onnx::Reshape", [logits], shape=[seq, cfg.vocab])
    vals, idx = g.op("llm::TopK", [logits2], n_out=2, k=top_k, softmax=0)
    index = {"logits": g.output(logits2), "topk_idx": g.output(idx), "topk_val": g.output(vals)}
    return g, index


def seeded_weights(cfg: LlamaConfig, seed: int = 0, np_dtype=np.float32) -> dict:
    """Weights ~ N(0, 0.02) drawn from numpy's default_rng(seed) in fp32 and rounded to np_dtype; norm weights
    are 1 + N(0, 0.02)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in weight_inputs(cfg):
        w = 0.02 * rng.standard_normal(shape, dtype=np.float32)
        if "norm" in name:
            w = 1.0 + w
        out[name] = w.astype(np_dtype)
    return out
