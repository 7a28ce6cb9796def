"""Host-side tensor-parallel logic without a GPU: the weight splitter, and the exchange order of one decoder layer
run as two gloo ranks (each rank computes its shard with the numpy oracle, the partial outputs are summed with
all_reduce, and every rank must reproduce the unsharded result)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle_np as onp
from refactorgraph_b200.llama import LlamaConfig, seeded_weights, shard_config, shard_weights

CFG = dict(layers=1, hidden=64, heads=4, kv_heads=2, head_dim=16, ffn=96, vocab=50, max_seq=16, batch=3)


def _layer(cfg, w, x, kc, vc, pos, reduce):
    """One decoder layer on the (possibly sharded) weights; `reduce` sums partial outputs across ranks."""
    B, D = x.shape[0], cfg.head_dim
    q, k, v = onp.linear_fused(x, w["l0.wqkv"], g=w["l0.norm1"], eps=cfg.eps, epilogue=3, n_heads=cfg.heads, n_kv=cfg.kv_heads,
                               head_dim=D, positions=pos)
    kc, vc = kc.copy(), vc.copy()
    for b in range(B):
        kc[b, :, pos[b]], vc[b, :, pos[b]] = k[b], v[b]
    a = onp.attn_decode(q, kc, vc, pos + 1).reshape(B, cfg.heads * D)
    h = x + reduce(a.astype(np.float64) @ w["l0.wo"].astype(np.float64).T)
    u = onp.linear_fused(h.astype(np.float32), w["l0.wgu"], g=w["l0.norm2"], eps=cfg.eps, epilogue=2)
    return h + reduce(u.astype(np.float64) @ w["l0.wd"].astype(np.float64).T)


def _inputs(cfg):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((cfg.batch, cfg.hidden)).astype(np.float32)
    kc = rng.standard_normal((cfg.batch, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float32)
    vc = rng.standard_normal((cfg.batch, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float32)
    pos = np.array([3, 7, 11], np.int64)
    return x, kc, vc, pos


def test_shard_weights_reassemble():
    cfg = LlamaConfig(**CFG)
    w = seeded_weights(cfg, 0)
    parts = [shard_weights(cfg, w, 2, r) for r in range(2)]
    sc = shard_config(cfg, 2)
    assert parts[0]["l0.wqkv"].shape == ((sc.heads + 2 * sc.kv_heads) * cfg.head_dim, cfg.hidden)
    np.testing.assert_array_equal(np.concatenate([p["l0.wo"] for p in parts], axis=1), w["l0.wo"])
    np.testing.assert_array_equal(np.concatenate([p["l0.wd"] for p in parts], axis=1), w["l0.wd"])
    F, fr = cfg.ffn, cfg.ffn // 2
    np.testing.assert_array_equal(np.concatenate([p["l0.wgu"][:fr] for p in parts]), w["l0.wgu"][:F])
    np.testing.assert_array_equal(np.concatenate([p["l0.wgu"][fr:] for p in parts]), w["l0.wgu"][F:])
    with pytest.raises(AssertionError):
        shard_config(cfg, 3)


def test_sharded_layer_equals_unsharded_in_one_process():
    cfg = LlamaConfig(**CFG)
    w = seeded_weights(cfg, 0)
    x, kc, vc, pos = _inputs(cfg)
    want = _layer(cfg, w, x, kc, vc, pos, lambda p: p)
    sc = shard_config(cfg, 2)
    partial = []

    def collect(p):
        partial.append(p)
        return p
    # run both ranks, recording the partials of each reduce point, then replay with the summed values
    sums = []
    for point in range(2):
        vals = []
        for r in range(2):
            ws = shard_weights(cfg, w, 2, r)
            kr = cfg.kv_heads // 2
            seen = []

            def red(p, seen=seen):
                seen.append(p)
                return sums[len(seen) - 1] if len(seen) - 1 < len(sums) else p
            _layer(sc, ws, x, kc[:, r * kr:(r + 1) * kr], vc[:, r * kr:(r + 1) * kr], pos, red)
            vals.append(seen[point])
        sums.append(vals[0] + vals[1])
    got = _layer(sc, shard_weights(cfg, w, 2, 0), x, kc[:, :1], vc[:, :1], pos, lambda p, it=iter(sums): next(it))
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-7)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = LlamaConfig(**CFG)
    w = seeded_weights(cfg, 0)
    x, kc, vc, pos = _inputs(cfg)
    sc, kr = shard_config(cfg, world), cfg.kv_heads // world

    def reduce(p):
        t = torch.from_numpy(np.ascontiguousarray(p))
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t.numpy()
    got = _layer(sc, shard_weights(cfg, w, world, rank), x, kc[:, rank * kr:(rank + 1) * kr], vc[:, rank * kr:(rank + 1) * kr], pos, reduce)
    want = _layer(cfg, w, x, kc, vc, pos, lambda p: p)
    ok = np.allclose(got, want, rtol=1e-6, atol=1e-7)
    # a rank that never joins the next collective is noticed through the process-group timeout, not by a hang
    out.put((rank, bool(ok)))
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_layer():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
