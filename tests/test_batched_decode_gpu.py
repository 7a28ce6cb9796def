"""Batched decode path (batch > 4): tensor-core MatMul + QkvRopeAppend + AttentionDecode + SwiGLU, contiguous and
paged KV cache, against the numpy oracle; and the single-GPU parts of the all-reduce (world 1, bounded wait)."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as onp
from refactorgraph_b200 import capi
from refactorgraph_b200.graph_builder import FP16
from refactorgraph_b200.llama import LlamaConfig, decode_step_graph_batched, seeded_weights, weight_inputs

import _ops as ops
from _decode_oracle import KvHistory, oracle_decode, oracle_decode_step_rounded

pytestmark = pytest.mark.gpu


def test_qkv_rope_append_and_swiglu_kernels():
    rng = np.random.default_rng(0)
    m, nq, nkv, D, page, max_blocks, n_blocks = 5, 8, 2, 128, 16, 8, 64
    qkv = torch.from_numpy(rng.standard_normal((m, (nq + 2 * nkv) * D)).astype(np.float32)).half()
    pos = rng.integers(0, page * max_blocks, (m,)).astype(np.int64)
    table = rng.permutation(n_blocks)[: m * max_blocks].reshape(m, max_blocks).astype(np.int32)
    kc = torch.zeros(n_blocks, nkv, page, D, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    q = torch.empty(m, nq * D, dtype=torch.float16, device="cuda")
    p = capi.QkvRopeAppendParams(capi.FP16, m, nq, 10000.0, ops.kv_layout(nkv, D, 0, page, max_blocks))
    qkv_d, pos_d, table_d = qkv.cuda(), ops.dev(pos), ops.dev(table)   # keep the device copies alive across the call
    capi.call("qkv_rope_append", p, [qkv_d.data_ptr(), pos_d.data_ptr(), table_d.data_ptr()],
              [q.data_ptr(), kc.data_ptr(), vc.data_ptr()])
    torch.cuda.synchronize()
    x = qkv.float().numpy()
    want_q = onp.rope(x[:, : nq * D].reshape(m, nq, D), pos)
    want_k = onp.rope(x[:, nq * D: (nq + nkv) * D].reshape(m, nkv, D), pos)
    want_v = x[:, (nq + nkv) * D:].reshape(m, nkv, D)
    np.testing.assert_allclose(q.float().cpu().numpy().reshape(m, nq, D), want_q, atol=2e-2, rtol=1e-2)
    k_got = torch.stack([kc[table[i, pos[i] // page], :, pos[i] % page] for i in range(m)]).float().cpu().numpy()
    v_got = torch.stack([vc[table[i, pos[i] // page], :, pos[i] % page] for i in range(m)]).float().cpu().numpy()
    np.testing.assert_allclose(k_got, want_k, atol=2e-2, rtol=1e-2)
    np.testing.assert_array_equal(v_got, want_v)       # v is a plain copy
    gu = torch.from_numpy(rng.standard_normal((7, 2 * 344)).astype(np.float32)).half()
    y = torch.empty(7, 344, dtype=torch.float16, device="cuda")
    gu_d = gu.cuda()
    capi.call("swiglu", capi.SwigluParams(capi.FP16, 7, 344), [gu_d.data_ptr()], [y.data_ptr()])
    torch.cuda.synchronize()
    g, u = gu.float().numpy()[:, :344], gu.float().numpy()[:, 344:]
    np.testing.assert_allclose(y.float().cpu().numpy(), onp.silu(g) * u, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("paged", [False, True])
def test_batched_decode_graph(paged):
    cfg = LlamaConfig(layers=2, hidden=512, heads=8, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, max_seq=256, batch=16)
    rng = np.random.default_rng(3)
    w16 = seeded_weights(cfg, 0, np.float16)
    w16["lm_head"] = (0.2 * rng.standard_normal(w16["lm_head"].shape)).astype(np.float16)
    w = {k: v.astype(np.float32) for k, v in w16.items()}
    B, page = cfg.batch, 16
    past = rng.integers(1, 200, (B,)).astype(np.int64)
    kc = [rng.standard_normal((B, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    vc = [rng.standard_normal((B, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    token = rng.integers(0, cfg.vocab, (B,)).astype(np.int64)
    steps = 3
    # the oracle rounds every intermediate where this graph stores it (normalised activations, products, rotated q / k, ...)
    r16 = lambda a: np.asarray(a, np.float32).astype(np.float16).astype(np.float32)
    kh = [[KvHistory(kc[l][b], past[b]) for b in range(B)] for l in range(cfg.layers)]
    vh = [[KvHistory(vc[l][b], past[b]) for b in range(B)] for l in range(cfg.layers)]
    max_blocks = cfg.max_seq // page
    n_blocks = B * max_blocks
    table = rng.permutation(n_blocks).reshape(B, max_blocks).astype(np.int32)
    g, index = decode_step_graph_batched(cfg, paged=paged, page=page, max_blocks=max_blocks, n_blocks=n_blocks)
    ex = g.compiler().compile("cuda", "flat", [])
    for name, _ in weight_inputs(cfg):
        ex.set_input(index[name], w16[name])
    for l in range(cfg.layers):
        if paged:  # scatter the contiguous caches into their pages
            for nm, src in (("k_cache", kc[l]), ("v_cache", vc[l])):
                pages = np.zeros((n_blocks, cfg.kv_heads, page, cfg.head_dim), np.float16)
                for b in range(B):
                    for j in range(max_blocks):
                        pages[table[b, j]] = src[b, :, j * page:(j + 1) * page]
                ex.set_input(index[f"l{l}.{nm}"], pages)
        else:
            ex.set_input(index[f"l{l}.k_cache"], kc[l])
            ex.set_input(index[f"l{l}.v_cache"], vc[l])
    if paged:
        ex.set_input(index["block_table"], table)
    tok = token
    for s in range(steps):
        # the GPU's own token is fed to both sides, so a legitimate arg-max flip on a near-tie cannot part the trajectories
        ex.set_input(index["token"], tok)
        ex.set_input(index["pos"], past + s)
        ex.set_input(index["lens"], past + s + 1)
        ex.run()
        want = oracle_decode_step_rounded(cfg, w, kh, vh, tok, past + s, r16)
        logits = ex.get_output(index["logits"]).astype(np.float32)
        np.testing.assert_allclose(logits, want, atol=2e-2, rtol=1e-2)
        tok = ex.get_output(index["next"])[:, 0].copy()
        np.testing.assert_array_equal(tok, onp.topk(logits, 1)[1][:, 0])           # arg-max of its own logits, bit-exact
        gap = want.max(axis=1) - want[np.arange(B), tok]
        assert (gap <= 2e-2).all()                                                   # and (near-)maximal in the oracle's
    assert capi.load().rg_b200_error_state() == 0


def test_all_reduce_world_one_and_limits():
    comm = capi.Comm(1, 0, 1 << 16)
    x = torch.arange(1000, dtype=torch.float32, device="cuda")
    r = torch.ones_like(x)
    y = torch.empty_like(x)
    comm.all_reduce(capi.F32, 0, x.numel(), x.data_ptr(), y.data_ptr())
    assert torch.equal(y, x)
    comm.all_reduce(capi.F32, 1, x.numel(), x.data_ptr(), y.data_ptr(), residual=r.data_ptr())   # Avg of one rank + residual
    assert torch.equal(y, x + 1)
    h = torch.randn(4099, device="cuda").half()                                                    # ragged tail (not a multiple of 8)
    yh = torch.empty_like(h)
    comm.all_reduce(capi.FP16, 0, h.numel(), h.data_ptr(), yh.data_ptr())
    assert torch.equal(yh, h)
    assert comm.all_reduce(capi.F32, 0, 1 << 20, x.data_ptr(), y.data_ptr(), check=False) == capi.ERR_LIMIT
    assert comm.all_reduce(capi.BOOL, 0, 8, x.data_ptr(), y.data_ptr(), check=False) == capi.ERR_DTYPE
    i64 = torch.arange(-5, 1000, dtype=torch.int64, device="cuda")                                # integer types pass through a group of one
    yi = torch.zeros_like(i64)
    comm.all_reduce(capi.I64, 0, i64.numel(), i64.data_ptr(), yi.data_ptr())
    assert torch.equal(yi, i64)
    assert comm.status() == capi.OK
    comm.destroy()


def test_fused_all_reduce_forms_on_a_group_of_one():
    """AllReduce + residual + RMSNorm in one launch, and the product whose epilogue is the sending half of the all-reduce, on
    a communicator of one rank (no second GPU needed): values against the separate kernels, and the shapes they refuse."""
    comm = capi.Comm(1, 0, 1 << 20)
    g = torch.Generator(device="cuda").manual_seed(3)
    for dt, code in ((torch.float16, capi.FP16), (torch.bfloat16, capi.BF16)):
        x = torch.randn(16, 1024, device="cuda", generator=g).to(dt)
        r = torch.randn(16, 1024, device="cuda", generator=g).to(dt)
        w = (1 + 0.1 * torch.randn(1024, device="cuda", generator=g)).to(dt)
        y0 = torch.empty_like(x)
        comm.all_reduce(code, 0, x.numel(), x.data_ptr(), y0.data_ptr(), residual=r.data_ptr())
        n0 = ops.rms_norm(y0, w, 1e-5)
        y1, n1 = torch.zeros_like(x), torch.zeros_like(x)
        comm.all_reduce_norm(code, 16, 1024, 1e-5, x.data_ptr(), w.data_ptr(), y1.data_ptr(), n1.data_ptr(), residual=r.data_ptr())
        torch.cuda.synchronize()
        assert torch.equal(y0.view(torch.int16), y1.view(torch.int16)) and torch.equal(n0.view(torch.int16), n1.view(torch.int16))
        # product + all-reduce: 16 tokens x [512, 1024] weights, residual added by the receiving half
        a = torch.randn(16, 1024, device="cuda", generator=g).to(dt)
        wt = (0.05 * torch.randn(512, 1024, device="cuda", generator=g)).to(dt)
        res = torch.randn(16, 512, device="cuda", generator=g).to(dt)
        p = capi.MatMulParams()
        p.dtype, p.m, p.n, p.k, p.trans_b, p.alpha, p.beta, p.batch, p.stride_y, p.force_kernel = code, 16, 512, 1024, 1, 1.0, 0.0, 1, 16 * 512, 3
        nws = capi.workspace("mat_mul", p)
        ws = torch.zeros(max(nws, 1), dtype=torch.uint8, device="cuda")
        part = torch.empty(16, 512, dtype=dt, device="cuda")
        capi.call("mat_mul", p, [a.data_ptr(), wt.data_ptr(), 0], [part.data_ptr()], ws=ws.data_ptr() if nws else 0)
        z0 = torch.empty_like(part)
        comm.all_reduce(code, 0, part.numel(), part.data_ptr(), z0.data_ptr(), residual=res.data_ptr())
        p.force_kernel = 0
        z1 = torch.zeros_like(part)
        comm.mat_mul_push(p, a.data_ptr(), wt.data_ptr(), ws=ws.data_ptr() if nws else 0)
        comm.all_reduce_recv(code, part.numel(), z1.data_ptr(), residual=res.data_ptr())
        torch.cuda.synchronize()
        assert torch.equal(z0.view(torch.int16), z1.view(torch.int16))
        want = (a.float() @ wt.float().T).to(dt).float() + res.float()
        assert torch.allclose(z1.float(), want, atol=2e-2, rtol=1e-2)
    # refusals: nothing is launched
    x = torch.zeros(4, 1024, dtype=torch.float16, device="cuda")
    assert comm.all_reduce_norm(capi.F32, 4, 1024, 1e-5, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), check=False) == capi.ERR_DTYPE
    assert comm.all_reduce_norm(capi.FP16, 4, 1028, 1e-5, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), check=False) == capi.ERR_SHAPE
    assert comm.all_reduce_norm(capi.FP16, 4, 32768, 1e-5, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), check=False) == capi.ERR_SHAPE
    assert comm.all_reduce_norm(capi.FP16, 1 << 12, 1024, 1e-5, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), check=False) == capi.ERR_LIMIT
    assert comm.all_reduce_norm(capi.FP16, 0, 1024, 1e-5, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), check=False) == capi.OK
    p = capi.MatMulParams()
    p.dtype, p.m, p.n, p.k, p.trans_b, p.alpha, p.batch = capi.FP16, 65, 512, 1024, 1, 1.0, 1
    assert comm.mat_mul_push(p, x.data_ptr(), x.data_ptr(), check=False) == capi.ERR_UNSUPPORTED      # more than 64 tokens
    p.m, p.n = 16, 516
    assert comm.mat_mul_push(p, x.data_ptr(), x.data_ptr(), check=False) == capi.ERR_UNSUPPORTED      # rows of Y not whole 16-byte chunks
    p.n, p.dtype = 512, capi.F32
    assert comm.mat_mul_push(p, x.data_ptr(), x.data_ptr(), check=False) == capi.ERR_UNSUPPORTED
    p.dtype, p.m, p.n = capi.FP16, 64, 1 << 14
    assert comm.mat_mul_push(p, x.data_ptr(), x.data_ptr(), check=False) == capi.ERR_LIMIT            # 2 MiB of results, 1 MiB of slots
    assert comm.all_reduce_recv(capi.FP16, 1004, x.data_ptr(), check=False) == capi.ERR_SHAPE            # not whole 16-byte chunks
    assert comm.status() == capi.OK and capi.load().rg_b200_error_state() == 0
    comm.destroy()


def test_all_reduce_missing_peer_reports_timeout_instead_of_hanging():
    """Failure detection without faulting a GPU: rank 0 of a 2-rank group whose peer never raises its flag (a zeroed
    buffer stands in for the peer).  The device-side wait is bounded (20 ms here); the kernel returns, the status
    word says so, and the context stays usable."""
    comm = capi.Comm(2, 0, 1 << 12)
    fake_peer = torch.zeros(comm.nbytes(), dtype=torch.uint8, device="cuda")       # rank 0 stores its input there
    comm.connect_ptrs([comm.base(), fake_peer.data_ptr()])
    comm.set_wait_ns(20_000_000)
    x = torch.ones(256, device="cuda")
    y = torch.full_like(x, -1.0)
    comm.all_reduce(capi.F32, 0, x.numel(), x.data_ptr(), y.data_ptr())
    assert comm.status() == capi.ERR_TIMEOUT
    assert capi.load().rg_b200_error_state() & 8             # bit 3: a communicator on this device gave up a wait
    assert torch.equal(y, torch.full_like(x, -1.0))          # output left untouched
    z = x + 1                                                   # the context is still alive
    assert float(z.sum()) == 512.0
    # the communicator is out of step with its peers for good: a second call is refused on the host ...
    assert comm.all_reduce(capi.F32, 0, x.numel(), x.data_ptr(), y.data_ptr(), check=False) == capi.ERR_TIMEOUT
    assert torch.equal(y, torch.full_like(x, -1.0)) and comm.status() == capi.ERR_TIMEOUT
    comm.destroy()
    assert capi.load().rg_b200_error_state() == 0            # ... and the error follows the communicator, not the library
    # a communicator that is recreated works again (a group of one here: no second GPU is needed to show it)
    fresh = capi.Comm(1, 0, 1 << 12)
    fresh.all_reduce(capi.F32, 0, x.numel(), x.data_ptr(), y.data_ptr())
    assert torch.equal(y, x) and fresh.status() == capi.OK
    fresh.destroy()


@pytest.mark.parametrize("np_dtype", [np.float16])
def test_prefill_graph(np_dtype):
    """Token-major causal prefill (tensor-core MatMul + QkvRopeAppend + AttentionPrefill + SwiGLU): last-token logits and
    the K/V caches it writes, against the numpy oracle."""
    from refactorgraph_b200.llama import prefill_graph
    cfg = LlamaConfig(layers=2, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, max_seq=128, batch=2)
    S, B, D, nH, nKV = 80, 2, 128, 4, 2
    rng = np.random.default_rng(11)
    w16 = seeded_weights(cfg, 0, np_dtype)
    w = {k: v.astype(np.float32) for k, v in w16.items()}
    r16 = lambda a: np.asarray(a, np.float32).astype(np_dtype).astype(np.float32)
    ids = rng.integers(0, cfg.vocab, (B, S)).astype(np.int64)
    pos = np.tile(np.arange(S, dtype=np.int64), B)
    # oracle
    x = w["embed"][ids.ravel()]
    k_want, v_want = [], []
    for l in range(cfg.layers):
        q, k, v = onp.linear_fused(x, w[f"l{l}.wqkv"], g=w[f"l{l}.norm1"], eps=cfg.eps, epilogue=3, n_heads=nH, n_kv=nKV, head_dim=D, positions=pos)
        # the GPU path rounds the normalised activations and the projection before the rotation
        n1 = r16(onp.rms_norm(x, w[f"l{l}.norm1"], cfg.eps))
        qkv = r16(n1.astype(np.float64) @ w[f"l{l}.wqkv"].astype(np.float64).T)
        q = r16(onp.rope(qkv[:, : nH * D].reshape(-1, nH, D), pos))
        k = r16(onp.rope(qkv[:, nH * D: (nH + nKV) * D].reshape(-1, nKV, D), pos))
        v = qkv[:, (nH + nKV) * D:].reshape(-1, nKV, D)
        k_want.append(k), v_want.append(v)
        to4 = lambda t, h: t.reshape(B, S, h, D).transpose(0, 2, 1, 3)
        a, _, _ = onp.attention(to4(q, nH), to4(k, nKV), to4(v, nKV))
        a = r16(a.transpose(0, 2, 1, 3).reshape(B * S, nH * D))
        h = r16(r16(a.astype(np.float64) @ w[f"l{l}.wo"].astype(np.float64).T) + x)
        n2 = r16(onp.rms_norm(h, w[f"l{l}.norm2"], cfg.eps))
        gu = r16(n2.astype(np.float64) @ w[f"l{l}.wgu"].astype(np.float64).T)
        u = r16(onp.silu(gu[:, : cfg.ffn]) * gu[:, cfg.ffn:])
        x = r16(r16(u.astype(np.float64) @ w[f"l{l}.wd"].astype(np.float64).T) + h)
    last = np.array([S - 1, 2 * S - 1], np.int64)
    xf = r16(onp.rms_norm(x[last], w["norm_f"], cfg.eps))
    want_logits = xf.astype(np.float64) @ w["lm_head"].astype(np.float64).T
    # GPU
    g, index = prefill_graph(cfg, S)
    ex = g.compiler().compile("cuda", "flat", [])
    for name, _ in weight_inputs(cfg):
        ex.set_input(index[name], w16[name])
    ex.set_input(index["ids"], ids.ravel())
    ex.set_input(index["positions"], pos)
    ex.set_input(index["last"], last)
    ex.run()
    logits = ex.get_output(index["logits"]).astype(np.float32)
    np.testing.assert_allclose(logits, want_logits, atol=2e-2, rtol=1e-2)
    ex.run()  # CUDA-graph replay: same bytes
    np.testing.assert_array_equal(ex.get_output(index["logits"]).astype(np.float32), logits)
    assert capi.load().rg_b200_error_state() == 0
