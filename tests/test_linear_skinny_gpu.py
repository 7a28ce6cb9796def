"""The streaming linear kernel for 5..32 rows of X (batched decode, one rank of a tensor-parallel step) against the numpy
oracle: every epilogue, one and two row tiles, one and several k parts, ragged row and column counts, contiguous and paged
caches, repeated calls on one workspace (the arrival counters reset themselves), and the MatMul entry point's routing."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as onp
from refactorgraph_b200 import capi

import _ops as ops

pytestmark = pytest.mark.gpu


def r16(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dtype).float().numpy()


def close(got, want, atol=2e-2, rtol=1e-2):
    np.testing.assert_allclose(got.float().cpu().numpy(), want, atol=atol, rtol=rtol)


@pytest.mark.parametrize("m,n,k", [(5, 1280, 8192), (16, 8192, 1024), (16, 1000, 256), (17, 4096, 4096), (32, 1288, 11008), (9, 24, 128)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_plain_and_residual_products(m, n, k, dtype):
    rng = np.random.default_rng(m * 1000 + n + k)
    x = r16(rng.standard_normal((m, k)), dtype)
    w = r16(rng.standard_normal((n, k)) / np.sqrt(k), dtype)
    r = r16(rng.standard_normal((m, n)), dtype)
    xd, wd, rd = ops.dev(x, dtype), ops.dev(w, dtype), ops.dev(r, dtype)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    tol = dict(atol=2e-2, rtol=1e-2) if dtype == torch.float16 else dict(atol=4e-2, rtol=2e-2)   # outputs of magnitude ~1-4 stored in bf16
    close(ops.linear(xd, wd), want, **tol)
    close(ops.linear(xd, wd, residual=rd, epilogue=1), want + r, **tol)
    # the MatMul entry point can be told to use this kernel (force 4); left alone it picks it for up to 16 rows against few
    # weight rows with a long k, where it is the faster one, and the tensor-core kernel otherwise
    y_auto = ops.mat_mul(xd, wd, trans_b=True)
    y_forced = ops.mat_mul(xd, wd, trans_b=True, force=4)
    close(y_auto, want, **tol)
    close(y_forced, want, **tol)
    if m <= 16 and n <= 2560 and k >= 4096:
        assert torch.equal(y_auto, y_forced)
    close(ops.mat_mul(xd, wd, c=rd, trans_b=True, alpha=0.5, beta=2.0, force=4), 0.5 * want + 2.0 * r, **tol)
    bias = r16(rng.standard_normal(n), dtype)
    close(ops.mat_mul(xd, wd, c=ops.dev(bias, dtype), trans_b=True, force=4), want + bias, **tol)  # row-broadcast bias
    assert capi.load().rg_b200_error_state() == 0


@pytest.mark.parametrize("m,f,k", [(16, 3584, 8192), (32, 11008, 4096), (7, 344, 256), (20, 1001 * 2 // 2, 384)])
def test_silu_gate_epilogue(m, f, k):
    dtype = torch.float16
    rng = np.random.default_rng(m + f)
    x = r16(rng.standard_normal((m, k)), dtype)
    w = r16(rng.standard_normal((2 * f, k)) / np.sqrt(k), dtype)
    got = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), epilogue=2)
    assert got.shape == (m, f)
    gu = x.astype(np.float64) @ w.astype(np.float64).T
    close(got, onp.silu(gu[:, :f]) * gu[:, f:])
    assert capi.load().rg_b200_error_state() == 0


@pytest.mark.parametrize("m,nq,nkv,D,k,paged", [(16, 8, 1, 128, 8192, False), (32, 32, 32, 128, 4096, True), (6, 4, 2, 64, 512, False),
                                                (16, 8, 2, 128, 1024, True)])
def test_qkv_rope_append_epilogue(m, nq, nkv, D, k, paged):
    dtype = torch.float16
    rng = np.random.default_rng(m + nq + k)
    x = r16(rng.standard_normal((m, k)), dtype)
    w = r16(rng.standard_normal(((nq + 2 * nkv) * D, k)) / np.sqrt(k), dtype)
    page, max_blocks = 16, 6
    max_seq = page * max_blocks
    pos = rng.integers(0, max_seq, (m,)).astype(np.int64)
    if paged:
        n_blocks = m * max_blocks
        table = rng.permutation(n_blocks).reshape(m, max_blocks).astype(np.int32)
        kc = torch.zeros(n_blocks, nkv, page, D, dtype=dtype, device="cuda")
        kv = ops.kv_layout(nkv, D, 0, page, max_blocks, n_blocks)
        td = ops.dev(table)
    else:
        kc = torch.zeros(m, nkv, max_seq, D, dtype=dtype, device="cuda")
        kv, td = ops.kv_layout(nkv, D, max_seq), None
    vc = torch.zeros_like(kc)
    for _ in range(2):                      # twice on purpose: a fresh workspace each call, identical results
        q = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), epilogue=3, n_heads=nq, kv=kv, positions=ops.dev(pos), table=td,
                       k_cache=kc, v_cache=vc)
    y = x.astype(np.float64) @ w.astype(np.float64).T
    want_q = onp.rope(y[:, : nq * D].reshape(m, nq, D), pos)
    want_k = onp.rope(y[:, nq * D: (nq + nkv) * D].reshape(m, nkv, D), pos)
    want_v = y[:, (nq + nkv) * D:].reshape(m, nkv, D)
    close(q.reshape(m, nq, D), want_q)
    if paged:
        k_got = torch.stack([kc[table[i, pos[i] // page], :, pos[i] % page] for i in range(m)])
        v_got = torch.stack([vc[table[i, pos[i] // page], :, pos[i] % page] for i in range(m)])
    else:
        k_got = torch.stack([kc[i, :, pos[i]] for i in range(m)])
        v_got = torch.stack([vc[i, :, pos[i]] for i in range(m)])
    close(k_got, want_k)
    close(v_got, want_v)
    assert int((kc != 0).any(dim=-1).sum()) == m * nkv        # nothing but the m appended rows was written
    assert capi.load().rg_b200_error_state() == 0


def test_workspace_is_reusable_and_results_are_deterministic():
    dtype, m, n, k = torch.float16, 16, 7168, 8192              # four k parts
    rng = np.random.default_rng(0)
    xd = ops.dev(r16(rng.standard_normal((m, k)), dtype), dtype)
    wd = ops.dev(r16(rng.standard_normal((n, k)) / np.sqrt(k), dtype), dtype)
    p = capi.LinearParams()
    p.dtype, p.m, p.n, p.k = capi.FP16, m, n, k
    nws = capi.workspace("linear", p)
    assert nws > 0
    ws = torch.zeros(nws, dtype=torch.uint8, device="cuda")
    outs = []
    for _ in range(4):                                           # the same workspace, never cleared between calls
        y = torch.empty(m, n, dtype=dtype, device="cuda")
        capi.call("linear", p, [xd.data_ptr(), wd.data_ptr(), 0, 0, 0, 0], [y.data_ptr(), 0, 0], ws=ws.data_ptr(), stream=ops.stream())
        torch.cuda.synchronize()
        outs.append(y)
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    assert capi.call("linear", p, [xd.data_ptr(), wd.data_ptr(), 0, 0, 0, 0], [outs[0].data_ptr(), 0, 0], ws=0, check=False) == capi.ERR_NULL


def test_out_of_range_append_is_skipped():
    dtype, m, nq, nkv, D, k, max_seq = torch.float16, 8, 4, 2, 128, 512, 16
    rng = np.random.default_rng(1)
    x = ops.dev(r16(rng.standard_normal((m, k)), dtype), dtype)
    w = ops.dev(r16(rng.standard_normal(((nq + 2 * nkv) * D, k)) / np.sqrt(k), dtype), dtype)
    kc = torch.zeros(m, nkv, max_seq, D, dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    pos = np.arange(m, dtype=np.int64)
    pos[3] = max_seq
    ops.linear(x, w, epilogue=3, n_heads=nq, kv=ops.kv_layout(nkv, D, max_seq), positions=ops.dev(pos), k_cache=kc, v_cache=vc)
    torch.cuda.synchronize()
    lib = capi.load()
    assert lib.rg_b200_error_state() == 32
    assert lib.rg_b200_error_clear() == capi.OK
    assert not (kc[3] != 0).any() and not (vc[3] != 0).any() and (kc[2, :, 2] != 0).any()
