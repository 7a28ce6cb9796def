"""Causal flash attention for prefill (tensor-core kernel behind rg_b200_attention and rg_b200_attn_prefill) against the
numpy oracle at small sizes and a torch fp32 evaluation of the same formula at the benchmark's size."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as onp
from refactorgraph_b200 import capi

import _ops as ops

pytestmark = pytest.mark.gpu
HALF = [torch.float16, torch.bfloat16]


def _rnd(a, dtype):
    return torch.from_numpy(a).to(dtype).float().numpy()


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("N,nH,nKV,S,past", [(1, 4, 4, 64, 0), (2, 8, 2, 100, 37), (1, 2, 1, 257, 0), (1, 2, 2, 16, 200), (3, 4, 4, 65, 63)])
def test_reference_layout_operator(dtype, N, nH, nKV, S, past):
    D = 128
    rng = np.random.default_rng(N + nH + S + past)
    q = _rnd(rng.standard_normal((N, nH, S, D)).astype(np.float32), dtype)
    k = _rnd(rng.standard_normal((N, nKV, S, D)).astype(np.float32), dtype)
    v = _rnd(rng.standard_normal((N, nKV, S, D)).astype(np.float32), dtype)
    if past == 0:
        o = ops.attention(ops.dev(q, dtype), ops.dev(k, dtype), ops.dev(v, dtype))
        want, _, _ = onp.attention(q, k, v)
    else:
        max_seq = past + S + 5
        kc = _rnd(rng.standard_normal((N, nKV, max_seq, D)).astype(np.float32), dtype)
        vc = _rnd(rng.standard_normal((N, nKV, max_seq, D)).astype(np.float32), dtype)
        kcd, vcd = ops.dev(kc, dtype), ops.dev(vc, dtype)
        o = ops.attention(ops.dev(q, dtype), ops.dev(k, dtype), ops.dev(v, dtype), past=past, k_cache=kcd, v_cache=vcd)
        want, kc2, _ = onp.attention(q, k, v, past=past, k_cache=kc, v_cache=vc)
        np.testing.assert_array_equal(kcd.float().cpu().numpy(), kc2)
    np.testing.assert_allclose(o.float().cpu().numpy(), want, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", HALF)
def test_token_major_strides_from_a_fused_qkv_buffer(dtype):
    """q, k, v read in place from one [N, S, (nH + 2 nKV) * D] projection output; o written token-major."""
    N, S, nH, nKV, D = 2, 300, 8, 2, 128
    rng = np.random.default_rng(5)
    W = (nH + 2 * nKV) * D
    qkv = torch.from_numpy(rng.standard_normal((N, S, W)).astype(np.float32)).to(dtype).cuda()
    o = torch.empty(N, S, nH * D, dtype=dtype, device="cuda")
    p = capi.AttnPrefillParams()
    p.dtype, p.batch, p.n_heads, p.n_kv_heads, p.seq_len, p.head_dim, p.kv_capacity = ops.DT[dtype], N, nH, nKV, S, D, S
    p.strides[:] = [S * W, D, W, S * W, D, W, S * W, D, W, S * nH * D, D, nH * D]
    base = qkv.data_ptr()
    es = 2
    capi.call("attn_prefill", p, [base, base + nH * D * es, base + (nH + nKV) * D * es, 0], [o.data_ptr()])
    torch.cuda.synchronize()
    x = qkv.float().cpu().numpy()
    q = x[:, :, : nH * D].reshape(N, S, nH, D).transpose(0, 2, 1, 3)
    k = x[:, :, nH * D: (nH + nKV) * D].reshape(N, S, nKV, D).transpose(0, 2, 1, 3)
    v = x[:, :, (nH + nKV) * D:].reshape(N, S, nKV, D).transpose(0, 2, 1, 3)
    want, _, _ = onp.attention(q, k, v)
    got = o.float().cpu().numpy().reshape(N, S, nH, D).transpose(0, 2, 1, 3)
    np.testing.assert_allclose(got, want, atol=2e-2, rtol=1e-2)


def test_prefill_size_against_fp32_formula():
    """The benchmark's shape (2048 tokens, 32 heads) against the same formula evaluated in fp32 by torch, plus a property
    that needs no reference: the first row of every head attends only to itself, so o[0] = v[0]."""
    dtype = torch.bfloat16
    N, nH, S, D = 1, 32, 2048, 128
    g = torch.Generator(device="cuda").manual_seed(0)
    q, k, v = (torch.randn(N, nH, S, D, device="cuda", generator=g).to(dtype) for _ in range(3))
    o = ops.attention(q, k, v)
    s = torch.einsum("nhid,nhjd->nhij", q.float(), k.float()) / D ** 0.5
    s = s.masked_fill(~torch.tril(torch.ones(S, S, dtype=torch.bool, device="cuda")), float("-inf"))
    want = torch.einsum("nhij,nhjd->nhid", torch.softmax(s, dim=-1), v.float())
    torch.testing.assert_close(o.float(), want, atol=2e-2, rtol=1e-2)
    assert torch.equal(o[:, :, 0], v[:, :, 0])


def test_one_query_tile_kernel_in_a_child_process():
    """RG_B200_ATTN_Q2=0 selects the kernel with one query tile per CTA (read once per process, hence the child): the same
    ragged grouped-query case against the oracle, and bit-for-bit the same output twice."""
    import os
    import subprocess
    import sys
    code = r"""
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1])
sys.path.insert(0, sys.argv[2])
from oracle import oracle_np as onp
import _ops as ops
rng = np.random.default_rng(3)
N, nH, nKV, S, D = 2, 8, 2, 300, 128
r = lambda *s: torch.from_numpy(rng.standard_normal(s).astype(np.float32)).to(torch.bfloat16).float().numpy()
q, k, v = r(N, nH, S, D), r(N, nKV, S, D), r(N, nKV, S, D)
o = ops.attention(ops.dev(q, torch.bfloat16), ops.dev(k, torch.bfloat16), ops.dev(v, torch.bfloat16))
o2 = ops.attention(ops.dev(q, torch.bfloat16), ops.dev(k, torch.bfloat16), ops.dev(v, torch.bfloat16))
want, _, _ = onp.attention(q, k, v)
np.testing.assert_allclose(o.float().cpu().numpy(), want, atol=2e-2, rtol=1e-2)
assert torch.equal(o, o2)
print("child ok")
"""
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, RG_B200_ATTN_Q2="0")
    r = subprocess.run([sys.executable, "-c", code, os.path.dirname(here), here], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=600)
    assert r.returncode == 0 and "child ok" in r.stdout, r.stdout[-2000:]
