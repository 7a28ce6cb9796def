"""Parity of the sm_100a kernels (through the C ABI) with the oracle on seeded inputs.

Tolerances: byte/index work (gather, transpose, where, top-k indices) is bit-exact.  fp32 kernels: 1e-5 relative
(fp32 statistics in a different summation order than the sequential CPU loop).  fp16/bf16 kernels: outputs are
compared with the fp32/fp64 oracle evaluated on the same rounded inputs, max-abs 2e-2 / relative 1e-2.
"""
import os

import numpy as np
import pytest
import torch

import oracle
from oracle import oracle_np as onp
from refactorgraph_b200 import capi

import _ops as ops

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_kernels.npz"))
HALF = [torch.float16, torch.bfloat16]


def close_half(got, want, atol=2e-2, rtol=1e-2):
    np.testing.assert_allclose(got.float().cpu().numpy(), want, atol=atol, rtol=rtol)


def rnd16(a, dtype):
    """Round an fp32 array to the run dtype and back (the oracle sees exactly what the GPU sees)."""
    return torch.from_numpy(a).to(dtype).float().numpy()


# ---- RMSNorm ---------------------------------------------------------------------------------------------------
def test_rms_norm_reference_vectors():
    # src/04kernel/test/kernels/rms_normalization/test_cpu.cpp:21-38, literally: x = 0..23 as [2,3,4], w = 1..4, eps = 0
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    w = np.arange(1, 5, dtype=np.float32)
    expect = np.stack([row * np.float32(1.0 / np.sqrt(np.float32((row * row).sum() / 4))) * w for row in x.reshape(6, 4)]).reshape(2, 3, 4)
    got = ops.rms_norm(ops.dev(x), ops.dev(w), 0.0).cpu().numpy()
    np.testing.assert_allclose(got, expect, rtol=4e-7 * 4)           # EXPECT_FLOAT_EQ is 4 ULP
    np.testing.assert_allclose(got, oracle.port_rms_norm(x, w, 0.0), rtol=1e-6)
    x = np.full((2, 3, 4096), 2, np.float32)
    w = np.full(4096, 3, np.float32)
    np.testing.assert_allclose(ops.rms_norm(ops.dev(x), ops.dev(w), 0.0).cpu().numpy(), 3.0, rtol=1e-6)


@pytest.mark.parametrize("tag", ["rms_a", "rms_b"])
def test_rms_norm_golden(tag):
    y = ops.rms_norm(ops.dev(GOLD[f"{tag}_x"]), ops.dev(GOLD[f"{tag}_w"]), 1e-6)
    np.testing.assert_allclose(y.cpu().numpy(), GOLD[f"{tag}_y"], rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("rows,dim", [(1, 4096), (32, 4096), (3, 8192), (5, 11008), (7, 100), (2, 20000), (1, 1)])
@pytest.mark.parametrize("dtype", [torch.float32] + HALF)
def test_rms_norm_seeded(rows, dim, dtype):
    rng = np.random.default_rng(rows * 131 + dim)
    x = rnd16(rng.standard_normal((rows, dim)).astype(np.float32), dtype)
    w = rnd16((1 + 0.1 * rng.standard_normal(dim)).astype(np.float32), dtype)
    y = ops.rms_norm(ops.dev(x, dtype), ops.dev(w, dtype), 1e-6)
    want = onp.rms_norm(x, w, 1e-6)
    if dtype == torch.float32:
        np.testing.assert_allclose(y.cpu().numpy(), want, rtol=1e-5, atol=1e-6)
    else:
        close_half(y, want)


@pytest.mark.parametrize("dtype", HALF)
def test_rms_norm_residual(dtype):
    rng = np.random.default_rng(5)
    x = rnd16(rng.standard_normal((4, 4096)).astype(np.float32), dtype)
    r = rnd16(rng.standard_normal((4, 4096)).astype(np.float32), dtype)
    w = rnd16(rng.standard_normal(4096).astype(np.float32), dtype)
    y, s = ops.rms_norm(ops.dev(x, dtype), ops.dev(w, dtype), 1e-6, residual=ops.dev(r, dtype))
    s_want = rnd16(x + r, dtype)
    np.testing.assert_array_equal(s.float().cpu().numpy(), s_want)
    close_half(y, onp.rms_norm(s_want, w, 1e-6))


# ---- Softmax ---------------------------------------------------------------------------------------------------
def test_softmax_reference_vectors():
    for shape in ((2, 3, 2, 4), (2, 3, 2, 5, 4)):
        y = ops.softmax(torch.zeros(shape, device="cuda"), 1)
        np.testing.assert_allclose(y.cpu().numpy(), 1.0 / 3, rtol=1e-6)


def test_softmax_vs_asbuilt_where_they_coincide():
    # rows with a unique max: as-built = intended * sum(exp)  =>  intended = as-built / sum(as-built)
    x = GOLD["sm_x"][[0, 2]]
    y = ops.softmax(ops.dev(x), 2).cpu().numpy()
    ab = oracle.port_softmax_asbuilt(x, 2)
    np.testing.assert_allclose(y, ab / ab.sum(axis=2, keepdims=True), rtol=1e-5)


@pytest.mark.parametrize("shape,axis", [((32, 32000), 1), ((1, 4, 32, 32), 3), ((3, 4, 32), 1), ((2, 1000), 1),
                                        ((5, 7, 3), 0), ((2, 50001), 1)])
@pytest.mark.parametrize("dtype", [torch.float32] + HALF)
def test_softmax_seeded(shape, axis, dtype):
    rng = np.random.default_rng(sum(shape))
    x = rnd16((3 * rng.standard_normal(shape)).astype(np.float32), dtype)
    y = ops.softmax(ops.dev(x, dtype), axis)
    want = onp.softmax_intended(x, axis)
    if dtype == torch.float32:
        np.testing.assert_allclose(y.cpu().numpy(), want, rtol=2e-5, atol=1e-9)
    else:
        close_half(y, want, atol=2e-3)
        np.testing.assert_allclose(y.float().sum(dim=axis).cpu().numpy(), 1.0, atol=2e-2)


# ---- TopK (indices bit-exact) ------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,n,k", [(1, 32000, 1), (32, 32000, 50), (32, 1000, 5), (3, 64, 64), (2, 50000, 8), (4, 7, 3)])
@pytest.mark.parametrize("dtype", [torch.float32] + HALF)
def test_topk_indices_exact(rows, n, k, dtype):
    rng = np.random.default_rng(n + k)
    x = rnd16(rng.standard_normal((rows, n)).astype(np.float32), dtype)  # 16-bit rounding creates real ties
    vals, idx = ops.topk(ops.dev(x, dtype), k)
    wv, wi = onp.topk(x, k)
    np.testing.assert_array_equal(idx.cpu().numpy(), wi)
    np.testing.assert_array_equal(vals.float().cpu().numpy(), wv)


def test_topk_ties_nan_and_signed_zero():
    x = np.zeros((3, 4096), np.float32)
    x[0, :] = 1.0                      # everything tied: lowest indices win
    x[1, 100:200] = 5.0                # tie wider than k at the top
    x[1, 7] = np.nan
    x[2, ::2] = -0.0                   # +0 sorts above -0
    x[2, 5] = np.inf
    vals, idx = ops.topk(ops.dev(x), 16)
    np.testing.assert_array_equal(idx.cpu().numpy(), onp.topk(x, 16)[1])
    np.testing.assert_array_equal(idx[0].cpu().numpy(), np.arange(16))
    np.testing.assert_array_equal(idx[1].cpu().numpy(), np.arange(100, 116))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_topk_softmax_probabilities(dtype):
    rng = np.random.default_rng(9)
    x = rnd16((2 * rng.standard_normal((4, 32000))).astype(np.float32), dtype)
    p, idx = ops.topk(ops.dev(x, dtype), 5, softmax=True)
    wp, wi = onp.topk_softmax(x, 5)
    np.testing.assert_array_equal(idx.cpu().numpy(), wi)
    np.testing.assert_allclose(p.cpu().numpy(), wp, rtol=1e-4)


def test_topk_sample_matches_oracle():
    rng = np.random.default_rng(10)
    x = rnd16((2 * rng.standard_normal((32, 32000))).astype(np.float32), torch.float16)
    xd = ops.dev(x, torch.float16)
    for step in (0, 1, 63, 2 ** 33 + 5):
        tok = ops.topk_sample(xd, 50, 1.0, seed=1234, step=step).cpu().numpy()
        want = onp.topk_sample(x, 50, 1.0, 1234, step)
        assert (tok == want).mean() >= 31 / 32  # an fp32 exp rounding may move one boundary draw
        top = onp.topk(x, 50)[1]
        assert all(tok[r] in top[r] for r in range(32))
    # draws vary with the step and are reproducible
    a = ops.topk_sample(xd, 50, 1.0, 1, 7).cpu().numpy()
    b = ops.topk_sample(xd, 50, 1.0, 1, 7).cpu().numpy()
    c = ops.topk_sample(xd, 50, 1.0, 1, 8).cpu().numpy()
    np.testing.assert_array_equal(a, b)
    assert (a != c).any()


# ---- Gather / element-wise / transpose (bit-exact moves) -----------------------------------------------------------
def test_gather_reference_vectors_and_golden():
    a = np.array([1.0, 1.2, 2.3, 3.4, 4.5, 5.7], np.float32).reshape(3, 2)
    idx = np.array([0, 1, 1, 2], np.int64).reshape(2, 2)
    np.testing.assert_array_equal(ops.gather(ops.dev(a), ops.dev(idx), 0).cpu().numpy(), onp.gather(a, idx, 0))
    a = np.array([1.0, 1.2, 1.9, 2.3, 3.4, 3.9, 4.5, 5.7, 5.9], np.float32).reshape(3, 3)
    idx = np.array([0, 2], np.int32).reshape(1, 2)
    np.testing.assert_array_equal(ops.gather(ops.dev(a), ops.dev(idx), 1).cpu().numpy(), onp.gather(a, idx, 1))
    np.testing.assert_array_equal(ops.gather(ops.dev(GOLD["g_table"]), ops.dev(GOLD["g_ids"]), 0).cpu().numpy(), GOLD["g_y"])


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_gather_embedding(dtype):
    rng = np.random.default_rng(11)
    table = torch.from_numpy(rng.standard_normal((32000, 4096)).astype(np.float32)).to(dtype).cuda()
    ids = torch.from_numpy(rng.integers(-32000, 32000, (32,))).cuda()
    out = ops.gather(table, ids, 0)
    assert torch.equal(out, table[ids % 32000])
    odd = table[:, :1001].contiguous()  # row bytes not a multiple of 16
    assert torch.equal(ops.gather(odd, ids, 0), odd[ids % 32000])
    assert ops.gather(table, ids[:0], 0).shape[0] == 0  # empty index list


def test_binary_unary_where_transpose():
    a, b = GOLD["bin_a"], GOLD["bin_b"]
    np.testing.assert_array_equal(ops.binary(0, ops.dev(a), ops.dev(b)).cpu().numpy(), GOLD["bin_add"])
    np.testing.assert_array_equal(ops.binary(2, ops.dev(a), ops.dev(b)).cpu().numpy(), GOLD["bin_mul"])
    np.testing.assert_allclose(ops.unary(15, ops.dev(GOLD["un_x"])).cpu().numpy(), GOLD["un_sigmoid"], rtol=1e-6)
    rng = np.random.default_rng(12)
    x = rng.standard_normal((1 << 20,)).astype(np.float32)
    y = rng.standard_normal((1 << 20,)).astype(np.float32)
    np.testing.assert_array_equal(ops.binary(0, ops.dev(x), ops.dev(y)).cpu().numpy(), x + y)
    np.testing.assert_array_equal(ops.binary(3, ops.dev(x), ops.dev(np.float32([8.0]))).cpu().numpy(), x / 8)
    h = torch.from_numpy(x).half().cuda()
    close_half(ops.unary(100, h), onp.silu(h.float().cpu().numpy()))
    m = rng.integers(0, 2, (1, 1, 32, 32)).astype(np.bool_)
    s = rng.standard_normal((1, 4, 32, 32)).astype(np.float32)
    neg = np.float32([-1e9])
    np.testing.assert_array_equal(ops.where(ops.dev(m), ops.dev(s), ops.dev(neg)).cpu().numpy(), np.where(m, s, neg))
    t = rng.standard_normal((2, 32, 4, 64)).astype(np.float32)
    np.testing.assert_array_equal(ops.transpose(ops.dev(t), (0, 2, 1, 3)).cpu().numpy(), t.transpose(0, 2, 1, 3))
    np.testing.assert_array_equal(ops.transpose(ops.dev(t[0, 0]), (1, 0)).cpu().numpy(), t[0, 0].T)


UNARY_OPS = {0: (-3, 3), 1: (-1, 1), 2: (1, 6), 3: (-1, 1), 4: (-4, 4), 5: (-6, 6), 6: (-0.95, 0.95), 7: (-6, 6), 8: (-4, 4), 9: (-6, 6), 10: (-4, 4),
             11: (-1.4, 1.4), 12: (-4, 4), 13: (-3, 3), 14: (0, 9), 15: (-8, 8), 16: (-3, 3), 17: (-3, 3), 19: (-7, 7), 20: (-6, 6)}


@pytest.mark.parametrize("op", sorted(UNARY_OPS))
def test_unary_every_reference_operator(op):
    """Every SimpleUnaryType of the reference on fp32 (against float64 numpy at 2e-6 relative) and on fp16 (input rounded first,
    result within the half tolerance); Not on bool."""
    lo, hi = UNARY_OPS[op]
    rng = np.random.default_rng(op)
    x = rng.uniform(lo, hi, 4099).astype(np.float32)
    np.testing.assert_allclose(ops.unary(op, ops.dev(x)).cpu().numpy(), onp.unary(op, x), rtol=2e-6, atol=2e-6)
    xh = x.astype(np.float16)
    close_half(ops.unary(op, torch.from_numpy(xh).cuda()), onp.unary(op, xh.astype(np.float32)))


def test_unary_not_and_the_integer_and_bool_binary_operators():
    rng = np.random.default_rng(3)
    b1 = torch.from_numpy(rng.integers(0, 2, 1000).astype(np.bool_)).cuda()
    b2 = torch.from_numpy(rng.integers(0, 2, 1000).astype(np.bool_)).cuda()
    assert torch.equal(ops.unary(18, b1), ~b1)
    for op, fn in ((5, torch.logical_and), (6, torch.logical_or), (7, torch.logical_xor)):
        assert torch.equal(ops.binary(op, b1, b2), fn(b1, b2))
    for dt in (torch.int32, torch.int64, torch.int8, torch.uint8, torch.int16):
        lo = 0 if dt == torch.uint8 else -11
        a = torch.from_numpy(rng.integers(lo, 12, (7, 33))).to(dt).cuda()
        b = torch.from_numpy(rng.integers(1, 6, (33,))).to(dt).cuda()          # broadcast over the rows; no zero divisor
        an, bn = a.cpu().numpy(), b.cpu().numpy()
        for op in (0, 1, 2, 3, 8, 9):
            got = ops.binary(op, a, b).cpu().numpy()
            np.testing.assert_array_equal(got, onp.binary(op, an, bn).astype(an.dtype), err_msg=f"{dt} op {op}")
        small = torch.from_numpy(rng.integers(0, 4, (33,))).to(dt).cuda()
        two = torch.full((1,), 2, dtype=dt, device="cuda")
        np.testing.assert_array_equal(ops.binary(4, two, small).cpu().numpy(), (2 ** small.cpu().numpy().astype(np.int64)).astype(an.dtype))
    # float Pow and Fmod; pairs the library does not have are refused
    x = torch.from_numpy(rng.uniform(0.5, 3, 2048).astype(np.float32)).cuda()
    y = torch.from_numpy(rng.uniform(-2, 2, 2048).astype(np.float32)).cuda()
    np.testing.assert_allclose(ops.binary(4, x, y).cpu().numpy(), np.power(x.cpu().numpy().astype(np.float64), y.cpu().numpy()), rtol=3e-6)
    np.testing.assert_allclose(ops.binary(9, y, x).cpu().numpy(), np.fmod(y.cpu().numpy(), x.cpu().numpy()), rtol=1e-6, atol=1e-7)
    assert ops.binary(5, x, y, check=False)[0] == capi.ERR_UNSUPPORTED      # And on floats
    assert ops.binary(8, x, y, check=False)[0] == capi.ERR_UNSUPPORTED      # Mod on floats (Fmod is)
    assert ops.binary(0, b1, b2, check=False)[0] == capi.ERR_UNSUPPORTED    # Add on bool


# ---- RoPE ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32] + HALF)
def test_rope(dtype):
    rng = np.random.default_rng(13)
    x = rnd16(rng.standard_normal((6, 8, 128)).astype(np.float32), dtype)
    pos = np.array([0, 1, 17, 2047, 4095, 300], np.int64)
    y = ops.rope(ops.dev(x, dtype), ops.dev(pos))
    want = onp.rope(x, pos)
    # the fp32 angle pos * inv_freq carries ~pos * 1e-7 absolute error
    if dtype == torch.float32:
        np.testing.assert_allclose(y.cpu().numpy(), want, atol=3e-3, rtol=1e-4)
        np.testing.assert_allclose(y[:3].cpu().numpy(), want[:3], atol=1e-5, rtol=1e-5)
    else:
        close_half(y, want)


# ---- MatMul ------------------------------------------------------------------------------------------------------
def test_mat_mul_reference_vectors():
    a = np.array([1.0, 2.0, 0.0, 0.5], np.float32).reshape(1, 2, 2)
    b = np.array([1.0, 2.0, 0.0, 0.5], np.float32).reshape(2, 2)
    c = np.float32([1.0])
    np.testing.assert_array_equal(ops.mat_mul(ops.dev(a), ops.dev(b), ops.dev(c)).cpu().numpy().ravel(), [2, 4, 1, 1.25])
    A = (np.arange(512) % 4 - 2).astype(np.float32).reshape(1, 512)
    B = (np.arange(1000 * 512) % 4 - 2).astype(np.float32).reshape(1000, 512)
    Cb = (np.arange(1000) % 4 - 2).astype(np.float32)
    want = onp.mat_mul(A, B, Cb, trans_b=True)
    np.testing.assert_array_equal(ops.mat_mul(ops.dev(A), ops.dev(B), ops.dev(Cb), trans_b=True).cpu().numpy(), want)
    # the same integer-valued case in fp16 is exact too (|sum| <= 2048)
    got = ops.mat_mul(ops.dev(A).half(), ops.dev(B).half(), ops.dev(Cb).half(), trans_b=True)
    np.testing.assert_array_equal(got.float().cpu().numpy(), want)


def test_mat_mul_golden_and_layouts():
    a, b = GOLD["mm_a"], GOLD["mm_b"]
    np.testing.assert_allclose(ops.mat_mul(ops.dev(a), ops.dev(b)).cpu().numpy(), GOLD["mm_y"], rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(ops.mat_mul(ops.dev(a), ops.dev(b.T.copy()), trans_b=True).cpu().numpy(), GOLD["mm_y_tb"], rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(ops.mat_mul(ops.dev(a.T.copy()), ops.dev(b), trans_a=True).cpu().numpy(), GOLD["mm_y"], rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(ops.mat_mul(ops.dev(a), ops.dev(b), ops.dev(GOLD["mm_c"]), alpha=0.5, beta=2.0).cpu().numpy(),
                               GOLD["mm_y_bias"], rtol=1e-4, atol=1e-6)
    # batched with one operand broadcast (attention-score shaped)
    rng = np.random.default_rng(14)
    q = rng.standard_normal((4, 32, 64)).astype(np.float32)
    k = rng.standard_normal((4, 32, 64)).astype(np.float32)
    np.testing.assert_allclose(ops.mat_mul(ops.dev(q), ops.dev(k), trans_b=True).cpu().numpy(), onp.mat_mul(q, k, trans_b=True), rtol=1e-4, atol=1e-5)
    w = rng.standard_normal((64, 48)).astype(np.float32)
    np.testing.assert_allclose(ops.mat_mul(ops.dev(q), ops.dev(w)).cpu().numpy(), onp.mat_mul(q, w), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (1, 11008, 4096), (1, 4096, 11008), (1, 32000, 4096), (4, 4096, 4096),
                                   (2, 1000, 256), (3, 77, 4096), (1, 8192, 8192)])
@pytest.mark.parametrize("dtype", HALF)
def test_mat_mul_skinny_streaming(m, n, k, dtype):
    rng = np.random.default_rng(m + n + k)
    x = rnd16(rng.standard_normal((m, k)).astype(np.float32), dtype)
    w = rnd16((0.02 * rng.standard_normal((n, k))).astype(np.float32), dtype)
    y = ops.mat_mul(ops.dev(x, dtype), ops.dev(w, dtype), trans_b=True, force=2)
    close_half(y, onp.mat_mul(x, w, trans_b=True))
    y1 = ops.mat_mul(ops.dev(x, dtype), ops.dev(w, dtype), trans_b=True, force=1)  # the SIMT kernel agrees
    close_half(y1, onp.mat_mul(x, w, trans_b=True))


# ---- fused decode linear layer ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("m", [1, 2, 4])
def test_linear_norm_prologue_and_residual(dtype, m):
    rng = np.random.default_rng(20 + m)
    k, n = 4096, 4096
    x = rnd16(rng.standard_normal((m, k)).astype(np.float32), dtype)
    g = rnd16((1 + 0.1 * rng.standard_normal(k)).astype(np.float32), dtype)
    w = rnd16((0.02 * rng.standard_normal((n, k))).astype(np.float32), dtype)
    r = rnd16(rng.standard_normal((m, n)).astype(np.float32), dtype)
    y = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), g=ops.dev(g, dtype), eps=1e-6)
    close_half(y, onp.linear_fused(x, w, g=g, eps=1e-6))
    y = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), residual=ops.dev(r, dtype), epilogue=1)
    close_half(y, onp.linear_fused(x, w, residual=r, epilogue=1))


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("k,f", [(4096, 11008), (256, 688), (8192, 3584)])
def test_linear_silu_gate(dtype, k, f):
    rng = np.random.default_rng(k + f)
    x = rnd16(rng.standard_normal((1, k)).astype(np.float32), dtype)
    g = rnd16((1 + 0.1 * rng.standard_normal(k)).astype(np.float32), dtype)
    w = rnd16((0.02 * rng.standard_normal((2 * f, k))).astype(np.float32), dtype)
    y = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), g=ops.dev(g, dtype), epilogue=2)
    close_half(y, onp.linear_fused(x, w, g=g, epilogue=2))


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("nq,nkv,m", [(32, 32, 1), (8, 1, 2), (4, 4, 4)])
def test_linear_qkv_rope_append(dtype, paged, nq, nkv, m):
    rng = np.random.default_rng(nq * 7 + nkv + m)
    D, k = 128, 4096
    n = (nq + 2 * nkv) * D
    x = rnd16(rng.standard_normal((m, k)).astype(np.float32), dtype)
    g = rnd16((1 + 0.1 * rng.standard_normal(k)).astype(np.float32), dtype)
    w = rnd16((0.02 * rng.standard_normal((n, k))).astype(np.float32), dtype)
    pos = rng.integers(0, 200, (m,)).astype(np.int64)
    q_want, k_want, v_want = onp.linear_fused(x, w, g=g, epilogue=3, n_heads=nq, n_kv=nkv, head_dim=D, positions=pos)
    if paged:
        page, max_blocks, n_blocks = 16, 16, 64
        table = rng.permutation(n_blocks)[: m * max_blocks].reshape(m, max_blocks).astype(np.int32)
        kc = torch.zeros(n_blocks, nkv, page, D, dtype=dtype, device="cuda")
        vc = torch.zeros_like(kc)
        kv = ops.kv_layout(nkv, D, 0, page, max_blocks)
        q = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), g=ops.dev(g, dtype), epilogue=3, n_heads=nq, kv=kv,
                       positions=ops.dev(pos), table=ops.dev(table), k_cache=kc, v_cache=vc)
        k_got = torch.stack([kc[table[i, pos[i] // page], :, pos[i] % page] for i in range(m)])
        v_got = torch.stack([vc[table[i, pos[i] // page], :, pos[i] % page] for i in range(m)])
    else:
        max_seq = 256
        kc = torch.zeros(m, nkv, max_seq, D, dtype=dtype, device="cuda")
        vc = torch.zeros_like(kc)
        kv = ops.kv_layout(nkv, D, max_seq)
        q = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), g=ops.dev(g, dtype), epilogue=3, n_heads=nq, kv=kv,
                       positions=ops.dev(pos), k_cache=kc, v_cache=vc)
        k_got = torch.stack([kc[i, :, pos[i]] for i in range(m)])
        v_got = torch.stack([vc[i, :, pos[i]] for i in range(m)])
    close_half(q.reshape(m, nq, D), q_want)
    close_half(k_got, k_want)
    close_half(v_got, v_want)
    # nothing else in the caches was touched
    assert int((kc != 0).sum()) <= m * nkv * D and int((vc != 0).sum()) <= m * nkv * D


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("nq,nkv,seqs,S", [(4, 2, 2, 96), (3, 1, 1, 130), (2, 2, 3, 70), (3, 1, 2, 300), (4, 4, 1, 513)])  # 512 tokens and more: CTA pairs
def test_linear_qkv_rope_append_many_tokens(dtype, paged, nq, nkv, seqs, S):
    """More than 64 tokens (prefill): the same operator runs on the tcgen05 GEMM and splits, rotates and appends in its
    epilogue.  Token t belongs to sequence t // S; an odd head count leaves the last 256-column tile half empty."""
    rng = np.random.default_rng(nq * 7 + nkv + S)
    D, k, m = 128, 512, seqs * S
    n = (nq + 2 * nkv) * D
    x = rnd16(rng.standard_normal((m, k)).astype(np.float32), dtype)
    w = rnd16((0.05 * rng.standard_normal((n, k))).astype(np.float32), dtype)
    start = rng.integers(0, 40, (seqs,))
    pos = np.concatenate([start[b] + np.arange(S) for b in range(seqs)]).astype(np.int64)
    q_want, k_want, v_want = onp.linear_fused(x, w, epilogue=3, n_heads=nq, n_kv=nkv, head_dim=D, positions=pos)
    seq_of = np.arange(m) // S
    if paged:
        page, max_blocks = 16, max(16, (S + 40 + 15) // 16)
        n_blocks = seqs * max_blocks
        table = rng.permutation(n_blocks).reshape(seqs, max_blocks).astype(np.int32)
        kc = torch.zeros(n_blocks, nkv, page, D, dtype=dtype, device="cuda")
        vc = torch.zeros_like(kc)
        kv = ops.kv_layout(nkv, D, 0, page, max_blocks)
        q = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), epilogue=3, n_heads=nq, kv=kv, positions=ops.dev(pos), table=ops.dev(table),
                       k_cache=kc, v_cache=vc, tokens_per_seq=S)
        k_got = torch.stack([kc[table[seq_of[i], pos[i] // page], :, pos[i] % page] for i in range(m)])
        v_got = torch.stack([vc[table[seq_of[i], pos[i] // page], :, pos[i] % page] for i in range(m)])
    else:
        max_seq = max(256, S + 40)
        kc = torch.zeros(seqs, nkv, max_seq, D, dtype=dtype, device="cuda")
        vc = torch.zeros_like(kc)
        kv = ops.kv_layout(nkv, D, max_seq)
        q = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), epilogue=3, n_heads=nq, kv=kv, positions=ops.dev(pos), k_cache=kc, v_cache=vc,
                       tokens_per_seq=S)
        k_got = torch.stack([kc[seq_of[i], :, pos[i]] for i in range(m)])
        v_got = torch.stack([vc[seq_of[i], :, pos[i]] for i in range(m)])
    close_half(q.reshape(m, nq, D), q_want)
    close_half(k_got, k_want)
    close_half(v_got, v_want)
    assert int((kc != 0).sum()) <= m * nkv * D and int((vc != 0).sum()) <= m * nkv * D   # nothing else was touched
    assert capi.load().rg_b200_error_state() == 0


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("nq,nkv,m,k", [(32, 4, 16, 8200), (8, 8, 32, 520), (3, 1, 33, 1024), (24, 8, 64, 4096), (2, 2, 5, 64), (8, 8, 32, 512)])
def test_linear_qkv_rope_append_few_tokens_on_tensor_cores(dtype, paged, nq, nkv, m, k):
    """5..64 tokens, one token per sequence (a decode step).  More than 32 tokens, or a k that is not a multiple of 128, take the
    tcgen05 form: the weights sit on the M side of the instruction, a 128-row tile is one head, the k range is split over CTAs;
    the upper half of a tile hands its sums to the lower half, which rotates the pair and stores q / K / V where they belong.
    (The last case runs on the streaming skinny kernel: same contract.)"""
    rng = np.random.default_rng(nq * 7 + nkv + m + k)
    D = 128
    n = (nq + 2 * nkv) * D
    x = rnd16(rng.standard_normal((m, k)).astype(np.float32), dtype)
    w = rnd16((0.03 * rng.standard_normal((n, k))).astype(np.float32), dtype)
    pos = rng.integers(0, 100, (m,)).astype(np.int64)
    q_want, k_want, v_want = onp.linear_fused(x, w, epilogue=3, n_heads=nq, n_kv=nkv, head_dim=D, positions=pos)
    if paged:
        page, max_blocks = 16, 8
        n_blocks = m * max_blocks
        table = rng.permutation(n_blocks).reshape(m, max_blocks).astype(np.int32)
        kc = torch.zeros(n_blocks, nkv, page, D, dtype=dtype, device="cuda")
        vc = torch.zeros_like(kc)
        kv = ops.kv_layout(nkv, D, 0, page, max_blocks, n_blocks=n_blocks)
        q = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), epilogue=3, n_heads=nq, kv=kv, positions=ops.dev(pos), table=ops.dev(table),
                       k_cache=kc, v_cache=vc)
        k_got = torch.stack([kc[table[i, pos[i] // page], :, pos[i] % page] for i in range(m)])
        v_got = torch.stack([vc[table[i, pos[i] // page], :, pos[i] % page] for i in range(m)])
    else:
        max_seq = 128
        kc = torch.zeros(m, nkv, max_seq, D, dtype=dtype, device="cuda")
        vc = torch.zeros_like(kc)
        kv = ops.kv_layout(nkv, D, max_seq)
        q = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), epilogue=3, n_heads=nq, kv=kv, positions=ops.dev(pos), k_cache=kc, v_cache=vc)
        k_got = torch.stack([kc[i, :, pos[i]] for i in range(m)])
        v_got = torch.stack([vc[i, :, pos[i]] for i in range(m)])
    close_half(q.reshape(m, nq, D), q_want)
    close_half(k_got, k_want)
    close_half(v_got, v_want)
    assert int((kc != 0).sum()) <= m * nkv * D and int((vc != 0).sum()) <= m * nkv * D   # nothing else was touched
    assert capi.load().rg_b200_error_state() == 0


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("m,f,k", [(200, 256, 512), (65, 384, 64), (300, 128, 1024), (512, 256, 256), (700, 384, 1024)])  # 512 tokens and more: CTA pairs
def test_linear_silu_gate_many_tokens(dtype, m, f, k):
    """More than 64 tokens: silu(gate) * up computed in the epilogue of the tcgen05 GEMM (a B tile pairs 128 gate rows
    with their 128 up rows)."""
    rng = np.random.default_rng(m + f + k)
    x = rnd16(rng.standard_normal((m, k)).astype(np.float32), dtype)
    w = rnd16((0.05 * rng.standard_normal((2 * f, k))).astype(np.float32), dtype)
    y = ops.linear(ops.dev(x, dtype), ops.dev(w, dtype), epilogue=2)
    assert tuple(y.shape) == (m, f)
    close_half(y, onp.linear_fused(x, w, epilogue=2))
    assert capi.load().rg_b200_error_state() == 0


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("m,f,k", [(16, 3584, 8192), (5, 64, 64), (33, 448, 1024), (64, 1024, 512), (16, 11008, 4096), (32, 192, 8200)])
def test_linear_silu_gate_few_tokens_on_tensor_cores(dtype, m, f, k):
    """5..64 tokens: the weights sit on the M side of the tcgen05 instruction (a tile = 64 gate rows + their 64 up rows), the
    k range is split over CTAs; the up half of a tile hands its sums to the gate half.  Twice in a row: the arrival counters
    of the split must be back at zero."""
    rng = np.random.default_rng(m + f + k)
    x = rnd16(rng.standard_normal((m, k)).astype(np.float32), dtype)
    w = rnd16((0.03 * rng.standard_normal((2 * f, k))).astype(np.float32), dtype)
    xd, wd = ops.dev(x, dtype), ops.dev(w, dtype)
    want = onp.linear_fused(x, w, epilogue=2)
    for _ in range(2):
        y = ops.linear(xd, wd, epilogue=2)
        assert tuple(y.shape) == (m, f)
        close_half(y, want)
    assert capi.load().rg_b200_error_state() == 0


def test_linear_rejects_what_it_cannot_do():
    x = torch.zeros(33, 4096, dtype=torch.float16, device="cuda")
    w = torch.zeros(64, 4096, dtype=torch.float16, device="cuda")
    rc, _ = ops.linear(x, w, check=False)
    assert rc == capi.ERR_SHAPE  # 33..64 rows with a plain epilogue: neither streaming kernel takes them
    rc, _ = ops.linear(x[:1, :4095 * 1].contiguous()[:, :4090].contiguous(), w[:, :4090].contiguous(), check=False)
    assert rc == capi.ERR_SHAPE  # k not a multiple of 8


# ---- attention -------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32] + HALF)
@pytest.mark.parametrize("N,nH,nKV,S,D,past", [(1, 4, 4, 32, 64, 0), (2, 8, 2, 5, 128, 11), (1, 32, 32, 1, 128, 100), (1, 2, 1, 7, 32, 0)])
def test_attention_reference_layout(dtype, N, nH, nKV, S, D, past):
    rng = np.random.default_rng(N + nH + S + D + past)
    q = rnd16(rng.standard_normal((N, nH, S, D)).astype(np.float32), dtype)
    k = rnd16(rng.standard_normal((N, nKV, S, D)).astype(np.float32), dtype)
    v = rnd16(rng.standard_normal((N, nKV, S, D)).astype(np.float32), dtype)
    if past == 0:
        o = ops.attention(ops.dev(q, dtype), ops.dev(k, dtype), ops.dev(v, dtype))
        want, _, _ = onp.attention(q, k, v)
    else:
        max_seq = past + S + 3
        kc = rnd16(rng.standard_normal((N, nKV, max_seq, D)).astype(np.float32), dtype)
        vc = rnd16(rng.standard_normal((N, nKV, max_seq, D)).astype(np.float32), dtype)
        kcd, vcd = ops.dev(kc, dtype), ops.dev(vc, dtype)
        o = ops.attention(ops.dev(q, dtype), ops.dev(k, dtype), ops.dev(v, dtype), past=past, k_cache=kcd, v_cache=vcd)
        want, kc2, vc2 = onp.attention(q, k, v, past=past, k_cache=kc, v_cache=vc)
        np.testing.assert_array_equal(kcd.float().cpu().numpy(), kc2)  # append is a byte move
        np.testing.assert_array_equal(vcd.float().cpu().numpy(), vc2)
    if dtype == torch.float32:
        np.testing.assert_allclose(o.cpu().numpy(), want, rtol=1e-4, atol=1e-5)
    else:
        close_half(o, want)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("B,nH,nKV,D,lens", [
    (1, 32, 32, 128, [2049]), (1, 32, 32, 128, [1]), (3, 8, 2, 128, [64, 65, 1000]), (2, 4, 4, 64, [63, 129]),
    (4, 8, 1, 128, [512, 4096, 777, 16]),
    # enough tiles (4 x 32 heads x 64) for the tensor-path kernel with the two-stage ring; ragged lengths, one single token
    (4, 32, 32, 128, [4096, 1, 65, 1000])])
def test_attn_decode_contiguous(dtype, B, nH, nKV, D, lens):
    rng = np.random.default_rng(sum(lens) + B)
    max_seq = max(lens) + 5
    q = rnd16(rng.standard_normal((B, nH, D)).astype(np.float32), dtype)
    kc = rnd16(rng.standard_normal((B, nKV, max_seq, D)).astype(np.float32), dtype)
    vc = rnd16(rng.standard_normal((B, nKV, max_seq, D)).astype(np.float32), dtype)
    kv = ops.kv_layout(nKV, D, max_seq)
    lens_d = ops.dev(np.array(lens, np.int64))
    o, ws = ops.attn_decode(ops.dev(q, dtype), ops.dev(kc, dtype), ops.dev(vc, dtype), lens_d, kv, max(lens))
    want = onp.attn_decode(q, kc, vc, lens)
    close_half(o, want)
    # the arrival counters are left at zero, so the workspace is reusable without clearing
    o2, _ = ops.attn_decode(ops.dev(q, dtype), ops.dev(kc, dtype), ops.dev(vc, dtype), lens_d, kv, max(lens), ws=ws)
    assert torch.equal(o, o2)


@pytest.mark.parametrize("dtype", HALF)
def test_attn_decode_paged(dtype):
    rng = np.random.default_rng(33)
    B, nH, nKV, D, page = 8, 32, 32, 128, 16
    lens = rng.integers(512, 4097, (B,))
    lens[0], lens[1] = 4096, 512
    max_blocks = 4096 // page
    n_blocks = B * max_blocks
    table = rng.permutation(n_blocks).reshape(B, max_blocks).astype(np.int32)
    q = rnd16(rng.standard_normal((B, nH, D)).astype(np.float32), dtype)
    kc = torch.from_numpy(rng.standard_normal((n_blocks, nKV, page, D)).astype(np.float32)).to(dtype)
    vc = torch.from_numpy(rng.standard_normal((n_blocks, nKV, page, D)).astype(np.float32)).to(dtype)
    kv = ops.kv_layout(nKV, D, 0, page, max_blocks)
    o, _ = ops.attn_decode(ops.dev(q, dtype), kc.cuda(), vc.cuda(), ops.dev(lens.astype(np.int64)), kv, 4096, table=ops.dev(table))
    want = onp.attn_decode(q, kc.float().numpy(), vc.float().numpy(), lens, block_table=table, page=page)
    close_half(o, want)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("B,nH,nKV,lens,paged", [(16, 8, 1, "4096", False), (3, 64, 8, "mixed", False), (4, 32, 16, "mixed", True),
                                                (2, 16, 1, "mixed", True), (5, 8, 2, "short", False)])
def test_attn_decode_grouped_query(dtype, B, nH, nKV, lens, paged):
    """Grouped-query decode (2..16 query heads per KV head): the kernel that serves a whole group from one K/V tile."""
    rng = np.random.default_rng(B * nH + nKV)
    D, page = 128, 16
    L = {"4096": np.full(B, 4097), "mixed": rng.integers(1, 3000, (B,)), "short": np.array([1, 15, 16, 64, 65])[:B]}[lens].astype(np.int64)
    max_len = int(L.max())
    q = rnd16(rng.standard_normal((B, nH, D)).astype(np.float32), dtype)
    if paged:
        max_blocks = (max_len + page - 1) // page
        n_blocks = B * max_blocks
        table = rng.permutation(n_blocks).reshape(B, max_blocks).astype(np.int32)
        kc = torch.from_numpy(rng.standard_normal((n_blocks, nKV, page, D)).astype(np.float32)).to(dtype)
        vc = torch.from_numpy(rng.standard_normal((n_blocks, nKV, page, D)).astype(np.float32)).to(dtype)
        kv = ops.kv_layout(nKV, D, 0, page, max_blocks)
        o, ws = ops.attn_decode(ops.dev(q, dtype), kc.cuda(), vc.cuda(), ops.dev(L), kv, max_len, table=ops.dev(table))
        want = onp.attn_decode(q, kc.float().numpy(), vc.float().numpy(), L, block_table=table, page=page)
    else:
        max_seq = max_len + 7
        kc = torch.from_numpy(rng.standard_normal((B, nKV, max_seq, D)).astype(np.float32)).to(dtype)
        vc = torch.from_numpy(rng.standard_normal((B, nKV, max_seq, D)).astype(np.float32)).to(dtype)
        kv = ops.kv_layout(nKV, D, max_seq)
        kcd, vcd, qd, Ld = kc.cuda(), vc.cuda(), ops.dev(q, dtype), ops.dev(L)
        o, ws = ops.attn_decode(qd, kcd, vcd, Ld, kv, max_len)
        want = onp.attn_decode(q, kc.float().numpy(), vc.float().numpy(), L)
        o2, _ = ops.attn_decode(qd, kcd, vcd, Ld, kv, max_len, ws=ws)   # counters were left at zero
        assert torch.equal(o, o2)
    close_half(o, want)


def test_no_bounded_wait_expired():
    # all the kernels above ran; none of their bounded device-side waits may have expired
    torch.cuda.synchronize()
    assert capi.load().rg_b200_launch_count() > 0
    assert capi.load().rg_b200_error_state() == 0
