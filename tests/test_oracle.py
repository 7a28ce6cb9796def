"""Pins the oracle: numpy restatement and C port against (1) the literal known-answer vectors of the reference's
own kernel tests, (2) tests/golden/ref_kernels.npz, produced by the reference's unmodified CPU kernels, and
(3) those kernels directly where oracle/_ref is built.  No GPU."""
import os

import numpy as np
import pytest

import oracle
from oracle import oracle_np as onp

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_kernels.npz"))
HAVE_REF = oracle.load_ref() is not None


# ---- (1) literal vectors from the reference's tests ---------------------------------------------------------
def test_rms_norm_reference_kat():
    # src/04kernel/test/kernels/rms_normalization/test_cpu.cpp:21-38: x = 0..23 as [2,3,4], w = 1..4, eps = 0
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    w = np.arange(1, 5, dtype=np.float32)
    expect = np.empty_like(x)
    for i in range(6):
        row = x.reshape(6, 4)[i]
        rms = 1.0 / np.sqrt(np.float32((row * row).sum() / 4))
        expect.reshape(6, 4)[i] = row * rms * w
    got_np = onp.rms_norm(x, w, 0.0)
    got_c = oracle.port_rms_norm(x, w, 0.0)
    np.testing.assert_allclose(got_np, expect, rtol=4e-7)      # all six rows (row 0 = [0,1,2,3] has a non-zero mean square)
    np.testing.assert_allclose(got_c, expect, rtol=4e-7)


def test_rms_norm_cuda_test_vector():
    # src/04kernel/test/kernels/rms_normalization/test_cuda.cpp:31-51: x = 2, w = 3, D = 4096 -> y = 3
    x = np.full((2, 3, 4096), 2, np.float32)
    w = np.full(4096, 3, np.float32)
    np.testing.assert_allclose(onp.rms_norm(x, w, 0.0), 3.0, rtol=1e-6)
    np.testing.assert_allclose(oracle.port_rms_norm(x, w, 0.0), 3.0, rtol=1e-6)


def test_softmax_reference_kat():
    # src/04kernel/test/kernels/softmax/test_cpu.cpp:10-30: zeros [2,3,2,4], axis 1 -> 1/3 everywhere
    x = np.zeros((2, 3, 2, 4), np.float32)
    for f in (onp.softmax_asbuilt, onp.softmax_intended, oracle.port_softmax_asbuilt, oracle.port_softmax_intended):
        np.testing.assert_allclose(f(x, 1), 1.0 / 3, rtol=1e-6)
    # src/04kernel/test/kernels/softmax/test_cuda.cpp: zeros [2,3,2,5,4]
    x = np.zeros((2, 3, 2, 5, 4), np.float32)
    np.testing.assert_allclose(onp.softmax_intended(x, 1), 1.0 / 3, rtol=1e-6)


def test_softmax_asbuilt_divides_by_tie_count():
    # the integer accumulator makes the divisor the number of elements equal to the row max
    x = np.array([[0.0, 1.0, 2.0, 7.0, 7.0, 3.0]], np.float32)
    y = onp.softmax_asbuilt(x, 1)
    np.testing.assert_allclose(y[0, 3], 0.5)
    np.testing.assert_allclose(y, oracle.port_softmax_asbuilt(x, 1), rtol=1e-6)
    # a unique max: as built = intended * sum(exp)
    x = np.linspace(0, 7, 8, dtype=np.float32)[None]
    np.testing.assert_allclose(onp.softmax_asbuilt(x, 1), np.exp(x - 7), rtol=1e-6)


def test_mat_mul_reference_kats():
    # src/04kernel/test/kernels/mat_mul/test_cpu.cpp:24-74
    a = np.array([1.0, 2.0, 0.0, 0.5], np.float32).reshape(1, 2, 2)
    b = np.array([1.0, 2.0, 0.0, 0.5], np.float32).reshape(2, 2)
    c = np.array(1.0, np.float32)
    np.testing.assert_array_equal(onp.mat_mul(a, b, c, alpha=1, beta=1).ravel(), [2, 4, 1, 1.25])
    au = np.array([3, 2, 0, 1], np.uint16).reshape(2, 2)
    bu = np.array([1, 0, 2, 3], np.uint16).reshape(2, 2)
    np.testing.assert_array_equal(onp.mat_mul(au, bu).ravel(), [7, 6, 2, 3])
    a4 = np.array([1.0, 2.0, 0.0, 0.5, 1.0, 0.0, 0.0, 1.0], np.float32).reshape(2, 1, 2, 2)
    b4 = a4.reshape(1, 2, 2, 2)
    c4 = np.array([1.0, 0.0], np.float32).reshape(2, 1)
    expect = [2.0, 4.0, 0.0, 0.25, 2.0, 3.0, 0.0, 0.5, 2.0, 3.0, 0.0, 0.5, 2.0, 1.0, 0.0, 1.0]
    np.testing.assert_array_equal(onp.mat_mul(a4, b4, c4).ravel(), expect)
    # src/04kernel/test/kernels/mat_mul/test_cublas.cpp "Large": [1,512] x [1000,512]^T + [1000], data i%4-2
    A = (np.arange(512) % 4 - 2).astype(np.float32).reshape(1, 512)
    B = (np.arange(1000 * 512) % 4 - 2).astype(np.float32).reshape(1000, 512)
    Cb = (np.arange(1000) % 4 - 2).astype(np.float32)
    y = onp.mat_mul(A, B, Cb, trans_b=True)
    y_c = oracle.port_mat_mul(A, B, trans_b=True, beta=1.0, y=np.broadcast_to(Cb, (1, 1000)).copy())
    np.testing.assert_array_equal(y, y_c)


def test_gather_reference_kats():
    # src/04kernel/test/kernels/gather/test_gather_cpu.cpp:11-59
    a = np.array([1.0, 1.2, 2.3, 3.4, 4.5, 5.7], np.float32).reshape(3, 2)
    idx = np.array([0, 1, 1, 2], np.int64).reshape(2, 2)
    expect = [1.0, 1.2, 2.3, 3.4, 2.3, 3.4, 4.5, 5.7]
    np.testing.assert_allclose(onp.gather(a, idx, 0).ravel(), expect, rtol=1e-7)
    np.testing.assert_allclose(oracle.port_gather(a, idx, 0).ravel(), expect, rtol=1e-7)
    a = np.array([1.0, 1.2, 1.9, 2.3, 3.4, 3.9, 4.5, 5.7, 5.9], np.float32).reshape(3, 3)
    idx = np.array([0, 2], np.int32).reshape(1, 2)
    expect = [1.0, 1.9, 2.3, 3.9, 4.5, 5.9]
    np.testing.assert_allclose(onp.gather(a, idx, 1).ravel(), expect, rtol=1e-7)
    np.testing.assert_allclose(oracle.port_gather(a, idx, 1).ravel(), expect, rtol=1e-7)


# ---- (2) golden outputs of the reference's unmodified kernels -------------------------------------------------
@pytest.mark.parametrize("tag", ["rms_a", "rms_b"])
def test_rms_norm_golden(tag):
    x, w, y = GOLD[f"{tag}_x"], GOLD[f"{tag}_w"], GOLD[f"{tag}_y"]
    np.testing.assert_array_equal(oracle.port_rms_norm(x, w, 1e-6), y)  # same evaluation order: bit-exact
    np.testing.assert_allclose(onp.rms_norm(x, w, 1e-6), y, rtol=2e-6)


def test_softmax_golden():
    x = GOLD["sm_x"]
    for axis, key in ((2, "sm_y_axis2"), (1, "sm_y_axis1")):
        np.testing.assert_array_equal(oracle.port_softmax_asbuilt(x, axis), GOLD[key])
        np.testing.assert_allclose(onp.softmax_asbuilt(x, axis), GOLD[key], rtol=1e-6)
    # the tied row has divisor 2 or more; unique-max rows have divisor 1
    assert np.isfinite(GOLD["sm_y_axis2"]).all()


def test_mat_mul_golden():
    a, b = GOLD["mm_a"], GOLD["mm_b"]
    np.testing.assert_array_equal(oracle.port_mat_mul(a, b), GOLD["mm_y"])
    np.testing.assert_array_equal(oracle.port_mat_mul(a, np.ascontiguousarray(b.T), trans_b=True), GOLD["mm_y_tb"])
    np.testing.assert_allclose(onp.mat_mul(a, b), GOLD["mm_y"], rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(onp.mat_mul(a, b, GOLD["mm_c"], alpha=0.5, beta=2.0), GOLD["mm_y_bias"], rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(onp.mat_mul(GOLD["mm_a4"], GOLD["mm_b4"]), GOLD["mm_y4"], rtol=1e-4, atol=1e-5)


def test_gather_binary_unary_golden():
    np.testing.assert_array_equal(onp.gather(GOLD["g_table"], GOLD["g_ids"], 0), GOLD["g_y"])
    np.testing.assert_array_equal(oracle.port_gather(GOLD["g_table"], GOLD["g_ids"], 0), GOLD["g_y"])
    np.testing.assert_array_equal(onp.binary(0, GOLD["bin_a"], GOLD["bin_b"]), GOLD["bin_add"])
    np.testing.assert_array_equal(onp.binary(2, GOLD["bin_a"], GOLD["bin_b"]), GOLD["bin_mul"])
    np.testing.assert_allclose(onp.sigmoid(GOLD["un_x"]), GOLD["un_sigmoid"], rtol=1e-6)


# ---- (3) the reference's kernels themselves, where built ------------------------------------------------------
@pytest.mark.skipif(not HAVE_REF, reason="oracle/_ref not built (no reference checkout on this machine)")
def test_against_reference_build():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((7, 300)).astype(np.float32)
    w = rng.standard_normal(300).astype(np.float32)
    np.testing.assert_array_equal(oracle.port_rms_norm(x, w, 1e-5), oracle.ref_rms_norm(x, w, 1e-5))
    s = rng.standard_normal((4, 9, 5)).astype(np.float32)
    for ax in (0, 1, 2):
        np.testing.assert_array_equal(oracle.port_softmax_asbuilt(s, ax), oracle.ref_softmax(s, ax))
    a = rng.standard_normal((5, 33)).astype(np.float32)
    b = rng.standard_normal((33, 17)).astype(np.float32)
    np.testing.assert_array_equal(oracle.port_mat_mul(a, b), oracle.ref_mat_mul(a, b))
    np.testing.assert_array_equal(oracle.port_mat_mul(a.T.copy(), b.T.copy(), trans_a=True, trans_b=True, alpha=2.0),
                                  oracle.ref_mat_mul(a.T.copy(), b.T.copy(), trans_a=True, trans_b=True, alpha=2.0))
    t = rng.standard_normal((50, 3, 4)).astype(np.float32)
    ids = rng.integers(-50, 50, (6,)).astype(np.int32)
    np.testing.assert_array_equal(oracle.port_gather(t, ids, 0), oracle.ref_gather(t, ids, 0))


# ---- self-consistency of the unpinned definitions -------------------------------------------------------------
def test_topk_definition():
    x = np.array([[1.0, 5.0, 5.0, -0.0, 0.0, np.nan, 3.0, 5.0]], np.float32)
    v, i = onp.topk(x, 5)
    np.testing.assert_array_equal(i[0], [1, 2, 7, 6, 0])
    v2, i2 = oracle.port_topk(x, 5)
    np.testing.assert_array_equal(i2, i)
    rng = np.random.default_rng(2)
    y = rng.standard_normal((4, 1000)).astype(np.float16).astype(np.float32)  # fp16 rounding makes real ties
    np.testing.assert_array_equal(onp.topk(y, 50)[1], oracle.port_topk(y, 50)[1])


def test_attention_definition_matches_port():
    rng = np.random.default_rng(3)
    q = rng.standard_normal((2, 4, 5, 16)).astype(np.float32)
    k = rng.standard_normal((2, 2, 5, 16)).astype(np.float32)
    v = rng.standard_normal((2, 2, 5, 16)).astype(np.float32)
    kc = rng.standard_normal((2, 2, 12, 16)).astype(np.float32)
    vc = rng.standard_normal((2, 2, 12, 16)).astype(np.float32)
    o, kc2, vc2 = onp.attention(q, k, v, past=3, k_cache=kc, v_cache=vc)
    np.testing.assert_allclose(o, oracle.port_attention(q, kc2, vc2, 3), rtol=1e-5, atol=1e-6)
    # decode restatement = the general one with S = 1
    q1 = q[:, :, :1]
    o1, kc3, vc3 = onp.attention(q1, k[:, :, :1], v[:, :, :1], past=7, k_cache=kc, v_cache=vc)
    od = onp.attn_decode(q1[:, :, 0], kc3, vc3, np.array([8, 8]))
    np.testing.assert_allclose(od, o1[:, :, 0], rtol=1e-5, atol=1e-6)


def test_rope_definition():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, 2, 8)).astype(np.float32)
    pos = np.array([0, 1, 4095], np.int64)
    y = onp.rope(x, pos)
    np.testing.assert_allclose(y[0], x[0], rtol=1e-6)  # position 0 is the identity
    np.testing.assert_allclose((y ** 2).sum(-1), (x ** 2).sum(-1), rtol=1e-5)  # rotations preserve the norm
    np.testing.assert_allclose(y, oracle.port_rope(x, pos), rtol=1e-5, atol=1e-6)


def test_philox_known_answer():
    # Random123 known-answer vectors for philox4x32-10 (kat_vectors): zero counter/key and all-ones counter/key
    assert onp.philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert onp.philox4x32_10([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
