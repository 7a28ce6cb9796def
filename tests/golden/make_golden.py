"""Generates tests/golden/ref_kernels.npz from the reference's own CPU kernels (oracle/_ref/librg_ref.so, built
from an unmodified reference checkout by `make -C oracle ref`).  Run here once; the .npz travels with the repo so
the oracle can be pinned on machines that have no reference checkout.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402


def main():
    assert oracle.load_ref() is not None, "build oracle/_ref first: make -C oracle ref"
    rng = np.random.default_rng(0)
    out = {}
    # RMSNorm: seeded rows at the tiny-decoder width and an odd width
    for tag, shape in (("rms_a", (2, 8, 256)), ("rms_b", (5, 77))):
        x = rng.standard_normal(shape).astype(np.float32)
        w = (1 + 0.1 * rng.standard_normal(shape[-1])).astype(np.float32)
        out[f"{tag}_x"], out[f"{tag}_w"] = x, w
        out[f"{tag}_y"] = oracle.ref_rms_norm(x, w, 1e-6)
    # Softmax as built (integer-truncated sum): random rows, rows with ties at the max, last and middle axis
    x = rng.standard_normal((3, 4, 32)).astype(np.float32)
    x[1, :, 5] = x[1].max(axis=-1)  # a tie at the row max
    out["sm_x"] = x
    out["sm_y_axis2"] = oracle.ref_softmax(x, 2)
    out["sm_y_axis1"] = oracle.ref_softmax(x, 1)
    # MatMul: the tiny-decoder projections, transB, alpha/beta with broadcast bias, batch broadcast
    a = rng.standard_normal((8, 256)).astype(np.float32)
    b = (0.02 * rng.standard_normal((256, 96))).astype(np.float32)
    out["mm_a"], out["mm_b"] = a, b
    out["mm_y"] = oracle.ref_mat_mul(a, b)
    bt = np.ascontiguousarray(b.T)
    out["mm_y_tb"] = oracle.ref_mat_mul(a, bt, trans_b=True)
    c = rng.standard_normal((96,)).astype(np.float32)
    out["mm_c"] = c
    out["mm_y_bias"] = oracle.ref_mat_mul(a, b, c, alpha=0.5, beta=2.0)
    a4 = rng.standard_normal((2, 1, 8, 16)).astype(np.float32)
    b4 = rng.standard_normal((1, 3, 16, 8)).astype(np.float32)
    out["mm_a4"], out["mm_b4"] = a4, b4
    out["mm_y4"] = oracle.ref_mat_mul(a4, b4)
    # Gather: embedding rows with negative indices
    table = rng.standard_normal((100, 16)).astype(np.float32)
    ids = rng.integers(-100, 100, size=(2, 7)).astype(np.int64)
    out["g_table"], out["g_ids"] = table, ids
    out["g_y"] = oracle.ref_gather(table, ids, 0)
    # Element-wise: Add / Mul with broadcast, Sigmoid
    p = rng.standard_normal((4, 1, 8)).astype(np.float32)
    q = rng.standard_normal((3, 8)).astype(np.float32)
    out["bin_a"], out["bin_b"] = p, q
    out["bin_add"] = oracle.ref_binary(0, p, q)
    out["bin_mul"] = oracle.ref_binary(2, p, q)
    s = (4 * rng.standard_normal((5, 33))).astype(np.float32)
    out["un_x"] = s
    out["un_sigmoid"] = oracle.ref_unary(15, s)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_kernels.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
