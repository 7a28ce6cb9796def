"""TEST INFRASTRUCTURE ONLY — CPU restatement (numpy) of the reference's decoder kernel path.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may import this
module; the product path (refactorgraph_b200/) never does.

Pinned parts (checked against the reference's own test vectors in tests/test_oracle.py and, where
oracle/_ref/librg_ref.so is built, against the reference's unmodified CPU kernels):
  rms_norm, softmax_asbuilt, mat_mul, gather, binary, unary.
PARITY UNPINNED (the reference has no implementation, vector or test; definitions are written here):
  softmax_intended on non-constant rows, attention, rope, topk, topk_sample, paged KV.

File:line citations are relative to the reference repository root.
"""
from __future__ import annotations

import numpy as np

# ------------------------------------------------------------------------------------------------
# RmsNormalizationCpu — src/04kernel/src/kernels/rms_normalization/cpu_kernel.cc:41-66
#   ss = sum(x*x) (sequential, in T); ss /= D; ss += eps; ss = 1/sqrt(ss); y = x*ss*w
def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    xf = x.astype(np.float64)
    ss = (xf * xf).sum(axis=-1, keepdims=True) / x.shape[-1] + eps
    return (xf * (1.0 / np.sqrt(ss)) * w.astype(np.float64)).astype(np.float32 if x.dtype != np.float64 else np.float64)


# SoftmaxCpu as built — src/04kernel/src/kernels/softmax/cpu_kernel.cc:27-57.
# std::accumulate is seeded with the int literal 0, so the running sum is truncated to an integer after
# every addition (:46-51); the divisor is that integer.
def softmax_asbuilt(x: np.ndarray, axis: int) -> np.ndarray:
    xm = np.moveaxis(x, axis, -1)
    e = np.exp(xm - xm.max(axis=-1, keepdims=True))
    acc = np.zeros(e.shape[:-1], dtype=np.int64)
    for j in range(e.shape[-1]):
        acc = np.trunc(acc.astype(e.dtype) + e[..., j]).astype(np.int64)
    with np.errstate(divide="ignore", invalid="ignore"):
        y = e / acc[..., None].astype(e.dtype)
    return np.moveaxis(y, -1, axis)


# Softmax as the reference's CUDA / cuDNN kernels compute it
# (src/04kernel/src/kernels/softmax/cuda_kernel.cu:29-56) = the CPU kernel with the accumulator seeded T(0).
def softmax_intended(x: np.ndarray, axis: int) -> np.ndarray:
    xf = x.astype(np.float64)
    e = np.exp(xf - xf.max(axis=axis, keepdims=True))
    return (e / e.sum(axis=axis, keepdims=True)).astype(x.dtype if x.dtype in (np.float32, np.float64) else np.float32)


# MatMulCPU — src/04kernel/src/kernels/mat_mul/cpu_kernel.cc:28-91, inner loop
# src/04kernel/src/kernels/mat_mul_common/cpu_template.hpp:18-30:  Y = alpha * op(A) @ op(B) + beta * C,
# leading dims multidirectionally broadcast (Broadcaster, src/04kernel/src/attributes/broadcaster.cc:17-105),
# C broadcast to the output shape first (mat_mul_info.cc:5-25).
def mat_mul(a, b, c=None, trans_a=False, trans_b=False, alpha=1.0, beta=1.0):
    A = np.swapaxes(a, -1, -2) if trans_a else a
    B = np.swapaxes(b, -1, -2) if trans_b else b
    acc_t = np.float64 if a.dtype.kind == "f" else a.dtype
    y = np.matmul(A.astype(acc_t), B.astype(acc_t))
    if a.dtype.kind == "f":
        y = alpha * y
        if c is not None:
            y = y + beta * np.broadcast_to(c.astype(acc_t), y.shape)
        return y.astype(a.dtype if a.dtype in (np.float32, np.float64) else np.float32)
    y = (np.asarray(alpha, a.dtype) * y).astype(a.dtype)
    if c is not None:
        y = (y + np.asarray(beta, a.dtype) * np.broadcast_to(c, y.shape)).astype(a.dtype)
    return y


# GatherCpu — src/04kernel/src/kernels/gather/cpu_kernel.cc:24-42: out[p, i, :] = data[p, idx[i], :],
# negative idx counts from the end.
def gather(data: np.ndarray, indices: np.ndarray, axis: int) -> np.ndarray:
    return np.take(data, indices.astype(np.int64), axis=axis)


# BinaryCpu — src/04kernel/src/kernels/simple_binary/cpu_kernel.cc:33-154 (Add 0, Sub 1, Mul 2, Div 3).
def binary(op: int, a, b):
    """SimpleBinaryType 0-9 as BinaryCpu computes them (src/04kernel/src/kernels/simple_binary/cpu_kernel.cc:88-150): integer Div and
    Mod / Fmod are the C++ `/` and `%` (truncation toward zero, sign of the dividend); And / Or / Xor are for bool."""
    a, b = np.asarray(a), np.asarray(b)
    if op in (0, 1, 2):
        with np.errstate(over="ignore"):
            return {0: np.add, 1: np.subtract, 2: np.multiply}[op](a, b)
    if op == 3:
        return np.trunc(np.true_divide(a, b)).astype(a.dtype) if np.issubdtype(a.dtype, np.integer) else np.divide(a, b)
    if op == 4:
        return np.power(a.astype(np.float64), b.astype(np.float64)).astype(a.dtype) if np.issubdtype(a.dtype, np.integer) else np.power(a, b)
    if op in (5, 6, 7):
        return {5: np.logical_and, 6: np.logical_or, 7: np.logical_xor}[op](a, b)
    return np.fmod(a, b)      # 8 Mod (integers), 9 Fmod: both follow the sign of the dividend


UNARY = {0: np.abs, 1: np.arccos, 2: np.arccosh, 3: np.arcsin, 4: np.arcsinh, 5: np.arctan, 6: np.arctanh, 7: np.cos, 8: np.cosh, 9: np.sin,
         10: np.sinh, 11: np.tan, 12: np.tanh, 13: lambda x: np.maximum(x, 0), 14: np.sqrt, 15: lambda x: 1 / (1 + np.exp(-x)), 17: np.negative,
         18: np.logical_not, 20: np.exp}


def unary(op: int, x):
    """SimpleUnaryType values (src/04kernel/include/kernel/collectors/simple_unary.h:8-30) in float64; Erf (16) and HardSwish (19,
    x * clamp(x / 6 + 0.5, 0, 1): hardswishFun, src/04kernel/src/kernels/simple_unary/cpu_kernel.cc:54-59) spelled out."""
    if op == 18:
        return np.logical_not(x)
    xf = np.asarray(x, np.float64)
    if op == 16:
        import math
        return np.vectorize(math.erf)(xf)
    if op == 19:
        return xf * np.clip(xf / 6 + 0.5, 0, 1)
    return UNARY[op](xf)


# SimpleUnaryCpu — src/04kernel/src/kernels/simple_unary/cpu_kernel.cc:42-45 (sigmoid = 1/(1+exp(-x))).
def sigmoid(x):
    xf = x.astype(np.float64)
    return (1.0 / (1.0 + np.exp(-xf))).astype(x.dtype if x.dtype in (np.float32, np.float64) else np.float32)


def silu(x):
    xf = x.astype(np.float64)
    return (xf / (1.0 + np.exp(-xf))).astype(np.float32)


# ------------------------------------------------------------------------------------------------
# Definitions with no reference implementation (parity unpinned).

# ---- data movement: the reference's CPU kernels are block copies driven by ConcatInfo / SplitInfo / SliceInfo / ExpandInfo
# (src/04kernel/src/kernels/{concat,split,slice,expand}/cpu_kernel.cc), i.e. exactly numpy's concatenate / split / strided
# indexing / broadcast_to; Cast is `static_cast<U>(a)` per element (src/04kernel/src/kernels/cast/cpu_kernel.cc:36).
def concat(xs, axis: int) -> np.ndarray:
    return np.concatenate(xs, axis=axis)


def split(x: np.ndarray, sizes, axis: int):
    return np.split(x, np.cumsum(sizes)[:-1], axis=axis)


def slice_(x: np.ndarray, starts, steps, lengths) -> np.ndarray:
    """y[i0, i1, ..] = x[start0 + i0 * step0, ..] — the {start, step, length} triples of
    src/04kernel/include/kernel/attributes/slice_info.h:8-13."""
    idx = tuple(np.asarray(s + st * np.arange(n), np.int64) for s, st, n in zip(starts, steps, lengths))
    return x[np.ix_(*idx)] if idx else x.copy()


def expand(x: np.ndarray, shape) -> np.ndarray:
    return np.ascontiguousarray(np.broadcast_to(x, shape))


def cast(x: np.ndarray, to) -> np.ndarray:
    """static_cast semantics: float -> integer truncates toward zero, anything -> bool is `!= 0`; float -> half rounds to
    nearest even (what the reference's CUDA cast computes; its host fp16_t truncates)."""
    with np.errstate(invalid="ignore", over="ignore"):
        return x.astype(to)


def rope(x: np.ndarray, positions: np.ndarray, theta: float = 10000.0) -> np.ndarray:
    """x[tokens, heads, D]; rotate-half pairing (i, i + D/2); angle = pos * theta^(-2i/D)."""
    T, H, D = x.shape
    half = D // 2
    i = np.arange(half, dtype=np.float64)
    inv_freq = theta ** (-2.0 * i / D)
    ang = positions.astype(np.float64)[:, None] * inv_freq[None, :]
    cs, sn = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    xf = x.astype(np.float64)
    lo, hi = xf[..., :half], xf[..., half:]
    return np.concatenate([lo * cs - hi * sn, hi * cs + lo * sn], axis=-1).astype(np.float32)


def order_key(x: np.ndarray) -> np.ndarray:
    """Order-preserving uint32 key of a float32 array: -0 < +0, NaN below everything."""
    f = np.ascontiguousarray(x, dtype=np.float32)
    b = f.view(np.uint32)
    k = np.where(b & np.uint32(0x80000000), ~b, b | np.uint32(0x80000000)).astype(np.uint32)
    return np.where(np.isnan(f), np.uint32(0), k)


def topk(x: np.ndarray, k: int):
    """Per row: k largest, descending, ties by lower index.  Returns (values, int64 indices)."""
    key = order_key(x.astype(np.float32)).astype(np.int64)
    # stable sort on the negated key keeps equal keys in index order = ties by lower index
    idx = np.argsort(-key, axis=-1, kind="stable")[..., :k]
    return np.take_along_axis(x, idx, axis=-1), idx.astype(np.int64)


def topk_softmax(x: np.ndarray, k: int):
    vals, idx = topk(x, k)
    p = softmax_intended(x.astype(np.float32), -1)
    return np.take_along_axis(p, idx, axis=-1).astype(np.float32), idx


def philox4x32_10(counter, key):
    """Philox-4x32-10 (Salmon et al., SC'11).  counter: 4 uint32, key: 2 uint32 -> 4 uint32."""
    c = [int(v) & 0xFFFFFFFF for v in counter]
    k0, k1 = int(key[0]) & 0xFFFFFFFF, int(key[1]) & 0xFFFFFFFF
    for _ in range(10):
        p0 = 0xD2511F53 * c[0]
        p1 = 0xCD9E8D57 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k1) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return c


def topk_sample(x: np.ndarray, k: int, temperature: float, seed: int, step: int) -> np.ndarray:
    """One token per row from softmax(x/T) restricted to the top-k set; u from Philox keyed (seed, step, row)."""
    vals, idx = topk(x.astype(np.float32), k)
    out = np.zeros(x.shape[0], dtype=np.int64)
    inv_t = np.float32(1.0 / temperature)
    for r in range(x.shape[0]):
        rnd = philox4x32_10([r, 0, step & 0xFFFFFFFF, step >> 32], [seed & 0xFFFFFFFF, seed >> 32])[0]
        u = np.float32(rnd >> 8) * np.float32(1.0 / 16777216.0)
        w = np.exp((vals[r].astype(np.float32) - vals[r, 0].astype(np.float32)) * inv_t).astype(np.float32)
        total = np.float32(0)
        for j in range(k):
            total = np.float32(total + w[j])
        target = np.float32(u * total)
        cum, pick = np.float32(0), k - 1
        for j in range(k):
            cum = np.float32(cum + w[j])
            if cum > target:
                pick = j
                break
        out[r] = idx[r, pick]
    return out


def attention(q, k, v, past: int = 0, k_cache=None, v_cache=None):
    """Causal multi-head attention with optional KV cache — operator spec src/08-01llm/README.md:29-63, shape
    rules src/08-01llm/src/operators/attention.cc:37-128.  q[N,nH,S,D], k/v[N,nKV,S,D], caches [N,nKV,maxSeq,D].
    Query row i (absolute position past+i) sees keys j <= past+i; q head h uses kv head h // (nH // nKV);
    scores scaled by 1/sqrt(D).  Returns (out, k_cache, v_cache) with the new k/v written at [past, past+S)."""
    N, nH, S, D = q.shape
    nKV = k.shape[1]
    if k_cache is not None:
        k_cache = k_cache.copy()
        v_cache = v_cache.copy()
        k_cache[:, :, past:past + S] = k
        v_cache[:, :, past:past + S] = v
        K, V = k_cache[:, :, :past + S], v_cache[:, :, :past + S]
    else:
        assert past == 0
        K, V = k, v
    rep = nH // nKV
    Kf = np.repeat(K.astype(np.float64), rep, axis=1)
    Vf = np.repeat(V.astype(np.float64), rep, axis=1)
    s = np.einsum("nhid,nhjd->nhij", q.astype(np.float64), Kf) / np.sqrt(D)
    L = past + S
    mask = np.arange(L)[None, :] <= (past + np.arange(S))[:, None]
    s = np.where(mask[None, None], s, -np.inf)
    p = np.exp(s - s.max(axis=-1, keepdims=True))
    p /= p.sum(axis=-1, keepdims=True)
    out = np.einsum("nhij,nhjd->nhid", p, Vf).astype(np.float32)
    return out, k_cache, v_cache


def attn_decode(q, k_cache, v_cache, lens, block_table=None, page: int = 16):
    """One new token per sequence.  q[B,nH,D]; contiguous caches [B,nKV,maxSeq,D] or paged
    [blocks,nKV,page,D] with block_table[B,maxBlocks]; keys [0,len) attended."""
    B, nH, D = q.shape
    out = np.zeros((B, nH, D), np.float32)
    for b in range(B):
        L = int(lens[b])
        if L == 0:
            continue
        if block_table is None:
            K, V = k_cache[b, :, :L], v_cache[b, :, :L]
        else:
            nb = (L + page - 1) // page
            blocks = block_table[b, :nb]
            K = np.concatenate([k_cache[blk] for blk in blocks], axis=1)[:, :L]
            V = np.concatenate([v_cache[blk] for blk in blocks], axis=1)[:, :L]
        nKV = K.shape[0]
        rep = nH // nKV
        Kf = np.repeat(K.astype(np.float64), rep, axis=0)
        Vf = np.repeat(V.astype(np.float64), rep, axis=0)
        s = np.einsum("hd,hjd->hj", q[b].astype(np.float64), Kf) / np.sqrt(D)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        p /= p.sum(axis=-1, keepdims=True)
        out[b] = np.einsum("hj,hjd->hd", p, Vf)
    return out


def linear_fused(x, w, g=None, eps=1e-6, residual=None, epilogue=0, n_heads=0, n_kv=0, head_dim=0,
                 positions=None, theta=10000.0):
    """Y = epilogue(prologue(X) W^T): RMSNorm prologue when g is given; epilogue 0 none, 1 residual add,
    2 SiLU(gate)*up with W = [gate; up], 3 QKV split + RoPE (returns q, k, v as [m, heads, D])."""
    xf = x.astype(np.float64)
    if g is not None:
        xf = rms_norm(xf, g.astype(np.float64), eps).astype(np.float64)
    y = xf @ w.astype(np.float64).T
    if epilogue == 0:
        return y.astype(np.float32)
    if epilogue == 1:
        return (y + residual.astype(np.float64)).astype(np.float32)
    if epilogue == 2:
        f = y.shape[-1] // 2
        gt, up = y[..., :f], y[..., f:]
        return (gt / (1.0 + np.exp(-gt)) * up).astype(np.float32)
    m = y.shape[0]
    q = y[:, : n_heads * head_dim].reshape(m, n_heads, head_dim)
    k = y[:, n_heads * head_dim: (n_heads + n_kv) * head_dim].reshape(m, n_kv, head_dim)
    v = y[:, (n_heads + n_kv) * head_dim:].reshape(m, n_kv, head_dim)
    return rope(q, positions, theta), rope(k, positions, theta), v.astype(np.float32)
