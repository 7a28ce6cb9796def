"""TEST INFRASTRUCTURE ONLY — loaders for the two compiled oracles.

  load_port(): oracle/librg_oracle.so, the plain-C restatement (oracle_port.c); built on demand with gcc.
  load_ref():  oracle/_ref/librg_ref.so, the reference's own unmodified CPU kernels behind ref_capi.cpp; present
               only where it was built from a reference checkout (make -C oracle ref); None otherwise.
Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_port = None
_ref = None


def load_port() -> C.CDLL:
    global _port
    if _port is None:
        path = os.path.join(_HERE, "librg_oracle.so")
        src = os.path.join(_HERE, "oracle_port.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            subprocess.run(["gcc", "-O2", "-fPIC", "-shared", "-std=c11", "-ffp-contract=off", "-o", path, src, "-lm"],
                           check=True)
        _port = C.CDLL(path)
    return _port


def load_ref():
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "librg_ref.so")
        if not os.path.exists(path):
            return None
        _ref = C.CDLL(path)
    return _ref


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _shape(a):
    return (C.c_uint32 * max(1, len(a)))(*a)


_CODE = {np.dtype(np.float32): 1, np.dtype(np.float64): 11, np.dtype(np.int32): 6, np.dtype(np.int64): 7,
         np.dtype(np.uint16): 4}


# ---- the reference's own kernels (None-safe callers check load_ref() first) ---------------------------------
def ref_rms_norm(x, w, eps):
    x = np.ascontiguousarray(x); w = np.ascontiguousarray(w); y = np.empty_like(x)
    rc = load_ref().rg_ref_rms_norm(_CODE[x.dtype], _p(x), _p(w), _p(y), _shape(x.shape), x.ndim, C.c_float(eps))
    assert rc == 0
    return y


def ref_softmax(x, axis):
    x = np.ascontiguousarray(x); y = np.empty_like(x)
    rc = load_ref().rg_ref_softmax(_CODE[x.dtype], _p(x), _p(y), _shape(x.shape), x.ndim, axis)
    assert rc == 0
    return y


def ref_mat_mul(a, b, c=None, trans_a=False, trans_b=False, alpha=1.0, beta=1.0):
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    m = a.shape[-1] if trans_a else a.shape[-2]
    n = b.shape[-2] if trans_b else b.shape[-1]
    batch = np.broadcast_shapes(a.shape[:-2], b.shape[:-2])
    y = np.zeros(batch + (m, n), a.dtype)
    cc = np.ascontiguousarray(c) if c is not None else None
    rc = load_ref().rg_ref_mat_mul(_CODE[a.dtype], _p(a), _shape(a.shape), a.ndim, _p(b), _shape(b.shape), b.ndim,
                                   _p(cc) if cc is not None else None,
                                   _shape(cc.shape) if cc is not None else None, cc.ndim if cc is not None else 0,
                                   _p(y), int(trans_a), int(trans_b), C.c_float(alpha), C.c_float(beta))
    assert rc == 0
    return y


def ref_gather(data, idx, axis):
    data = np.ascontiguousarray(data); idx = np.ascontiguousarray(idx)
    out = np.empty(data.shape[:axis] + idx.shape + data.shape[axis + 1:], data.dtype)
    rc = load_ref().rg_ref_gather(_CODE[data.dtype], _p(data), _shape(data.shape), data.ndim, _CODE[idx.dtype],
                                  _p(idx), _shape(idx.shape), idx.ndim, _p(out), axis)
    assert rc == 0
    return out


def ref_binary(op, a, b):
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    y = np.empty(np.broadcast_shapes(a.shape, b.shape), a.dtype)
    rc = load_ref().rg_ref_binary(op, _CODE[a.dtype], _p(a), _shape(a.shape), a.ndim, _p(b), _shape(b.shape), b.ndim, _p(y))
    assert rc == 0
    return y


def ref_unary(op, x):
    x = np.ascontiguousarray(x); y = np.empty_like(x)
    rc = load_ref().rg_ref_unary(op, _CODE[x.dtype], _p(x), _p(y), _shape(x.shape), x.ndim)
    assert rc == 0
    return y


# ---- the C port ----------------------------------------------------------------------------------------------
def port_rms_norm(x, w, eps):
    x = np.ascontiguousarray(x, np.float32); w = np.ascontiguousarray(w, np.float32); y = np.empty_like(x)
    load_port().oracle_rms_norm_f32(_p(x), _p(w), _p(y), C.c_size_t(x.size // x.shape[-1]), C.c_size_t(x.shape[-1]), C.c_float(eps))
    return y


def _pmp(x, axis):
    pre = int(np.prod(x.shape[:axis], dtype=np.int64)); mid = x.shape[axis]
    post = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    return C.c_size_t(pre), C.c_size_t(mid), C.c_size_t(post)


def port_softmax_asbuilt(x, axis):
    x = np.ascontiguousarray(x, np.float32); y = np.empty_like(x)
    load_port().oracle_softmax_asbuilt_f32(_p(x), _p(y), *_pmp(x, axis % x.ndim))
    return y


def port_softmax_intended(x, axis):
    x = np.ascontiguousarray(x, np.float32); y = np.empty_like(x)
    load_port().oracle_softmax_intended_f32(_p(x), _p(y), *_pmp(x, axis % x.ndim))
    return y


def port_mat_mul(a, b, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, y=None):
    """2-D product; y (pre-filled with the broadcast bias when beta != 0) is updated in place."""
    a = np.ascontiguousarray(a, np.float32); b = np.ascontiguousarray(b, np.float32)
    m, k = (a.shape[1], a.shape[0]) if trans_a else a.shape
    n = b.shape[0] if trans_b else b.shape[1]
    if y is None:
        y = np.zeros((m, n), np.float32)
    load_port().oracle_mat_mul_f32(_p(a), _p(b), _p(y), C.c_size_t(m), C.c_size_t(k), C.c_size_t(n), int(trans_a),
                                   int(trans_b), C.c_float(alpha), C.c_float(beta))
    return y


def port_gather(data, idx, axis):
    data = np.ascontiguousarray(data); idx = np.ascontiguousarray(idx)
    out = np.empty(data.shape[:axis] + idx.shape + data.shape[axis + 1:], data.dtype)
    prefix = int(np.prod(data.shape[:axis], dtype=np.int64))
    postfix = int(np.prod(data.shape[axis + 1:], dtype=np.int64)) * data.dtype.itemsize
    load_port().oracle_gather(_p(data), _p(idx), int(idx.dtype == np.int64), _p(out), C.c_size_t(prefix),
                              C.c_size_t(data.shape[axis]), C.c_size_t(idx.size), C.c_size_t(postfix))
    return out


def port_rope(x, pos, theta=10000.0):
    x = np.ascontiguousarray(x, np.float32); pos = np.ascontiguousarray(pos, np.int64); y = np.empty_like(x)
    load_port().oracle_rope_f32(_p(x), _p(pos), _p(y), C.c_size_t(x.shape[0]), C.c_size_t(x.shape[1]),
                                C.c_size_t(x.shape[2]), C.c_float(theta))
    return y


def port_attention(q, K, V, past):
    """q[N,nH,S,D]; K,V[N,nKV,kv_tokens,D] with the new keys already at [past, past+S)."""
    q = np.ascontiguousarray(q, np.float32); K = np.ascontiguousarray(K, np.float32); V = np.ascontiguousarray(V, np.float32)
    o = np.empty_like(q)
    N, nH, S, D = q.shape
    load_port().oracle_attention_f32(_p(q), _p(K), _p(V), _p(o), C.c_size_t(N), C.c_size_t(nH), C.c_size_t(K.shape[1]),
                                     C.c_size_t(S), C.c_size_t(D), C.c_size_t(K.shape[2]), C.c_size_t(past))
    return o


def port_topk(x, k):
    x = np.ascontiguousarray(x, np.float32)
    vals = np.empty(x.shape[:-1] + (k,), np.float32); idx = np.empty(x.shape[:-1] + (k,), np.int64)
    load_port().oracle_topk_f32(_p(x), _p(vals), _p(idx), C.c_size_t(x.size // x.shape[-1]), C.c_size_t(x.shape[-1]), C.c_size_t(k))
    return vals, idx
