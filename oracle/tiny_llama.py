"""TEST INFRASTRUCTURE ONLY — the tiny Llama-style decoder of the CPU-runnable configuration (2 layers, hidden 256,
4 heads x 64, FFN 688 SiLU-gated, vocab 1000, fp32, batch-1 prefill of 32 tokens), composed operator by operator
from the reference's own CPU kernels (oracle/_ref) or from the C port, in the order a reference graph would run
them: Gather, RmsNormalization, MatMul, Transpose, MatMul, Div, Where, Softmax, MatMul, Transpose, MatMul, Add,
RmsNormalization, MatMul x2, Sigmoid, Mul, Mul, MatMul, Add, ..., RmsNormalization, MatMul.  Reshape / Transpose /
Where are byte moves and are done with numpy.

softmax = "asbuilt" uses the reference SoftmaxCpu exactly as it is (integer-truncated row sum,
src/04kernel/src/kernels/softmax/cpu_kernel.cc:46-51); softmax = "intended" seeds that accumulator with T(0),
which is what the reference's CUDA/cuDNN kernels compute and what the B200 kernels are compared with.
"""
from __future__ import annotations

import numpy as np

import oracle


def prefill(cfg, weights: dict, ids: np.ndarray, softmax: str = "intended", kernels: str = "ref"):
    use_ref = kernels == "ref" and oracle.load_ref() is not None
    rms = (lambda x, w: oracle.ref_rms_norm(x, w, cfg.eps)) if use_ref else (lambda x, w: oracle.port_rms_norm(x, w, cfg.eps))

    def mm(a, b):
        if use_ref:
            return oracle.ref_mat_mul(a, b)
        lead = np.broadcast_shapes(a.shape[:-2], b.shape[:-2])
        A = np.broadcast_to(a, lead + a.shape[-2:]).reshape((-1,) + a.shape[-2:])
        B = np.broadcast_to(b, lead + b.shape[-2:]).reshape((-1,) + b.shape[-2:])
        return np.stack([oracle.port_mat_mul(A[i], B[i]) for i in range(A.shape[0])]).reshape(lead + (a.shape[-2], b.shape[-1]))

    add = (lambda a, b: oracle.ref_binary(0, a, b)) if use_ref else np.add
    mul = (lambda a, b: oracle.ref_binary(2, a, b)) if use_ref else np.multiply
    div = (lambda a, b: oracle.ref_binary(3, a, b)) if use_ref else np.divide
    sig = (lambda x: oracle.ref_unary(15, x)) if use_ref else (lambda x: (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(np.float32))
    gather = (lambda t, i: oracle.ref_gather(t, i, 0)) if use_ref else (lambda t, i: oracle.port_gather(t, i, 0))
    if softmax == "asbuilt":
        sm = (lambda x: oracle.ref_softmax(x, 3)) if use_ref else (lambda x: oracle.port_softmax_asbuilt(x, 3))
    else:
        sm = lambda x: oracle.port_softmax_intended(x, 3)

    S = ids.shape[-1]
    H, D, nH, F = cfg.hidden, cfg.head_dim, cfg.heads, cfg.ffn
    mask = np.tril(np.ones((S, S), np.bool_))[None, None]
    neg, scale = np.float32([-3.0e38]), np.float32([np.sqrt(D)])
    x = gather(weights["embed"], ids.reshape(1, S))                        # [1, S, H]
    for l in range(cfg.layers):
        wqkv, wgu = weights[f"l{l}.wqkv"], weights[f"l{l}.wgu"]
        wq, wk, wv = wqkv[: nH * D], wqkv[nH * D: 2 * nH * D], wqkv[2 * nH * D:]
        n1 = rms(x, weights[f"l{l}.norm1"])
        q, k, v = (np.ascontiguousarray(mm(n1, np.ascontiguousarray(w.T)).reshape(1, S, nH, D).transpose(0, 2, 1, 3)) for w in (wq, wk, wv))
        s = mm(q, np.ascontiguousarray(k.transpose(0, 1, 3, 2)))
        s = div(s, scale)
        s = np.where(mask, s, neg).astype(np.float32)
        p = sm(np.ascontiguousarray(s))
        a = np.ascontiguousarray(mm(p, v).transpose(0, 2, 1, 3)).reshape(1, S, nH * D)
        x = add(x, mm(a, np.ascontiguousarray(weights[f"l{l}.wo"].T)))
        n2 = rms(x, weights[f"l{l}.norm2"])
        gt = mm(n2, np.ascontiguousarray(wgu[:F].T))
        up = mm(n2, np.ascontiguousarray(wgu[F:].T))
        act = mul(mul(gt, sig(gt)), up)
        x = add(x, mm(act, np.ascontiguousarray(weights[f"l{l}.wd"].T)))
    xf = rms(x, weights["norm_f"])
    logits = mm(xf, np.ascontiguousarray(weights["lm_head"].T)).reshape(S, cfg.vocab)
    return logits
