"""TEST INFRASTRUCTURE ONLY — decode steps composed from the numpy oracle (oracle_np.py): a greedy loop for the
fused single-token path and a step that rounds every intermediate where the multi-kernel GPU graph stores it
(optionally tensor-parallel, with the per-rank partial products rounded and summed in rank order)."""
import numpy as np

from . import oracle_np as onp


def oracle_decode(cfg, w, kc, vc, token, pos, steps, rnd=None):
    """Greedy decode with the numpy oracle on fp16-rounded weights; returns tokens [steps, B] and logits."""
    r16 = rnd or (lambda a: a.astype(np.float16).astype(np.float32))
    B, D, nH, nKV = cfg.batch, cfg.head_dim, cfg.heads, cfg.kv_heads
    kc = [k.astype(np.float32).copy() for k in kc]
    vc = [v.astype(np.float32).copy() for v in vc]
    toks, all_logits = [], []
    token, pos = token.copy(), pos.copy()
    for _ in range(steps):
        x = w["embed"][token].astype(np.float32)
        for l in range(cfg.layers):
            q, k, v = onp.linear_fused(x, w[f"l{l}.wqkv"], g=w[f"l{l}.norm1"], eps=cfg.eps, epilogue=3, n_heads=nH, n_kv=nKV,
                                       head_dim=D, positions=pos, theta=cfg.theta)
            for b in range(B):
                kc[l][b, :, pos[b]] = r16(k[b])
                vc[l][b, :, pos[b]] = r16(v[b])
            a = r16(onp.attn_decode(r16(q), kc[l], vc[l], pos + 1)).reshape(B, nH * D)
            h = r16(onp.linear_fused(a, w[f"l{l}.wo"], residual=x, epilogue=1))
            u = r16(onp.linear_fused(h, w[f"l{l}.wgu"], g=w[f"l{l}.norm2"], eps=cfg.eps, epilogue=2))
            x = r16(onp.linear_fused(u, w[f"l{l}.wd"], residual=h, epilogue=1))
        logits = r16(onp.linear_fused(x, w["lm_head"], g=w["norm_f"], eps=cfg.eps))
        token = onp.topk(logits, 1)[1][:, 0]
        pos = pos + 1
        toks.append(token.copy())
        all_logits.append(logits)
    return np.stack(toks), np.stack(all_logits)




def _mm(x, w):
    """x[m,k] (any float) times w[n,k]^T in float64."""
    return x.astype(np.float64) @ w.astype(np.float64).T


class KvHistory:
    """Per-layer, per-sequence K/V history for the oracle: a read-only prefix (any float array [nKV, >=past, D], views
    allowed, never written) plus the rows appended during the test.  Keeps a 7B-shaped, batch-32 cache affordable on
    the host: the prefix is not copied."""

    def __init__(self, prefix, past):
        self.prefix, self.past, self.rows = prefix, int(past), []

    def append(self, row):            # row [nKV, D]
        self.rows.append(np.asarray(row, np.float32))

    def all(self):
        head = np.asarray(self.prefix[:, :self.past], np.float32)
        if not self.rows:
            return head
        return np.concatenate([head, np.stack(self.rows, axis=1)], axis=1)


def oracle_decode_step_rounded(cfg, w, kh, vh, token, pos, rnd, world=1):
    """One decode step of the multi-kernel (batched) graph with every intermediate rounded to the storage type exactly
    where the GPU graph stores it: normalised activations, QKV product, rotated q / k, attention output, each rank's
    partial O and down products (tensor-parallel: rounded per rank, summed in fp32 in rank order, rounded, residual
    added, rounded), gate/up product, SiLU gate.  kh / vh: [layer][sequence] KvHistory.  Returns fp32 logits [B, vocab]
    (the last product is NOT rounded: the caller compares fp16 logits with a tolerance)."""
    B, D, nH, nKV, F = cfg.batch, cfg.head_dim, cfg.heads, cfg.kv_heads, cfg.ffn
    x = w["embed"][token].astype(np.float32)
    for l in range(cfg.layers):
        n1 = rnd(onp.rms_norm(x, w[f"l{l}.norm1"], cfg.eps))
        qkv = rnd(_mm(n1, w[f"l{l}.wqkv"]))
        q = rnd(onp.rope(qkv[:, : nH * D].reshape(B, nH, D), pos, cfg.theta))
        k = rnd(onp.rope(qkv[:, nH * D: (nH + nKV) * D].reshape(B, nKV, D), pos, cfg.theta))
        v = qkv[:, (nH + nKV) * D:].reshape(B, nKV, D)
        a = np.zeros((B, nH * D), np.float32)
        for b in range(B):
            kh[l][b].append(k[b]), vh[l][b].append(v[b])
            K, V = kh[l][b].all(), vh[l][b].all()
            a[b] = onp.attn_decode(q[b:b + 1], K[None], V[None], np.array([K.shape[1]]))[0].reshape(-1)
        a = rnd(a)
        wo, wd = w[f"l{l}.wo"], w[f"l{l}.wd"]
        if world == 1:
            h = rnd(_mm(a, wo) + x)                                   # residual rides in the GEMM epilogue (fp32), one rounding
        else:
            c = nH * D // world
            part = [rnd(_mm(a[:, r * c:(r + 1) * c], wo[:, r * c:(r + 1) * c])).astype(np.float32) for r in range(world)]
            acc = part[0]
            for r in range(1, world):
                acc = acc + part[r]                                   # fp32, rank order
            h = rnd(rnd(acc) + x)
        n2 = rnd(onp.rms_norm(h, w[f"l{l}.norm2"], cfg.eps))
        gu = rnd(_mm(n2, w[f"l{l}.wgu"]))
        u = rnd(onp.silu(gu[:, :F]) * gu[:, F:])
        if world == 1:
            x = rnd(_mm(u, wd) + h)
        else:
            c = F // world
            part = [rnd(_mm(u[:, r * c:(r + 1) * c], wd[:, r * c:(r + 1) * c])).astype(np.float32) for r in range(world)]
            acc = part[0]
            for r in range(1, world):
                acc = acc + part[r]
            x = rnd(rnd(acc) + h)
    xf = rnd(onp.rms_norm(x, w["norm_f"], cfg.eps))
    return _mm(xf, w["lm_head"]).astype(np.float32)
