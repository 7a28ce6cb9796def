"""Greedy decode loop composed from the numpy oracle (test helper)."""
import numpy as np

from oracle import oracle_np as onp


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


