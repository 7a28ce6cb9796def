"""Why the bf16 prefill comparison uses a wider tolerance than the fp16 ones.

Two CPU runs of the same oracle restatement of a 7B-shaped two-layer bf16 prefill (1024 tokens), identical except that
one accumulates the matrix products in fp32 and the other in fp64, do not agree to the fp16 tolerance (max-abs 2e-2,
relative 1e-2): a product that lands on the other side of a bf16 rounding boundary changes that element by 0.4-0.8 %, and
the next normalisation and 1024-key softmax spread the change.  The GPU differs from the fp64 oracle for the same
reason, so tests/test_baseline_shapes_gpu.py compares bf16 logits at the oracle's own reproducibility (max-abs 8e-2,
relative 2e-2, rms 2e-2).  This test keeps that statement checked: it fails if the two CPU runs start to agree within
the fp16 tolerance (then the GPU test should be tightened) or stop agreeing within the bf16 one."""
import numpy as np
import torch

from oracle import oracle_np as onp
from refactorgraph_b200.config import LlamaConfig


def _bf(a):
    return torch.as_tensor(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def test_fp32_and_fp64_accumulation_part_ways_in_bf16_storage():
    S = 1024
    cfg = LlamaConfig(layers=2, max_seq=S, batch=1)
    D, nH, F, H = cfg.head_dim, cfg.heads, cfg.ffn, cfg.hidden
    rng = np.random.default_rng(0)
    wgen = lambda *s: _bf(0.02 * rng.standard_normal(s, dtype=np.float32))
    gamma = lambda: _bf(1 + 0.02 * rng.standard_normal(H, dtype=np.float32))
    w = {"embed": wgen(cfg.vocab, H), "lm_head": wgen(cfg.vocab, H), "norm_f": gamma()}
    for l in range(cfg.layers):
        w[f"l{l}.norm1"], w[f"l{l}.norm2"] = gamma(), gamma()
        w[f"l{l}.wqkv"], w[f"l{l}.wo"], w[f"l{l}.wgu"], w[f"l{l}.wd"] = wgen(3 * H, H), wgen(H, H), wgen(2 * F, H), wgen(H, F)
    ids = rng.integers(0, cfg.vocab, (S,))
    pos = np.arange(S, dtype=np.int64)
    causal = torch.triu(torch.ones(S, S, dtype=torch.bool), 1)

    def run(acc):
        mm = lambda x, wt: (torch.from_numpy(np.asarray(x, np.float32)).to(acc) @ torch.from_numpy(wt).to(acc).T).double().numpy()
        x = w["embed"][ids]
        for l in range(cfg.layers):
            n1 = _bf(onp.rms_norm(x, w[f"l{l}.norm1"], cfg.eps))
            qkv = mm(n1, w[f"l{l}.wqkv"])
            q = _bf(onp.rope(qkv[:, :H].reshape(-1, nH, D), pos))
            k = _bf(onp.rope(qkv[:, H:2 * H].reshape(-1, nH, D), pos))
            v = _bf(qkv[:, 2 * H:].reshape(-1, nH, D))
            a = np.empty((S, H), np.float32)
            for h in range(nH):
                qs, ks, vs = (torch.from_numpy(t[:, h]).double() for t in (q, k, v))
                sc = ((qs @ ks.T) / np.sqrt(D)).masked_fill(causal, float("-inf"))
                a[:, h * D:(h + 1) * D] = (torch.softmax(sc, -1) @ vs).float().numpy()
            hid = _bf(mm(_bf(a), w[f"l{l}.wo"]) + x)
            gu = mm(_bf(onp.rms_norm(hid, w[f"l{l}.norm2"], cfg.eps)), w[f"l{l}.wgu"])
            x = _bf(mm(_bf(onp.silu(gu[:, :F]) * gu[:, F:]), w[f"l{l}.wd"]) + hid)
        return mm(_bf(onp.rms_norm(x[-1:], w["norm_f"], cfg.eps)), w["lm_head"])

    a64, a32 = run(torch.float64), run(torch.float32)
    diff = np.abs(a64 - a32)
    assert diff.max() > 2e-2, "fp32 and fp64 accumulation agree within the fp16 tolerance: tighten the bf16 GPU comparison"
    assert np.all(diff <= 8e-2 + 2e-2 * np.abs(a64)) and float(np.sqrt((diff ** 2).mean())) < 2e-2
