"""Generates tests/golden/tiny_llama_c1.npz: logits and top-5 of the tiny CPU-runnable decoder (seed 0) computed by
the reference's own unmodified CPU kernels (oracle/_ref), once with its SoftmaxCpu as built and once with the
intended softmax.  The weights are not stored: they are redrawn from numpy default_rng(0).

    python tests/golden/make_tiny_llama.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from oracle import oracle_np as onp  # noqa: E402
from oracle import tiny_llama  # noqa: E402
from refactorgraph_b200.llama import LlamaConfig, seeded_weights  # noqa: E402

TINY = dict(layers=2, hidden=256, heads=4, kv_heads=4, head_dim=64, ffn=688, vocab=1000, eps=1e-6, max_seq=32, dtype=1)


def main():
    assert oracle.load_ref() is not None, "build oracle/_ref first: make -C oracle ref"
    cfg = LlamaConfig(**TINY)
    w = seeded_weights(cfg, 0)
    ids = np.random.default_rng(0).integers(0, cfg.vocab, (1, 32)).astype(np.int64)
    out = {"ids": ids}
    for mode in ("intended", "asbuilt"):
        logits = tiny_llama.prefill(cfg, w, ids, softmax=mode, kernels="ref")
        out[f"logits_{mode}"] = logits
        out[f"top5_{mode}"] = onp.topk(logits, 5)[1]
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_llama_c1.npz")
    np.savez_compressed(path, **out)
    d = np.abs(out["logits_intended"] - out["logits_asbuilt"]).max()
    same = (out["top5_intended"] == out["top5_asbuilt"]).mean()
    print(f"wrote {path} ({os.path.getsize(path)} B); as-built vs intended softmax: max |dlogit| {d:.4f}, top-5 agreement {same:.3f}")


if __name__ == "__main__":
    main()
