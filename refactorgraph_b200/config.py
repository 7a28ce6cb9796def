"""Decoder shape description.  Pure Python with no native dependency, so that tools which only need the arithmetic of a
shape (parameter counts, bytes per step) can import it without loading the kernel library."""
from __future__ import annotations

from dataclasses import dataclass

FP16 = 10  # reference DataType code (src/00common/include/common/data_type.h:14-35)


@dataclass
class LlamaConfig:
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 32
    head_dim: int = 128
    ffn: int = 11008
    vocab: int = 32000
    eps: float = 1e-6
    theta: float = 10000.0
    max_seq: int = 2304   # tokens per sequence the contiguous KV cache can hold
    batch: int = 1
    dtype: int = FP16

    @property
    def params(self) -> int:
        qkv = (self.heads + 2 * self.kv_heads) * self.head_dim * self.hidden
        o = self.hidden * self.heads * self.head_dim
        ffn = 3 * self.hidden * self.ffn
        return self.layers * (qkv + o + ffn + 2 * self.hidden) + self.vocab * self.hidden + self.hidden

    @property
    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one decode step reads (embedding rows are gathered, not streamed)."""
        return 2 * self.params

    @property
    def kv_bytes_per_token(self) -> int:
        return 2 * self.layers * self.kv_heads * self.head_dim * 2
