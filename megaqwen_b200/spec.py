"""Model dimensions of the decode/prefill path.

The CUDA kernels are specialised at compile time for the Qwen3-0.6B block
geometry (hidden 1024, intermediate 3072, 16 query heads / 8 KV heads of
dimension 128), as the reference is (csrc/megakernel/config.cuh:64-73,
csrc/megakernel/megakernel_kernels.py:13-21).  The number of layers, the
vocabulary size and the cache length are run-time values, so the parity tests
can use a 2-layer / small-vocabulary model with the same kernels.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_q_heads: int = 16
    num_kv_heads: int = 8
    head_dim: int = 128
    num_layers: int = 28
    vocab_size: int = 151936
    rms_eps: float = 1e-6
    rope_theta: float = 1e6

    @property
    def q_size(self) -> int:
        return self.num_q_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def weight_bytes(self) -> int:
        """Bytes of weights one decoded token must read (bf16).

        Per layer: q,k,v,o,gate,up,down matrices plus four norm vectors; then
        the tied LM head read once, the final norm and one embedding row.
        """
        h, i, q, kv, d = self.hidden_size, self.intermediate_size, self.q_size, self.kv_size, self.head_dim
        per_layer = (q * h + 2 * kv * h + h * q + 2 * i * h + h * i) + (2 * h + 2 * d)
        return 2 * (self.num_layers * per_layer + self.vocab_size * h + h + h)

    def kv_bytes_per_position(self) -> int:
        """Bytes of K plus V one cached position holds over all layers (bf16)."""
        return self.num_layers * 2 * self.kv_size * 2

    def decode_bytes(self, cache_len: int) -> int:
        """Algorithmic HBM bytes of one batch-1 decode step that ends with
        ``cache_len`` cached positions: all weights, a read of every cached
        position and the write of the new one."""
        return self.weight_bytes() + self.kv_bytes_per_position() * (cache_len + 1)

    def prefill_flops(self, seq_len: int) -> float:
        h, i, q, kv, d = self.hidden_size, self.intermediate_size, self.q_size, self.kv_size, self.head_dim
        lin = q * h + 2 * kv * h + h * q + 3 * i * h
        attn = self.num_layers * self.num_q_heads * (2 * 2 * d) * seq_len * (seq_len + 1) / 2
        return 2.0 * seq_len * self.num_layers * lin + attn + 2.0 * self.vocab_size * h


QWEN3_0_6B = ModelSpec()

# Same block geometry, two layers and a 4096-entry vocabulary: runs through the
# CPU oracle in well under a second.
QWEN3_TINY = ModelSpec(num_layers=2, vocab_size=4096)
