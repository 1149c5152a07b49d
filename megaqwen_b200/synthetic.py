"""Deterministic synthetic weights and prompts.

No checkpoint or tokenizer of Qwen/Qwen3-0.6B is available offline, so the
benchmarks and parity tests run on random-init weights of that architecture:
every matrix is ``(randn(shape, float32) * 0.02).to(bfloat16)`` drawn from ONE
CPU generator seeded with ``seed`` in the fixed order embed, then per layer
q, k, v, o, gate, up, down; every norm weight is 1; the LM head is tied to the
embedding (reference: csrc/megakernel/megakernel_weights.py:269-272,478).
The result uses the reference's weight-dict layout
(csrc/megakernel/megakernel_weights.py:109-128, 424-450).
"""
from __future__ import annotations

import torch

from .spec import ModelSpec


def rope_tables(max_seq_len: int, rope_theta: float, head_dim: int, device="cpu"):
    """cos/sin [max_seq_len, head_dim] bf16, halves duplicated, computed in
    fp32 (reference: csrc/megakernel/megakernel_weights.py:131-137)."""
    inv_freq = 1.0 / (rope_theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    positions = torch.arange(max_seq_len, dtype=torch.float32)
    freqs = torch.outer(positions, inv_freq)
    cos = torch.cos(freqs).repeat(1, 2).to(torch.bfloat16).contiguous()
    sin = torch.sin(freqs).repeat(1, 2).to(torch.bfloat16).contiguous()
    return cos.to(device), sin.to(device)


def random_weights(spec: ModelSpec, max_seq_len: int, seed: int = 0, device="cpu") -> dict:
    g = torch.Generator().manual_seed(seed)

    def mat(rows, cols):
        w = (torch.randn((rows, cols), generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        return w.to(device)

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16, device=device)

    h, i, q, kv, d = spec.hidden_size, spec.intermediate_size, spec.q_size, spec.kv_size, spec.head_dim
    embed = mat(spec.vocab_size, h)
    layer_weights = []
    for _ in range(spec.num_layers):
        wq, wk, wv, wo = mat(q, h), mat(kv, h), mat(kv, h), mat(h, q)
        wg, wu, wd = mat(i, h), mat(i, h), mat(h, i)
        layer_weights.extend([ones(h), wq, wk, wv, ones(d), ones(d), wo, ones(h), wg, wu, wd])
    cos, sin = rope_tables(max_seq_len, spec.rope_theta, d, device)
    return {
        "embed_weight": embed,
        "layer_weights": layer_weights,
        "final_norm_weight": ones(h),
        "lm_head_weight": embed,
        "cos_table": cos,
        "sin_table": sin,
        "tokenizer": None,
    }


def random_prompt(spec: ModelSpec, length: int, cfg_idx: int = 1, seq_idx: int = 0) -> torch.Tensor:
    """Uniform random token ids, int32 [length], seed 1000 + 100*cfg + seq."""
    g = torch.Generator().manual_seed(1000 + cfg_idx * 100 + seq_idx)
    return torch.randint(0, spec.vocab_size, (length,), generator=g).to(torch.int32)


def random_lengths(count: int, low: int, high: int, seed: int = 4000) -> list[int]:
    """Per-sequence prompt lengths for the ragged batched configuration."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(low, high + 1, (count,), generator=g).tolist()
