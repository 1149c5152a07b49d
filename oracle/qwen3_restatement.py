"""CPU restatement of the Qwen3 greedy prefill+decode path, one op at a time.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Every function states the arithmetic of one stage of the reference path with
the rounding points of the reference's ground truth (HuggingFace
``Qwen3ForCausalLM`` in bf16, see oracle/hf_reference.py): a bf16 value leaves
every linear layer, norm, RoPE product and sum, activation, gate*up product,
residual add and the logits; dot products and norms accumulate in fp32.  The
CUDA kernels are written to the same rounding points, so they are compared
with this file stage by stage and with the HF model end to end.

Reference files followed (semantics, not code):
  layer order / residuals      demo_e2e.py:351-362, fused_decode_ldg_kernel.inl:43-101
  RMSNorm                      csrc/kernels/rms_norm.cu:1-11, qwen3-0.6b.py:62-69
  per-head QK-norm + RoPE      fused_decode_ldg_common.inl:268-394, csrc/kernels/rope.cu:1-11,
                               demo_e2e.py:180-195
  RoPE tables                  csrc/megakernel/megakernel_weights.py:131-137
  GQA attention, causal mask   demo_e2e.py:266-304, fused_decode_ldg_common.inl:417-602
  SwiGLU                       csrc/kernels/silu_mul.cu:1-8, fused_decode_ldg_mlp.inl:5-218
  KV cache layout / position   bindings_decode.cpp:127-130, fused_decode_ldg_kernel.inl:43-68
  LM head + argmax             fused_decode_ldg_lm.inl:47-163
  FP8 (e4m3) shadow KV cache   csrc/megakernel/split_decode_gemm.cu:74-78 (scale), 223-300
                               (quantise a span), 429-493 (append a row), 950-1310 (attention);
                               bindings_prefill.cpp:1371-1400 (when the span is quantised)
"""
from __future__ import annotations

import math

import torch

BF16 = torch.bfloat16
F32 = torch.float32


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """bf16 [.., n] -> bf16: fp32 x * rsqrt(mean(x^2) + eps), rounded to bf16,
    then multiplied by the bf16 weight (second rounding)."""
    xf = x.to(F32)
    var = xf.pow(2).mean(-1, keepdim=True)
    return w * (xf * torch.rsqrt(var + eps)).to(BF16)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """bf16 [m, k] x bf16 [n, k]^T -> bf16 [m, n], fp32 accumulation."""
    return (x.to(F32) @ w.to(F32).t()).to(BF16)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Split-half rotary embedding evaluated in bf16: both products and their
    sum round.  x [.., heads, d]; cos/sin broadcastable [.., 1, d]."""
    d = x.shape[-1]
    rot = torch.cat((-x[..., d // 2:], x[..., : d // 2]), dim=-1)
    return (x * cos) + (rot * sin)


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """bf16(silu(gate)) * up, both steps rounding to bf16."""
    g = gate.to(F32)
    act = (g / (1.0 + torch.exp(-g))).to(BF16)
    return act * up


FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


def fp8_scale_of(amax: torch.Tensor) -> torch.Tensor:
    """amax / 448, or 1 where amax < 1e-8 (split_decode_gemm.cu:74-78)."""
    return torch.where(amax < 1.0e-8, torch.ones_like(amax), amax / FP8_MAX)


def to_fp8(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """e4m3(x * (1 / scale)): fp32 product, round to nearest even, saturating at +-448."""
    inv = (1.0 / scale.to(F32))
    return (x.to(F32) * inv).clamp(-FP8_MAX, FP8_MAX).to(FP8)


def attention_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos0: int, scale: float,
                   k_scale=None, v_scale=None) -> torch.Tensor:
    """Causal GQA attention for query rows at absolute positions q_pos0.. over
    keys 0..kv_len-1.  q [s, Hq, d] bf16, k/v [Hkv, kv_len, d] bf16 ->
    [s, Hq*d] bf16.  Scores and softmax in fp32; the probabilities are rounded
    to bf16 before the value product, which accumulates in fp32 and is divided
    by the fp32 row sum.  With k_scale / v_scale ([Hkv] fp32) k and v hold the
    unscaled e4m3 values: the scores are multiplied by scale * k_scale and the
    output by v_scale, both in fp32."""
    s, hq, d = q.shape
    hkv, kv_len, _ = k.shape
    rep = hq // hkv
    out = torch.empty((s, hq, d), dtype=BF16)
    pos_q = torch.arange(q_pos0, q_pos0 + s).view(s, 1)
    pos_k = torch.arange(kv_len).view(1, kv_len)
    allowed = pos_k <= pos_q
    for h in range(hq):
        kh = k[h // rep].to(F32)
        vh = v[h // rep].to(F32)
        sc_mul = scale if k_scale is None else float(torch.tensor(scale, dtype=F32) * k_scale[h // rep])
        sc = (q[:, h].to(F32) @ kh.t()) * sc_mul
        sc = sc.masked_fill(~allowed, float("-inf"))
        m = sc.max(-1, keepdim=True).values
        p = torch.exp(sc - m)
        l = p.sum(-1, keepdim=True)
        o = (p.to(BF16).to(F32) @ vh) / l
        if v_scale is not None:
            o = o * v_scale[h // rep]
        out[:, h] = o.to(BF16)
    return out.reshape(s, hq * d)


class RestatedQwen3:
    """State: KV cache [L, Hkv, max_seq, D] bf16 (K after QK-norm and RoPE, V
    raw) and ``position`` = number of tokens consumed, as the reference's
    decoder object keeps them (bindings_decode.cpp:80-271)."""

    def __init__(self, spec, weights: dict, max_seq_len: int, kv_fp8: bool = False):
        self.spec = spec
        self.w = weights
        self.max_seq_len = max_seq_len
        self.k_cache = torch.zeros((spec.num_layers, spec.num_kv_heads, max_seq_len, spec.head_dim), dtype=BF16)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.position = 0
        self.scale = 1.0 / math.sqrt(spec.head_dim)
        # FP8 shadow cache: single-token steps attend over e4m3 copies of K and V with one scale per
        # (layer, kv head); multi-token forwards (prefill) read and write the bf16 cache only
        self.kv_fp8 = kv_fp8
        if kv_fp8:
            self.k8 = torch.zeros(self.k_cache.shape, dtype=FP8)
            self.v8 = torch.zeros(self.k_cache.shape, dtype=FP8)
            self.k_scale = torch.ones((spec.num_layers, spec.num_kv_heads), dtype=F32)
            self.v_scale = torch.ones_like(self.k_scale)
            self.fp8_ready = 0

    def reset(self):
        self.k_cache.zero_()
        self.v_cache.zero_()
        self.position = 0
        if self.kv_fp8:
            self.k8 = torch.zeros(self.k_cache.shape, dtype=FP8)
            self.v8 = torch.zeros(self.k_cache.shape, dtype=FP8)
            self.k_scale.fill_(1.0)
            self.v_scale.fill_(1.0)
            self.fp8_ready = 0

    def quantize_kv(self, start: int, end: int):
        """Positions [start, end) of the bf16 caches -> shadow caches; the scales are SET from
        the span (split_decode_gemm.cu:223-300)."""
        if start >= end:
            return
        for cache, c8, sc in ((self.k_cache, self.k8, self.k_scale), (self.v_cache, self.v8, self.v_scale)):
            span = cache[:, :, start:end].to(F32)
            sc.copy_(fp8_scale_of(span.abs().amax(dim=(2, 3))))
            c8[:, :, start:end] = to_fp8(span, sc.view(*sc.shape, 1, 1))

    def forward(self, ids, return_hidden: bool = False, patch=None) -> torch.Tensor:
        """Consume ``ids`` (s >= 1 tokens) at positions position..position+s-1;
        returns fp32 logits [V] of the last row (bf16 values).  ``patch`` = (start, rows
        [n, H] bf16) replaces embedded rows start..start+n-1 before the first layer, as the
        reference's speech front-end does (csrc/megakernel/fused_prefill_kernels.inl:28-45)."""
        sp, w = self.spec, self.w
        ids = torch.as_tensor(ids, dtype=torch.long).view(-1)
        s = ids.numel()
        p0 = self.position
        assert p0 + s <= self.max_seq_len
        cos = w["cos_table"][p0:p0 + s].view(s, 1, sp.head_dim)
        sin = w["sin_table"][p0:p0 + s].view(s, 1, sp.head_dim)
        h = w["embed_weight"][ids]                                   # [s, H] bf16
        fp8_step = self.kv_fp8 and s == 1
        if fp8_step and self.fp8_ready < p0:                          # rows a prefill wrote (bindings_prefill.cpp:1371-1400)
            self.quantize_kv(0, p0)
        if patch is not None:
            h = h.clone()
            h[patch[0]:patch[0] + patch[1].shape[0]] = patch[1].to(h.dtype)
        for l in range(sp.num_layers):
            (w_in, wq, wk, wv, w_qn, w_kn, wo, w_post, wg, wu, wd) = w["layer_weights"][11 * l: 11 * l + 11]
            x = rms_norm(h, w_in, sp.rms_eps)
            q = linear(x, wq).view(s, sp.num_q_heads, sp.head_dim)
            k = linear(x, wk).view(s, sp.num_kv_heads, sp.head_dim)
            v = linear(x, wv).view(s, sp.num_kv_heads, sp.head_dim)
            q = rope(rms_norm(q, w_qn, sp.rms_eps), cos, sin)
            k = rope(rms_norm(k, w_kn, sp.rms_eps), cos, sin)
            self.k_cache[l, :, p0:p0 + s] = k.transpose(0, 1)
            self.v_cache[l, :, p0:p0 + s] = v.transpose(0, 1)
            if fp8_step:
                ks = torch.where(self.k_scale[l] < 1.0e-8, torch.ones_like(self.k_scale[l]), self.k_scale[l])
                vs = torch.where(self.v_scale[l] < 1.0e-8, torch.ones_like(self.v_scale[l]), self.v_scale[l])
                self.k8[l, :, p0:p0 + 1] = to_fp8(k.transpose(0, 1), ks.view(-1, 1, 1))
                self.v8[l, :, p0:p0 + 1] = to_fp8(v.transpose(0, 1), vs.view(-1, 1, 1))
                a = attention_rows(q, self.k8[l, :, :p0 + 1].to(F32), self.v8[l, :, :p0 + 1].to(F32), p0, self.scale, ks, vs)
            else:
                a = attention_rows(q, self.k_cache[l, :, :p0 + s], self.v_cache[l, :, :p0 + s], p0, self.scale)
            h = h + linear(a, wo)
            x = rms_norm(h, w_post, sp.rms_eps)
            m = silu_mul(linear(x, wg), linear(x, wu))
            h = h + linear(m, wd)
        self.position = p0 + s
        if self.kv_fp8:
            self.fp8_ready = self.position if fp8_step else 0
        if return_hidden:
            return h
        x = rms_norm(h[-1:], w["final_norm_weight"], sp.rms_eps)
        return linear(x, w["lm_head_weight"])[0].to(F32)

    def decode_step(self, token: int) -> int:
        """One token in, greedy next token out (first index among ties)."""
        return int(torch.argmax(self.forward([token])))

    def prefill_step(self, ids) -> int:
        return int(torch.argmax(self.forward(ids)))

    def step_logits(self, prompt_ids, forced_tokens, token_by_token_prompt: bool = False) -> torch.Tensor:
        """Teacher-forced logits, same contract as hf_reference.hf_step_logits."""
        self.reset()
        if token_by_token_prompt:
            for t in torch.as_tensor(prompt_ids).tolist():
                lg = self.forward([t])
        else:
            lg = self.forward(prompt_ids)
        rows = [lg]
        for t in forced_tokens:
            rows.append(self.forward([int(t)]))
        return torch.stack(rows)
