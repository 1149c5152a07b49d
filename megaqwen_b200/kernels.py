"""Standalone ops with the reference's Python surface.

``get_kernels()`` returns an object with ``rms_norm``, ``silu_mul``, ``rope``,
``rope_single`` and ``attention_decode`` taking bf16 CUDA tensors in the shapes
of the reference's extension (csrc/kernels/__init__.py:112-291, 345-379).
Every op is one call into the C ABI; there is no PyTorch fallback.
"""
from __future__ import annotations

import math

import torch

from . import _lib


def _chk(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if t.dtype != torch.bfloat16:
        raise RuntimeError(f"{name} must be bfloat16")


class _Kernels:
    def __init__(self):
        self._lib = _lib.lib()

    @staticmethod
    def _stream(t):
        return torch.cuda.current_stream(t.device).cuda_stream

    def rms_norm(self, x, weight, eps: float = 1e-6):
        _chk(x, "x"); _chk(weight, "weight")
        x = x.contiguous()
        n_cols = x.shape[-1]
        out = torch.empty_like(x)
        if x.numel() == 0:
            return out
        with torch.cuda.device(x.device):
            _lib.check(self._lib.mq_launch_rms_norm(x.data_ptr(), weight.contiguous().data_ptr(), out.data_ptr(),
                                                    x.numel() // n_cols, n_cols, float(eps), self._stream(x)), "mq_launch_rms_norm")
        return out

    def silu_mul(self, gate, up):
        _chk(gate, "gate"); _chk(up, "up")
        if gate.shape != up.shape:
            raise RuntimeError("gate and up must have the same shape")
        gate, up = gate.contiguous(), up.contiguous()
        out = torch.empty_like(gate)
        if gate.numel() == 0:
            return out
        with torch.cuda.device(gate.device):
            _lib.check(self._lib.mq_launch_silu_mul(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), self._stream(gate)),
                       "mq_launch_silu_mul")
        return out

    def rope(self, q, k, cos, sin):
        """q (batch, n_q_heads, seq, d), k (batch, n_kv_heads, seq, d), cos/sin (seq, d) -> rotated (q, k)."""
        for t, n in ((q, "q"), (k, "k"), (cos, "cos"), (sin, "sin")):
            _chk(t, n)
        b, hq, s, d = q.shape
        hk = k.shape[1]
        qr = q.permute(2, 0, 1, 3).contiguous()       # [seq, batch*heads, d]
        kr = k.permute(2, 0, 1, 3).contiguous()
        qo, ko = torch.empty_like(qr), torch.empty_like(kr)
        with torch.cuda.device(q.device):
            _lib.check(self._lib.mq_launch_rope(qr.data_ptr(), kr.data_ptr(), cos.contiguous().data_ptr(), sin.contiguous().data_ptr(),
                                                qo.data_ptr(), ko.data_ptr(), s, b * hq, b * hk, d, self._stream(q)), "mq_launch_rope")
        return qo.permute(1, 2, 0, 3).contiguous(), ko.permute(1, 2, 0, 3).contiguous()

    def rope_single(self, x, cos, sin, position: int):
        """x (n_heads, d) at one position; cos/sin are the full tables (positions, d)."""
        _chk(x, "x"); _chk(cos, "cos"); _chk(sin, "sin")
        if position >= cos.shape[0]:
            raise RuntimeError("position outside the RoPE table")
        x = x.contiguous()
        out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _lib.check(self._lib.mq_launch_rope_single(x.data_ptr(), cos.contiguous().data_ptr(), sin.contiguous().data_ptr(), out.data_ptr(),
                                                       x.shape[0], x.shape[1], int(position), self._stream(x)), "mq_launch_rope_single")
        return out

    def attention_decode(self, q, k_cache, v_cache, cache_len: int):
        """q (batch, n_q_heads, 1, d); caches (batch, n_kv_heads, max_seq, d) -> (batch, n_q_heads, d)."""
        _chk(q, "q"); _chk(k_cache, "k_cache"); _chk(v_cache, "v_cache")
        b, hq, _, d = q.shape
        hk, max_seq = k_cache.shape[1], k_cache.shape[2]
        qf = q.squeeze(2).contiguous()
        out = torch.empty_like(qf)
        with torch.cuda.device(q.device):
            _lib.check(self._lib.mq_launch_attention_decode(qf.data_ptr(), k_cache.contiguous().data_ptr(), v_cache.contiguous().data_ptr(),
                                                            out.data_ptr(), b, int(cache_len), hq, hk, d, max_seq, 1.0 / math.sqrt(d),
                                                            self._stream(q)), "mq_launch_attention_decode")
        return out


_kernels = None


def get_kernels() -> _Kernels:
    global _kernels
    if _kernels is None:
        if not torch.cuda.is_available():
            raise RuntimeError("megaqwen_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        _kernels = _Kernels()
    return _kernels
