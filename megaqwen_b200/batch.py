"""Batched greedy decoding: many independent sequences, weights read once per step.

The reference is batch-1 only; this is the batched counterpart of
``MegakernelPrefillDecoder`` with the same state semantics per sequence
(``positions()[b]`` = tokens consumed by sequence b).  Every sequence owns a
slice ``[b][L, 8, max_seq_len, 128]`` of the KV cache in the reference's
per-sequence layout.  All arithmetic runs through the C ABI
(``mq_launch_prefill`` per sequence, ``mq_launch_decode_batch`` per step).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import MqBatchBuffers, MqDecodeBuffers, MqKvFp8, MqLayerWeights, MqModel, MqPrefillBuffers
from .decoder import _D, _HIDDEN, _INTER, _LAYER_SHAPES, _NKV, _NQ, _ptr


class MegakernelBatchDecoder:
    def __init__(self, embed_weight, layer_weights, final_norm_weight, lm_head_weight, cos_table, sin_table,
                 num_layers, max_seq_len, max_batch, max_prefill_len=None, kv_fp8=False):
        if not torch.cuda.is_available():
            raise RuntimeError("megaqwen_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        self._lib = _lib.lib()
        if len(layer_weights) != 11 * num_layers:
            raise RuntimeError(f"layer_weights must hold 11 tensors per layer, got {len(layer_weights)} for {num_layers} layers")
        self.device = embed_weight.device
        self.num_layers_, self.max_seq_len_, self.max_batch_ = int(num_layers), int(max_seq_len), int(max_batch)
        self.max_prefill_len_ = int(max_prefill_len or max_seq_len)
        self.vocab_size_ = int(embed_weight.shape[0])
        if self.vocab_size_ % 128 != 0:
            raise RuntimeError("batched decode needs a vocabulary size that is a multiple of 128")
        for i, t in enumerate(layer_weights):
            if t.dtype != torch.bfloat16 or not t.is_contiguous() or tuple(t.shape) != _LAYER_SHAPES[i % 11]:
                raise RuntimeError(f"layer_weights[{i}]: expected contiguous bf16 {_LAYER_SHAPES[i % 11]}")
        self._weights = (embed_weight, list(layer_weights), final_norm_weight, lm_head_weight, cos_table, sin_table)
        self._layers = (MqLayerWeights * self.num_layers_)()
        for l in range(self.num_layers_):
            for j, (name, _) in enumerate(MqLayerWeights._fields_):
                setattr(self._layers[l], name, _ptr(layer_weights[11 * l + j]))
        self._model = MqModel(_ptr(embed_weight), self._layers, _ptr(final_norm_weight), _ptr(lm_head_weight),
                              _ptr(cos_table), _ptr(sin_table), self.num_layers_, self.vocab_size_, self.max_seq_len_)
        dev, bf, i32 = self.device, torch.bfloat16, torch.int32
        B = self.max_batch_
        with torch.cuda.device(dev):
            _lib.check(self._lib.mq_init_device(), "mq_init_device")
            self.k_cache_ = torch.zeros((B, self.num_layers_, _NKV, self.max_seq_len_, _D), dtype=bf, device=dev)
            self.v_cache_ = torch.zeros_like(self.k_cache_)
            self._positions = torch.zeros(B, dtype=i32, device=dev)
            self._logits = torch.empty((B, self.vocab_size_), dtype=bf, device=dev)
            # room for a ragged batch of prompts packed into one pass (at most 16384 rows, 370 MB)
            cap = max(B, self.max_prefill_len_, min(B * self.max_prefill_len_, 16384))
            self._act = [torch.empty((cap, w), dtype=bf, device=dev)
                         for w in (_HIDDEN, _HIDDEN, _NQ * _D + 2 * _NKV * _D, _NQ * _D, _INTER)]
            self._pf = MqPrefillBuffers(*[_ptr(t) for t in self._act], cap)
            self._scalars = torch.zeros(4, dtype=i32, device=dev)          # [0] prefill out token, [1] status
            self._hidden = torch.zeros(_HIDDEN, dtype=bf, device=dev)
            self._counters = torch.zeros(16, dtype=i32, device=dev)
            self._slot = torch.zeros(1, dtype=torch.int64, device=dev)
            self._tok_a = torch.zeros(B, dtype=i32, device=dev)
            self._partials = torch.empty(4 * min(B, 64) * 2 * _INTER, dtype=torch.float32, device=dev)
            # split-KV scratch of the batched attention: (m, l, acc[128]) per (sequence, kv head, part, head) and one ticket per item
            self._attn_parts = torch.empty(B * _NKV * 4 * 2 * (_D + 2), dtype=torch.float32, device=dev)
            self._attn_tickets = torch.zeros(B * _NKV, dtype=i32, device=dev)
            self.use_split_kv = True
            self.use_splitk = True
            self.use_packed_prefill = True
            self._chain = None
            self._graphs = {}
            # e4m3 shadow caches, one scale per (sequence, layer, kv head): prefill_batch quantises
            # every prompt, the decode steps append with those scales and attend over the shadow
            self.kv_fp8 = bool(kv_fp8)
            self._kv8 = None
            if self.kv_fp8:
                self.k_cache_fp8_ = torch.zeros(self.k_cache_.shape, dtype=torch.uint8, device=dev)
                self.v_cache_fp8_ = torch.zeros_like(self.k_cache_fp8_)
                self.kv_scales_ = torch.ones((2, B, self.num_layers_, _NKV), dtype=torch.float32, device=dev)   # [k | v]
                self._kv8 = MqKvFp8(_ptr(self.k_cache_fp8_), _ptr(self.v_cache_fp8_), _ptr(self.kv_scales_[0]), _ptr(self.kv_scales_[1]))
        self.batch_ = 0
        self.launches = 0

    # ------------------------------------------------------------------ helpers
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _bb(self, batch: int) -> MqBatchBuffers:
        return MqBatchBuffers(_ptr(self.k_cache_), _ptr(self.v_cache_), _ptr(self._positions), _ptr(self._logits),
                              self._pf, _ptr(self._scalars) + 4, batch,
                              _ptr(self._partials) if self.use_splitk else None, self._partials.numel() * 4,
                              _ptr(self._attn_parts) if self.use_split_kv else None, self._attn_parts.numel() * 4,
                              _ptr(self._attn_tickets) if self.use_split_kv else None)

    def check_status(self) -> None:
        st = int(self._scalars[1].item())
        if st:
            self._scalars[1] = 0
            raise RuntimeError(f"megaqwen_b200 device status: {st:#x}")

    def reset(self) -> None:
        self.k_cache_.zero_()
        self.v_cache_.zero_()
        self._positions.zero_()
        self.batch_ = 0
        if self.kv_fp8:
            self.k_cache_fp8_.zero_()
            self.v_cache_fp8_.zero_()
            self.kv_scales_.fill_(1.0)

    def _quantize_prompts(self, lens) -> None:
        """Shadow caches and scales of sequences 0 .. len(lens) - 1 from their prompts' bf16 rows."""
        if not self.kv_fp8:
            return
        with torch.cuda.device(self.device):
            for b, n in enumerate(lens):
                kv8 = MqKvFp8(_ptr(self.k_cache_fp8_[b]), _ptr(self.v_cache_fp8_[b]), _ptr(self.kv_scales_[0, b]), _ptr(self.kv_scales_[1, b]))
                rc = self._lib.mq_launch_kv_quantize_fp8(_ptr(self.k_cache_[b]), _ptr(self.v_cache_[b]), C.byref(kv8), self.num_layers_,
                                                         self.max_seq_len_, 0, int(n), self._stream())
                _lib.check(rc, "mq_launch_kv_quantize_fp8")
                self.launches += 1

    def positions(self) -> torch.Tensor:
        return self._positions[: self.batch_].clone()

    def get_k_cache(self) -> torch.Tensor:
        return self.k_cache_

    def get_v_cache(self) -> torch.Tensor:
        return self.v_cache_

    # ------------------------------------------------------------------ API
    def _prefill_packed(self, prompts, b0: int, out: torch.Tensor) -> None:
        """Sequences b0 .. b0+len(prompts)-1 in ONE pass: prompts packed row after row."""
        lens = torch.tensor([int(p.numel()) for p in prompts], dtype=torch.int64)
        nb, total = len(prompts), int(lens.sum())
        row0 = torch.cumsum(lens, 0) - lens
        row_seq = torch.repeat_interleave(torch.arange(nb), lens)
        row_pos = torch.arange(total) - row0[row_seq]
        ntile = (lens + 63) // 64
        tile_seq = torch.repeat_interleave(torch.arange(nb), ntile)
        tile_q0 = (torch.arange(int(ntile.sum())) - (torch.cumsum(ntile, 0) - ntile)[tile_seq]) * 64
        order = torch.argsort(tile_q0, descending=True, stable=True)      # long query tiles first
        tile_seq, tile_q0 = tile_seq[order], tile_q0[order]
        tables = torch.cat([torch.cat(prompts).to(torch.int64), row_seq, row_pos, tile_seq, tile_q0, lens, row0]).to(torch.int32)
        dev_t = tables.to(self.device)
        offs, acc = [], 0
        for n in (total, total, total, tile_seq.numel(), tile_seq.numel(), nb, nb):
            offs.append(_ptr(dev_t) + 4 * acc)
            acc += n
        self._positions[b0:b0 + nb].copy_((lens - 1).to(torch.int32))
        bb = MqBatchBuffers(_ptr(self.k_cache_[b0]), _ptr(self.v_cache_[b0]), _ptr(self._positions) + 4 * b0, _ptr(self._logits),
                            self._pf, _ptr(self._scalars) + 4, nb, None, 0)
        rc = self._lib.mq_launch_prefill_packed(C.byref(self._model), C.byref(bb), *offs, total, int(tile_seq.numel()),
                                                _ptr(out) + 4 * b0, self._stream())
        _lib.check(rc, "mq_launch_prefill_packed")
        self.launches += 1 + 8 * self.num_layers_ + 4
        self._keep = dev_t     # the launch reads the tables asynchronously

    def prefill_batch(self, prompts) -> torch.Tensor:
        """Prefill one prompt per sequence (ragged lengths allowed); sequence b
        takes prompts[b].  Returns the next token of every sequence (cpu int32).
        Consecutive sequences are packed into passes of at most the activation
        buffers' row capacity; a prompt that fills a pass alone goes through the
        single-sequence entry point."""
        if len(prompts) == 0 or len(prompts) > self.max_batch_:
            raise RuntimeError(f"prefill_batch: batch must be in 1..{self.max_batch_}")
        out = torch.zeros(len(prompts), dtype=torch.int32, device=self.device)
        prompts = [torch.as_tensor(p, dtype=torch.int32).reshape(-1).cpu() for p in prompts]
        for ids in prompts:
            n = int(ids.numel())
            if n <= 0:
                raise RuntimeError("Empty input sequence")
            if n > self.max_prefill_len_ or n > self.max_seq_len_:
                raise RuntimeError("Prefill sequence length exceeds maximum")
        cap = int(self._pf.max_tokens)
        if self.use_packed_prefill and len(prompts) > 1:
            with torch.cuda.device(self.device):
                b = 0
                while b < len(prompts):
                    e, rows = b, 0
                    while e < len(prompts) and rows + int(prompts[e].numel()) <= cap:
                        rows += int(prompts[e].numel())
                        e += 1
                    self._prefill_packed(prompts[b:e], b, out)
                    b = e
            self.batch_ = len(prompts)
            self._quantize_prompts([int(p.numel()) for p in prompts])
            res = out.cpu()
            self.check_status()
            return res
        lens = []
        with torch.cuda.device(self.device):
            for b, ids in enumerate(prompts):
                n = int(ids.numel())
                dev_ids = ids.to(self.device, non_blocking=True)
                dbuf = MqDecodeBuffers(_ptr(self.k_cache_[b]), _ptr(self.v_cache_[b]), _ptr(self._hidden), None, None, None, None,
                                       _ptr(self._counters), _ptr(self._slot), _ptr(self._scalars) + 4, 0)
                rc = self._lib.mq_launch_prefill(C.byref(self._model), C.byref(dbuf), C.byref(self._pf), _ptr(dev_ids), n, 0,
                                                 _ptr(out) + 4 * b, None, self._stream())
                _lib.check(rc, "mq_launch_prefill")
                self.launches += self._lib.mq_prefill_launch_count(self.num_layers_)
                lens.append(n)
            self._positions[: len(prompts)].copy_(torch.tensor(lens, dtype=torch.int32), non_blocking=False)
        self.batch_ = len(prompts)
        self._quantize_prompts(lens)
        res = out.cpu()
        self.check_status()
        return res

    def _step(self, in_ptr: int, out_ptr: int, logits_ptr=None) -> None:
        bb = self._bb(self.batch_)
        if self.kv_fp8:
            rc = self._lib.mq_launch_decode_batch_kv8(C.byref(self._model), C.byref(bb), C.byref(self._kv8), in_ptr, out_ptr, logits_ptr,
                                                      self._stream())
        else:
            rc = self._lib.mq_launch_decode_batch(C.byref(self._model), C.byref(bb), in_ptr, out_ptr, logits_ptr, self._stream())
        _lib.check(rc, "mq_launch_decode_batch")
        self.launches += self._lib.mq_decode_batch_launch_count(self.num_layers_)

    def decode_batch(self, tokens, return_logits: bool = False):
        """One step for every sequence: tokens int32 [batch] -> next tokens (cpu int32)."""
        tokens = torch.as_tensor(tokens, dtype=torch.int32).reshape(-1)
        if tokens.numel() != self.batch_:
            raise RuntimeError(f"decode_batch: expected {self.batch_} tokens")
        if int(self._positions[: self.batch_].max().item()) >= self.max_seq_len_:
            raise RuntimeError("decode_step would exceed max_seq_len")
        with torch.cuda.device(self.device):
            tin = tokens.to(self.device)
            out = torch.empty(self.batch_, dtype=torch.int32, device=self.device)
            lg = torch.empty((self.batch_, self.vocab_size_), dtype=torch.float32, device=self.device) if return_logits else None
            self._step(_ptr(tin), _ptr(out), _ptr(lg) if return_logits else None)
            res = out.cpu()
        self.check_status()
        return (res, lg) if return_logits else res

    def decode_batch_steps(self, first_tokens, num_steps: int, use_graph: bool = True) -> torch.Tensor:
        """Device-resident chain of num_steps steps; returns cuda int32 [num_steps, batch]."""
        B = self.batch_
        first = torch.as_tensor(first_tokens, dtype=torch.int32).reshape(-1)
        if first.numel() != B:
            raise RuntimeError(f"decode_batch_steps: expected {B} tokens")
        if int(self._positions[:B].max().item()) + num_steps > self.max_seq_len_:
            raise RuntimeError("decode_steps would exceed max_seq_len")
        with torch.cuda.device(self.device):
            if self._chain is None or self._chain.shape[0] < num_steps + 1 or self._chain.shape[1] != B:
                self._chain = torch.zeros((max(num_steps, 32) + 1, B), dtype=torch.int32, device=self.device)
                self._graphs = {}
            ch = self._chain
            ch[0].copy_(first.to(self.device))
            key = (num_steps, B, self.use_splitk, self.use_split_kv)     # the scratch pointers are baked into the captured launches
            if use_graph:
                g = self._graphs.get(key)
                if g is None:
                    # warm the tensor-map cache and shared-memory opt-ins outside the capture
                    saved = self._positions.clone()
                    self._step(_ptr(ch), _ptr(ch) + 4 * B)
                    self._positions.copy_(saved)
                    torch.cuda.synchronize(self.device)
                    g = torch.cuda.CUDAGraph()
                    n0 = self.launches
                    s = torch.cuda.Stream(device=self.device)
                    s.wait_stream(torch.cuda.current_stream(self.device))
                    with torch.cuda.stream(s):
                        with torch.cuda.graph(g, stream=s):
                            for i in range(num_steps):
                                self._step(_ptr(ch) + 4 * B * i, _ptr(ch) + 4 * B * (i + 1))
                    torch.cuda.current_stream(self.device).wait_stream(s)
                    self.launches = n0
                    self._graphs[key] = g
                g.replay()
                self.launches += num_steps * self._lib.mq_decode_batch_launch_count(self.num_layers_)
            else:
                for i in range(num_steps):
                    self._step(_ptr(ch) + 4 * B * i, _ptr(ch) + 4 * B * (i + 1))
            return ch[1:num_steps + 1].clone()
