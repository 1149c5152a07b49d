"""Host-side decoder object: the Python mirror of the reference's pybind
classes ``MegakernelDecoder`` (csrc/megakernel/bindings_decode.cpp:80-280) and
``MegakernelPrefillDecoder`` (csrc/megakernel/bindings_prefill.cpp:1637-1701),
with the same constructor arguments, method names, state semantics and error
texts.  It owns the KV cache, scratch and the position counter as torch CUDA
tensors (torch is used for device memory, streams and graph capture only) and
calls the C ABI of libmegaqwen_b200.so for every piece of arithmetic.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _lib
from ._lib import MqDecodeBuffers, MqKvFp8, MqLayerWeights, MqModel, MqPrefillBuffers

_HIDDEN, _INTER, _NQ, _NKV, _D = 1024, 3072, 16, 8, 128
_LAYER_SHAPES = [(_HIDDEN,), (_NQ * _D, _HIDDEN), (_NKV * _D, _HIDDEN), (_NKV * _D, _HIDDEN), (_D,), (_D,),
                 (_HIDDEN, _NQ * _D), (_HIDDEN,), (_INTER, _HIDDEN), (_INTER, _HIDDEN), (_HIDDEN, _INTER)]


def _ptr(t: torch.Tensor) -> int:
    return t.data_ptr()


class MegakernelDecoder:
    """Batch-1 greedy decoder.

    ``position()`` is the number of tokens consumed.  ``decode_step(t)`` writes
    K/V at ``position``, attends over ``position + 1`` entries, returns the
    arg-max next token and increments the position.  ``prefill_step(ids)`` sets
    ``position = len(ids)`` and returns the token following the prompt.
    ``reset()`` zeroes the KV cache and the position.

    ``kv_fp8=True`` (default: the reference's switch, environment variable
    ``MEGAQWEN_SPLIT_KV_FP8``, bindings_prefill.cpp:513) keeps an e4m3 shadow of
    the KV cache with one scale per (layer, kv head) and lets the decode
    attention read it.  As in the reference (bindings_prefill.cpp:1371-1400) the
    rows a prefill wrote are quantised, and the scales set from them, right before
    the next decode launch; decode steps quantise their own rows with those scales.
    The bf16 caches stay complete (``get_k_cache``).  The persistent kernel reads
    the bf16 cache only and is not available in this mode.
    """

    def __init__(self, embed_weight, layer_weights, final_norm_weight, lm_head_weight, cos_table, sin_table,
                 num_layers, max_seq_len, max_prefill_len=512, *w4_args, kv_fp8=None, **w4_kwargs):
        if not torch.cuda.is_available():
            raise RuntimeError("megaqwen_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        self._lib = _lib.lib()
        for extra in list(w4_args) + list(w4_kwargs.values()):
            if extra is not None and hasattr(extra, "__len__") and len(extra) > 0:
                raise RuntimeError("W4 / paged-KV options are not supported by this engine")
        if len(layer_weights) != 11 * num_layers:
            raise RuntimeError(f"layer_weights must hold 11 tensors per layer, got {len(layer_weights)} for {num_layers} layers")
        self.device = embed_weight.device
        if self.device.type != "cuda":
            raise RuntimeError("weights must live on a CUDA device")
        self.num_layers_ = int(num_layers)
        self.max_seq_len_ = int(max_seq_len)
        self.max_prefill_len_ = int(max_prefill_len)
        self.vocab_size_ = int(embed_weight.shape[0])

        def chk(t, shape, name):
            if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.device != self.device or tuple(t.shape) != tuple(shape):
                raise RuntimeError(f"{name}: expected contiguous bf16 {tuple(shape)} on {self.device}, got {t.dtype} {tuple(t.shape)}")

        chk(embed_weight, (self.vocab_size_, _HIDDEN), "embed_weight")
        chk(lm_head_weight, (self.vocab_size_, _HIDDEN), "lm_head_weight")
        chk(final_norm_weight, (_HIDDEN,), "final_norm_weight")
        chk(cos_table, (self.max_seq_len_, _D), "cos_table")
        chk(sin_table, (self.max_seq_len_, _D), "sin_table")
        for i, t in enumerate(layer_weights):
            chk(t, _LAYER_SHAPES[i % 11], f"layer_weights[{i}]")
        # keep references: the C side only holds raw pointers
        self._weights = (embed_weight, list(layer_weights), final_norm_weight, lm_head_weight, cos_table, sin_table)

        self._layers = (MqLayerWeights * self.num_layers_)()
        for l in range(self.num_layers_):
            for j, (name, _) in enumerate(MqLayerWeights._fields_):
                setattr(self._layers[l], name, _ptr(layer_weights[11 * l + j]))
        self._model = MqModel(_ptr(embed_weight), self._layers, _ptr(final_norm_weight), _ptr(lm_head_weight),
                              _ptr(cos_table), _ptr(sin_table), self.num_layers_, self.vocab_size_, self.max_seq_len_)

        dev = self.device
        with torch.cuda.device(dev):
            _lib.check(self._lib.mq_init_device(), "mq_init_device")
            bf, i32 = torch.bfloat16, torch.int32
            self.k_cache_ = torch.zeros((self.num_layers_, _NKV, self.max_seq_len_, _D), dtype=bf, device=dev)
            self.v_cache_ = torch.zeros_like(self.k_cache_)
            self._hidden = torch.zeros(_HIDDEN, dtype=bf, device=dev)
            self._qkv = torch.zeros(_NQ * _D + 2 * _NKV * _D, dtype=bf, device=dev)
            self._attn = torch.zeros(_NQ * _D, dtype=bf, device=dev)
            self._act = torch.zeros(_INTER, dtype=bf, device=dev)
            nsplit = self._lib.mq_decode_attn_nsplit(self.max_seq_len_)
            self._partials = torch.zeros(self._lib.mq_decode_partials_bytes(self.max_seq_len_) // 4, dtype=torch.float32, device=dev)
            self._counters = torch.zeros(16, dtype=i32, device=dev)
            self._slot = torch.zeros(1, dtype=torch.int64, device=dev)
            # [0] = output token of single steps, [1] = sticky status word
            self._scalars = torch.zeros(4, dtype=i32, device=dev)
            self._in_token = torch.zeros(1, dtype=i32, device=dev)
            self._pos_dev = torch.zeros(1, dtype=i32, device=dev)
            self._logits = None
            self._pf = None            # prefill activation buffers, allocated at the first prefill
            self._pf_tensors = None
            self.use_gemm_prefill = True
            # Persistent decode (mq_launch_decode_stream): the weights repacked into per-CTA streams
            # (built at the first use) and the scratch that carries its phase counter.
            self._stream_packed = None
            self._stream_scratch = torch.zeros(self._lib.mq_stream_scratch_bytes(), dtype=torch.uint8, device=dev)
            self._stream_max_context = self._lib.mq_stream_max_context()
            self.persistent_available = self._stream_max_context > 0
            # opt-in: measured on B200 the graph-replayed per-phase kernels are still faster
            # (389 vs 425 us/token at context 1, 477 vs 508 at 2048)
            self.use_persistent = False
            self._chain_cap = 0
            self._chain_tokens = None
            self._chain_pos = None
            self._graphs = {}
            if kv_fp8 is None:
                kv_fp8 = os.environ.get("MEGAQWEN_SPLIT_KV_FP8", "0").strip().lower() in ("1", "true", "yes", "on")
            self.kv_fp8 = bool(kv_fp8)
            self._kv8 = None
            self._kv8_ready = 0        # positions [0, _kv8_ready) of the shadow cache are current
            if self.kv_fp8:
                self.k_cache_fp8_ = torch.zeros(self.k_cache_.shape, dtype=torch.uint8, device=dev)
                self.v_cache_fp8_ = torch.zeros_like(self.k_cache_fp8_)
                self.kv_scales_ = torch.ones((2, self.num_layers_, _NKV), dtype=torch.float32, device=dev)   # [k | v]
                self._kv8 = MqKvFp8(_ptr(self.k_cache_fp8_), _ptr(self.v_cache_fp8_), _ptr(self.kv_scales_[0]), _ptr(self.kv_scales_[1]))
                self.persistent_available = False
        self._buf = MqDecodeBuffers(_ptr(self.k_cache_), _ptr(self.v_cache_), _ptr(self._hidden), _ptr(self._qkv),
                                    _ptr(self._attn), _ptr(self._act), _ptr(self._partials), _ptr(self._counters),
                                    _ptr(self._slot), _ptr(self._scalars) + 4, nsplit)
        self.position_ = 0
        self.use_pdl = True
        self.use_step_graph = True  # decode_step replays a captured one-step graph instead of 141 eager launches
        self._step_graph = None
        self._step_graph_pdl = None
        self.launches = 0          # kernels launched through the C ABI by this object

    # ------------------------------------------------------------------ helpers
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _launch(self, in_ptr: int, out_ptr: int, pos_ptr: int, logits_ptr, chained: bool) -> None:
        flags = (_lib.MQ_FLAG_CHAINED if chained else 0) | (0 if self.use_pdl else _lib.MQ_FLAG_NO_PDL)
        if self.kv_fp8:
            rc = self._lib.mq_launch_decode_kv8(C.byref(self._model), C.byref(self._buf), C.byref(self._kv8), in_ptr, out_ptr,
                                                pos_ptr, logits_ptr, flags, self._stream())
        else:
            rc = self._lib.mq_launch_decode(C.byref(self._model), C.byref(self._buf), in_ptr, out_ptr, pos_ptr,
                                            logits_ptr, flags, self._stream())
        _lib.check(rc, "mq_launch_decode")
        self.launches += 5 * self.num_layers_ + 1

    def _kv8_sync(self) -> None:
        """Before a decode launch: rows written by a prefill since the last decode are quantised into
        the shadow cache and the scales are set from them (the whole prefix, so that one scale
        covers every cached row).  Not inside a graph capture: callers run it first."""
        if self.kv_fp8 and self._kv8_ready < self.position_:
            rc = self._lib.mq_launch_kv_quantize_fp8(_ptr(self.k_cache_), _ptr(self.v_cache_), C.byref(self._kv8), self.num_layers_,
                                                     self.max_seq_len_, 0, self.position_, self._stream())
            _lib.check(rc, "mq_launch_kv_quantize_fp8")
            self.launches += 1
            self._kv8_ready = self.position_

    def _check_status(self, status: int) -> None:
        if status:
            self._scalars[1] = 0
            what = []
            if status & _lib.MQ_STATUS_WAIT_TIMEOUT:
                what.append("a bounded device-side wait expired")
            if status & _lib.MQ_STATUS_BAD_POSITION:
                what.append("position outside the KV cache")
            if status & _lib.MQ_STATUS_BAD_TOKEN:
                what.append("token id outside the vocabulary")
            raise RuntimeError("megaqwen_b200 device status: " + ", ".join(what))

    def check_status(self) -> None:
        """Read the sticky device status word (one 4-byte copy) and raise if set."""
        self._check_status(int(self._scalars[1].item()))

    def _ensure_chain(self, n: int) -> None:
        if n > self._chain_cap:
            cap = max(n, 64)
            self._chain_tokens = torch.zeros(cap + 1, dtype=torch.int32, device=self.device)
            self._chain_pos = torch.zeros(cap, dtype=torch.int32, device=self.device)
            self._chain_cap = cap
            self._graphs = {}

    # ------------------------------------------------------------------ reference API
    def position(self) -> int:
        return self.position_

    def max_prefill_len(self) -> int:
        return self.max_prefill_len_

    def get_k_cache(self) -> torch.Tensor:
        return self.k_cache_

    def get_v_cache(self) -> torch.Tensor:
        return self.v_cache_

    def reset(self) -> None:
        self.position_ = 0
        self.k_cache_.zero_()
        self.v_cache_.zero_()
        if self.kv_fp8:
            self._kv8_ready = 0
            self.k_cache_fp8_.zero_()
            self.v_cache_fp8_.zero_()
            self.kv_scales_.fill_(1.0)

    def _single(self, input_token_id: int, logits_ptr) -> int:
        if self.position_ >= self.max_seq_len_:
            raise RuntimeError("decode_step would exceed max_seq_len")
        with torch.cuda.device(self.device):
            # scalar fills carry the value as a kernel argument: no host buffer to race on
            self._in_token.fill_(int(input_token_id))
            self._pos_dev.fill_(self.position_)
            self._kv8_sync()
            if logits_ptr is None and self.use_step_graph:
                self._replay_step_graph()
            else:
                self._launch(_ptr(self._in_token), _ptr(self._scalars), _ptr(self._pos_dev), logits_ptr, False)
            self.position_ += 1
            self._kv8_ready = self.position_
            tok, status = self._scalars[:2].tolist()
        self._check_status(status)
        return tok

    def _replay_step_graph(self) -> None:
        """One decode step (token and position in device scalars) captured once and replayed:
        the host cost of a step is one graph launch instead of 141 kernel launches."""
        if self._step_graph is None or self._step_graph_pdl != self.use_pdl:
            g = torch.cuda.CUDAGraph()
            launches0 = self.launches
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                with torch.cuda.graph(g, stream=s):
                    self._launch(_ptr(self._in_token), _ptr(self._scalars), _ptr(self._pos_dev), None, False)
            torch.cuda.current_stream(self.device).wait_stream(s)
            self.launches = launches0
            self._step_graph, self._step_graph_pdl = g, self.use_pdl
        self._step_graph.replay()
        self.launches += 5 * self.num_layers_ + 1

    def decode_step(self, input_token_id: int) -> int:
        return self._single(input_token_id, None)

    def decode_step_logits(self, input_token_id: int):
        """One step that also returns the bf16-rounded logits as fp32 [vocab]
        (reference: launch_ldg_decode_with_logits, chat.py:241-314)."""
        if self._logits is None:
            self._logits = torch.empty(self.vocab_size_, dtype=torch.float32, device=self.device)
        tok = self._single(input_token_id, _ptr(self._logits))
        return tok, self._logits.clone()

    def _chain(self, first_token, num_steps: int, use_graph: bool, what: str = "decode_steps") -> torch.Tensor:
        """Device-resident chain token[i] -> token[i+1]; returns the view of the
        num_steps generated tokens (cuda int32).  No host synchronisation."""
        if num_steps <= 0:
            return torch.empty(0, dtype=torch.int32, device=self.device)
        # the reference's bound (bindings_prefill.cpp:1049-1051, 1092): the last cache row stays unused
        if self.position_ + num_steps >= self.max_seq_len_:
            raise RuntimeError(f"{what} would exceed max_seq_len")
        with torch.cuda.device(self.device):
            self._ensure_chain(num_steps)
            self._kv8_sync()
            tk, ps = self._chain_tokens, self._chain_pos
            if torch.is_tensor(first_token):
                tk[0:1].copy_(first_token.reshape(1).to(torch.int32), non_blocking=True)
            else:
                tk[0:1].fill_(int(first_token))
            if self.use_persistent and not self.kv_fp8 and use_graph and self.position_ + num_steps <= self._stream_max_context:
                self._launch_stream(_ptr(tk), None, _ptr(tk) + 4, num_steps, None, False, None)
                self.position_ += num_steps
                return tk[1:num_steps + 1]
            _lib.check(self._lib.mq_launch_fill_iota(_ptr(ps), self.position_, num_steps, self._stream()), "mq_launch_fill_iota")
            self.launches += 1
            if use_graph:
                self._replay_graph(num_steps)
            else:
                for i in range(num_steps):
                    self._launch(_ptr(tk) + 4 * i, _ptr(tk) + 4 * (i + 1), _ptr(ps) + 4 * i, None, i > 0)
            self.position_ += num_steps
            self._kv8_ready = self.position_
            return tk[1:num_steps + 1]

    def _replay_graph(self, num_steps: int) -> None:
        key = (num_steps, self.use_pdl)      # the PDL attribute is baked into the captured launches
        g = self._graphs.get(key)
        tk, ps = self._chain_tokens, self._chain_pos
        if g is None:
            g = torch.cuda.CUDAGraph()
            launches0 = self.launches
            # capture on a side stream as torch requires; the chain reads tokens[0]
            # and positions[] which are refreshed before every replay
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                with torch.cuda.graph(g, stream=s):
                    for i in range(num_steps):
                        self._launch(_ptr(tk) + 4 * i, _ptr(tk) + 4 * (i + 1), _ptr(ps) + 4 * i, None, i > 0)
            torch.cuda.current_stream(self.device).wait_stream(s)
            self.launches = launches0
            self._graphs[key] = g
        g.replay()
        self.launches += num_steps * (5 * self.num_layers_ + 1)

    def decode_steps_cuda(self, first_token, num_steps: int) -> torch.Tensor:
        return self._chain(first_token, num_steps, False).clone()

    def decode_steps_cuda_graph(self, first_token, num_steps: int) -> torch.Tensor:
        """Per-phase kernels replayed from a CUDA graph (reference:
        decode_steps_cuda_graph, bindings_prefill.cpp:1082-1150)."""
        keep, self.use_persistent = self.use_persistent, False
        try:
            return self._chain(first_token, num_steps, True, "decode_steps_cuda_graph").clone()
        finally:
            self.use_persistent = keep

    def _ensure_stream_pack(self) -> None:
        if self._stream_packed is None:
            nbytes = self._lib.mq_stream_packed_bytes(C.byref(self._model))
            if nbytes == 0:
                raise RuntimeError("persistent decode is not available on this device")
            self._stream_packed = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            _lib.check(self._lib.mq_stream_pack(C.byref(self._model), _ptr(self._stream_packed), nbytes, self._stream()),
                       "mq_stream_pack")
            self.launches += 2 * self.num_layers_ + 1

    def _launch_stream(self, first_ptr, forced_ptr, out_ptr, num_steps, logits_ptr, logits_all, cycles_ptr) -> None:
        """num_steps steps in one cooperative launch starting at position_ (not advanced here)."""
        self._ensure_stream_pack()
        self._pos_dev.fill_(self.position_)
        rc = self._lib.mq_launch_decode_stream(
            C.byref(self._model), _ptr(self._stream_packed), _ptr(self.k_cache_), _ptr(self.v_cache_),
            _ptr(self._stream_scratch), _ptr(self._scalars) + 4, first_ptr, _ptr(self._pos_dev), forced_ptr, out_ptr,
            num_steps, logits_ptr, 1 if logits_all else 0, cycles_ptr, self._stream())
        _lib.check(rc, "mq_launch_decode_stream")
        self.launches += 1

    def _check_stream(self, num_steps: int, what: str) -> None:
        if self.kv_fp8:
            raise RuntimeError("the persistent kernel reads the bf16 KV cache only (kv_fp8 is on)")
        if not self.persistent_available:
            raise RuntimeError("persistent decode is not available on this device")
        if self.position_ + num_steps >= self.max_seq_len_:
            raise RuntimeError(f"{what} would exceed max_seq_len")
        if self.position_ + num_steps > self._stream_max_context:
            raise RuntimeError(f"{what}: context beyond {self._stream_max_context} positions goes through decode_steps_cuda_graph")

    def decode_steps_cuda_persistent(self, first_token, num_steps: int) -> torch.Tensor:
        """All steps in one persistent cooperative launch (mq_launch_decode_stream)."""
        if num_steps <= 0:
            return torch.empty(0, dtype=torch.int32, device=self.device)
        self._check_stream(num_steps, "decode_steps")
        keep, self.use_persistent = self.use_persistent, True
        try:
            return self._chain(first_token, num_steps, True).clone()
        finally:
            self.use_persistent = keep

    def decode_forced_logits(self, tokens):
        """Teacher-forced steps in one persistent launch: step i consumes tokens[i].  Returns
        (predicted tokens cuda int32 [n], logits cuda fp32 [n, vocab]); used by the parity tests."""
        forced = torch.as_tensor(tokens, dtype=torch.int32).reshape(-1).to(self.device)
        n = int(forced.numel())
        self._check_stream(n, "decode_steps")
        with torch.cuda.device(self.device):
            out = torch.empty(n, dtype=torch.int32, device=self.device)
            logits = torch.empty((n, self.vocab_size_), dtype=torch.float32, device=self.device)
            self._launch_stream(None, _ptr(forced), _ptr(out), n, _ptr(logits), True, None)
            self.position_ += n
        self.check_status()
        return out, logits

    def debug_decode_cycles(self, input_token_id: int) -> torch.Tensor:
        """One decode step with the per-stage cycle counters on (reference:
        debug_ldg_decode_cycles, bindings_prefill.cpp:980-1043).  Returns a CUDA int64 tensor
        [CTAs, num_layers + 1, stages]; the stage list is in include/megaqwen_b200.h."""
        self._check_stream(1, "decode_steps")
        with torch.cuda.device(self.device):
            cycles = torch.zeros((self._lib.mq_stream_grid(), self.num_layers_ + 1, self._lib.mq_stream_stage_count()),
                                 dtype=torch.int64, device=self.device)
            self._in_token.fill_(int(input_token_id))
            self._launch_stream(_ptr(self._in_token), None, _ptr(self._scalars), 1, None, False, _ptr(cycles))
            self.position_ += 1
        self.check_status()
        return cycles

    def decode_steps(self, first_token_id: int, num_steps: int) -> torch.Tensor:
        out = self._chain(first_token_id, num_steps, True)
        host = torch.cat([out, self._scalars[1:2]]).cpu()
        self._check_status(int(host[-1]))
        return host[:-1]

    def decode_greedy_cuda(self, first_token, max_new_tokens: int, eos_ids, chunk: int = 32):
        """Greedy loop with tokens kept on the device; the EOS scan and one 4-byte
        read happen once per chunk.  Same contract as the reference
        (bindings_prefill.cpp:1159-1349): the result holds the CONSUMED tokens,
        i.e. per chunk ``[next_token] + generated[:-1]``, so ``out[0]`` is
        ``first_token`` and the last token a chunk generated is carried into the
        next chunk instead of being returned; EOS is searched in
        ``generated[:-1]`` of each chunk and excluded from the result;
        ``position()`` advances by whole chunks (the cache rows past an EOS were
        computed and stay).  Returns (tokens cuda int32[len], len, stop_reason)
        with stop_reason 0 = max_new_tokens, 1 = EOS."""
        max_new = int(max_new_tokens)
        if max_new <= 0:
            return torch.empty(0, dtype=torch.int32, device=self.device), 0, 0
        if chunk <= 0:
            chunk = 32
        if eos_ids is None or len(eos_ids) == 0:
            raise RuntimeError("eos_ids must be a non-empty int32 tensor")
        eos = torch.as_tensor(eos_ids).to(device=self.device, dtype=torch.int32).contiguous()
        out = torch.empty(max_new, dtype=torch.int32, device=self.device)
        hit = torch.empty(1, dtype=torch.int32, device=self.device)
        gen_len, stop_reason, cur = 0, 0, first_token
        while gen_len < max_new:
            steps = min(chunk, max_new - gen_len)
            tail = self._chain(cur, steps, steps == chunk)          # view of tokens[1 .. steps]
            tokens = self._chain_tokens                             # tokens[0] = consumed token of this chunk
            out[gen_len:gen_len + steps].copy_(tokens[:steps])
            stop_pos = -1
            if steps > 1:
                hit.fill_(steps - 1)
                _lib.check(self._lib.mq_launch_find_first_eos(_ptr(tokens) + 4, steps - 1, _ptr(eos), eos.numel(), _ptr(hit),
                                                              self._stream()), "mq_launch_find_first_eos")
                self.launches += 1
                idx = int(hit.item())
                if idx < steps - 1:
                    stop_pos = idx + 1          # tokens kept from this chunk; the EOS itself is dropped
            if stop_pos >= 0:
                gen_len += stop_pos
                stop_reason = 1
                break
            gen_len += steps
            cur = tail[steps - 1:steps].clone()
        self.check_status()
        return out[:gen_len], gen_len, stop_reason

    def _check_prefill(self, ids: torch.Tensor, pos0: int) -> int:
        """The reference's checks and texts (bindings_prefill.cpp:731-739); the ASR caller
        matches on them (megaqwen/qwen3_asr_megakernel.py:767-773)."""
        n = int(ids.numel())
        if n > self.max_prefill_len_:
            raise RuntimeError("Prefill sequence length exceeds maximum")
        if n == 0:
            raise RuntimeError("Empty input sequence")
        if pos0 + n > self.max_seq_len_:
            raise RuntimeError("Prefill sequence length exceeds maximum (max_seq_len)")
        return n

    def prefill_step(self, input_ids) -> int:
        """Full-sequence forward from position 0: afterwards ``position() == len(ids)``
        and the returned token follows the prompt (bindings_prefill.cpp:731-833)."""
        ids = torch.as_tensor(input_ids, dtype=torch.int32).reshape(-1)
        self._check_prefill(ids, 0)
        self.position_ = 0
        if self.use_gemm_prefill:
            return self._prefill_gemm(ids)
        return self._prefill_by_decode(ids)

    def prefill_append(self, input_ids) -> int:
        """Chunked prefill (no reference counterpart): the tokens continue the sequence at
        ``position()`` and attend over everything cached so far."""
        ids = torch.as_tensor(input_ids, dtype=torch.int32).reshape(-1)
        self._check_prefill(ids, self.position_)
        return self._prefill_gemm(ids)

    def prefill_asr(self, input_token_ids, audio_embeds, audio_start_idx: int) -> int:
        """prefill_step with rows audio_start_idx .. + audio_len - 1 of the embedded prompt replaced by
        ``audio_embeds`` [audio_len, 1024] (CUDA bf16).  Same checks and texts as the reference
        (bindings_prefill.cpp:835-861)."""
        ids = torch.as_tensor(input_token_ids, dtype=torch.int32).reshape(-1)
        n = self._check_prefill(ids, 0)
        if (not torch.is_tensor(audio_embeds) or not audio_embeds.is_cuda or audio_embeds.dtype != torch.bfloat16
                or audio_embeds.dim() != 2):
            raise RuntimeError("audio_embeds must be a CUDA bfloat16 2D tensor [audio_len, hidden_size]")
        audio_len, hidden = int(audio_embeds.shape[0]), int(audio_embeds.shape[1])
        if hidden != _HIDDEN:
            raise RuntimeError("audio_embeds hidden_size mismatch with compiled megakernel spec: "
                               f"expected={_HIDDEN}, got={hidden}")
        if audio_len <= 0:
            raise RuntimeError("audio_embeds must have audio_len > 0")
        if audio_start_idx < 0 or audio_start_idx + audio_len > n:
            raise RuntimeError("Invalid audio_start_idx/audio_len for the given seq_len")
        self.position_ = 0
        return self._prefill_gemm(ids, audio=(audio_embeds.contiguous(), int(audio_start_idx)))

    def _prefill_gemm(self, ids: torch.Tensor, want_logits: bool = False, audio=None):
        """Full-sequence forward on the tcgen05 GEMM path (mq_launch_prefill)."""
        n = int(ids.numel())
        with torch.cuda.device(self.device):
            if self._pf is None or self._pf.max_tokens < n:
                cap = max(n, self.max_prefill_len_)
                bf = torch.bfloat16
                t = [torch.empty((cap, w), dtype=bf, device=self.device) for w in (_HIDDEN, _HIDDEN, _NQ * _D + 2 * _NKV * _D, _NQ * _D, _INTER)]
                self._pf_tensors = t
                self._pf = MqPrefillBuffers(_ptr(t[0]), _ptr(t[1]), _ptr(t[2]), _ptr(t[3]), _ptr(t[4]), cap)
            dev_ids = ids.to(self.device, non_blocking=True)
            logits_ptr = None
            if want_logits:
                if self._logits is None:
                    self._logits = torch.empty(self.vocab_size_, dtype=torch.float32, device=self.device)
                logits_ptr = _ptr(self._logits)
            if audio is not None:
                rc = self._lib.mq_launch_prefill_asr(C.byref(self._model), C.byref(self._buf), C.byref(self._pf), _ptr(dev_ids), n,
                                                     self.position_, _ptr(audio[0]), audio[1], int(audio[0].shape[0]),
                                                     _ptr(self._scalars), logits_ptr, self._stream())
            else:
                rc = self._lib.mq_launch_prefill(C.byref(self._model), C.byref(self._buf), C.byref(self._pf), _ptr(dev_ids), n,
                                                 self.position_, _ptr(self._scalars), logits_ptr, self._stream())
            _lib.check(rc, "mq_launch_prefill")
            self.launches += self._lib.mq_prefill_launch_count(self.num_layers_)
            self.position_ += n
            self._kv8_ready = 0        # the prefill wrote bf16 rows only (bindings_prefill.cpp:831)
            tok, status = self._scalars[:2].tolist()
        self._check_status(status)
        if want_logits:
            return tok, self._logits.clone()
        return tok

    def prefill_step_logits(self, input_ids, append: bool = False):
        """prefill_step (or prefill_append) that also returns the fp32 logits of the last prompt position."""
        ids = torch.as_tensor(input_ids, dtype=torch.int32).reshape(-1)
        self._check_prefill(ids, self.position_ if append else 0)
        if not append:
            self.position_ = 0
        return self._prefill_gemm(ids, want_logits=True)

    def _prefill_by_decode(self, ids: torch.Tensor) -> int:
        """Feed the prompt one position at a time through the decode chain, as
        the reference's decode-only generator does
        (csrc/megakernel/megakernel_generators.py:29-33)."""
        n = int(ids.numel())
        with torch.cuda.device(self.device):
            self._ensure_chain(n)
            self._kv8_sync()
            dev_ids = ids.to(self.device, non_blocking=True)
            tk, ps = self._chain_tokens, self._chain_pos
            _lib.check(self._lib.mq_launch_fill_iota(_ptr(ps), self.position_, n, self._stream()), "mq_launch_fill_iota")
            self.launches += 1
            for i in range(n):
                self._launch(_ptr(dev_ids) + 4 * i, _ptr(self._scalars), _ptr(ps) + 4 * i, None, i > 0)
            self.position_ += n
            self._kv8_ready = self.position_
            tok, status = self._scalars[:2].tolist()
        self._check_status(status)
        return tok


# The reference exports the prefill-capable decoder under a second name with the
# same methods (bindings_prefill.cpp:1637-1701, bindings_fused_prefill.cpp:511-538).
MegakernelPrefillDecoder = MegakernelDecoder
MegakernelFusedPrefillDecoder = MegakernelDecoder
