"""Generators with the reference's entry points
(csrc/megakernel/megakernel_generators.py:12-193): ``generate`` /
``generate_stream`` on strings through the tokenizer, plus ``generate_ids`` on
token ids (no tokenizer files exist offline, so the id-level entry is what the
tests and the benchmark drive).
"""
from __future__ import annotations

import torch

from .decoder import MegakernelDecoder
from .weights import load_qwen3_weights


class MegakernelGenerator:
    """Decode-only generator: the prompt is fed one token at a time through
    ``decode_step`` (reference: megakernel_generators.py:12-63).  Greedy;
    ``temperature`` is accepted and ignored, as in the reference."""

    def __init__(self, model_name="Qwen/Qwen3-0.6B", max_seq_len=2048, weights=None, device="cuda"):
        weights = weights or load_qwen3_weights(model_name, max_seq_len=max_seq_len, device=device)
        self.decoder = MegakernelDecoder(
            weights["embed_weight"], weights["layer_weights"], weights["final_norm_weight"],
            weights["lm_head_weight"], weights["cos_table"], weights["sin_table"],
            len(weights["layer_weights"]) // 11, max_seq_len, max_seq_len)
        self.tokenizer = weights.get("tokenizer")
        self.max_seq_len = max_seq_len

    def _stops(self, stop_tokens):
        if stop_tokens is not None:
            return list(stop_tokens)
        if self.tokenizer is not None and self.tokenizer.eos_token_id is not None:
            return [self.tokenizer.eos_token_id]
        return []

    def _feed_prompt(self, input_ids):
        for token_id in input_ids[:-1]:
            self.decoder.decode_step(int(token_id))
        return int(input_ids[-1])

    def _iter_ids(self, input_ids, max_new_tokens, stop_tokens):
        self.decoder.reset()
        current = self._feed_prompt(list(input_ids))
        for _ in range(max_new_tokens):
            nxt = self.decoder.decode_step(current)
            if nxt in stop_tokens:
                break
            yield nxt
            current = nxt
            if self.decoder.position() >= self.max_seq_len - 1:
                break

    def generate_ids(self, input_ids, max_new_tokens=100, stop_tokens=None):
        return list(self._iter_ids(input_ids, max_new_tokens, stop_tokens or []))

    def generate(self, prompt, max_new_tokens=100, temperature=1.0, stop_tokens=None):
        ids = self.tokenizer.encode(prompt, add_special_tokens=True)
        out = list(self._iter_ids(ids, max_new_tokens, self._stops(stop_tokens)))
        return self.tokenizer.decode(out, skip_special_tokens=True)

    def generate_stream(self, prompt, max_new_tokens=100, stop_tokens=None):
        ids = self.tokenizer.encode(prompt, add_special_tokens=True)
        for t in self._iter_ids(ids, max_new_tokens, self._stops(stop_tokens)):
            yield self.tokenizer.decode([t])


class MegakernelPrefillGenerator(MegakernelGenerator):
    """Prefill + decode generator (reference: megakernel_generators.py:66-128).
    The stop token is excluded from the output; the first generated token is the
    one ``prefill_step`` returns."""

    def __init__(self, model_name="Qwen/Qwen3-0.6B", max_seq_len=2048, max_prefill_len=512, weights=None, device="cuda"):
        super().__init__(model_name, max_seq_len, weights=weights, device=device)
        self.decoder.max_prefill_len_ = max_prefill_len
        self.max_prefill_len = max_prefill_len

    def _check_len(self, input_ids):
        if len(input_ids) > self.max_prefill_len:
            raise ValueError(f"Prompt length {len(input_ids)} exceeds max prefill length {self.max_prefill_len}")
        return input_ids

    def _iter_ids(self, input_ids, max_new_tokens, stop_tokens):
        self.decoder.reset()
        ids = self._check_len(list(input_ids))
        nxt = self.decoder.prefill_step(torch.tensor(ids, dtype=torch.int32))
        for _ in range(max_new_tokens):
            if nxt in stop_tokens:
                break
            yield nxt
            if self.decoder.position() >= self.max_seq_len - 1:
                break
            nxt = self.decoder.decode_step(nxt)

    def generate_ids_fast(self, input_ids, max_new_tokens=100):
        """Prefill, then one device-resident greedy chain with a single read of
        the result (reference: decode_greedy_cuda, bindings_prefill.cpp:1159-1349).
        Returns a list of max_new_tokens ids."""
        self.decoder.reset()
        ids = self._check_len(list(input_ids))
        first = self.decoder.prefill_step(torch.tensor(ids, dtype=torch.int32))
        if max_new_tokens <= 1:
            return [first][:max_new_tokens]
        rest = self.decoder.decode_steps(first, max_new_tokens - 1)
        return [first] + rest.tolist()

    def prefill_only(self, prompt):
        self.decoder.reset()
        ids = self._check_len(self.tokenizer.encode(prompt, add_special_tokens=True))
        nxt = self.decoder.prefill_step(torch.tensor(ids, dtype=torch.int32))
        return nxt, self.decoder.position()


MegakernelFusedPrefillGenerator = MegakernelPrefillGenerator
