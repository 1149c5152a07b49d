"""Chat entry point on top of the decoder: the counterpart of the reference's
``MegakernelChat`` (chat.py:425-731) with the same three calls,
``generate(prompt, max_new_tokens, show_speed)``, ``generate_stream(prompt,
max_new_tokens)`` and the interactive ``chat()`` loop, the same ChatML prompt
with the ``/nothink`` system line (chat.py:700-706) and the same clean-up of
the answer (chat.py:716-726).

Semantics kept from the reference: the KV cache is reset for every prompt;
a prompt that leaves no room for ``max_new_tokens`` is cut from the left
(chat.py:438-441); the first generated token is the prediction after the last
prompt token (chat.py:447-479); generation stops after the EOS token, which is
kept in the id list and removed by ``skip_special_tokens`` when decoding.
The prompt goes through the tcgen05 prefill instead of one decode launch per
prompt token.

    python -m megaqwen_b200.chat <model_dir> [max_seq_len]
"""
from __future__ import annotations

import re
import sys
import time

import torch

from .decoder import MegakernelDecoder
from .weights import load_qwen3_weights

SYSTEM_LINE = "You are a helpful assistant. Be concise and direct. /nothink"


def build_chat_prompt(conversation) -> str:
    """ChatML prompt of a list of {"role", "content"} turns, ending with an open assistant turn."""
    parts = [f"<|im_start|>system\n{SYSTEM_LINE}<|im_end|>\n"]
    for msg in conversation:
        role = "user" if msg["role"] == "user" else "assistant"
        parts.append(f"<|im_start|>{role}\n{msg['content']}<|im_end|>\n")
    parts.append("<|im_start|>assistant\n")
    return "".join(parts)


def clean_response(text: str) -> str:
    """Cut at the end-of-turn marker and drop <think> blocks, closed or not."""
    text = text.split("<|im_end|>")[0].strip()
    text = re.sub(r"<think>.*?</think>", "", text, flags=re.DOTALL).strip()
    if "<think>" in text:
        text = text.split("<think>")[0].strip()
    return text or "[Model is thinking... try asking more directly]"


class MegakernelChat:
    def __init__(self, model_name="Qwen/Qwen3-0.6B", max_seq_len=2048, weights=None, device="cuda", out=None):
        weights = weights or load_qwen3_weights(model_name, max_seq_len=max_seq_len, device=device)
        self.tokenizer = weights["tokenizer"]
        if self.tokenizer is None:
            raise RuntimeError("MegakernelChat needs a tokenizer (none was found beside the weights)")
        self.max_seq_len = int(max_seq_len)
        self.decoder = MegakernelDecoder(
            weights["embed_weight"], weights["layer_weights"], weights["final_norm_weight"], weights["lm_head_weight"],
            weights["cos_table"], weights["sin_table"], len(weights["layer_weights"]) // 11, self.max_seq_len,
            self.max_seq_len)
        self._out = out or (lambda s: (sys.stdout.write(s), sys.stdout.flush()))

    # ------------------------------------------------------------------ generation
    def _prompt_ids(self, prompt: str, max_new_tokens: int):
        ids = list(self.tokenizer.encode(prompt))
        if len(ids) >= self.max_seq_len - max_new_tokens:
            self._out(f"Warning: prompt too long ({len(ids)} tokens), truncating\n")
            ids = ids[-max(1, self.max_seq_len - max_new_tokens - 1):]
        return ids

    def _run(self, prompt: str, max_new_tokens: int, stream: bool, show_speed: bool) -> str:
        ids = self._prompt_ids(prompt, max_new_tokens)
        eos = self.tokenizer.eos_token_id
        dec = self.decoder
        dec.reset()
        t0 = time.perf_counter()
        cur = dec.prefill_step(torch.tensor(ids, dtype=torch.int32))
        t1 = time.perf_counter()
        generated = [cur]
        if stream:
            self._out(self.tokenizer.decode([cur], skip_special_tokens=True))
        for _ in range(max_new_tokens - 1):
            if cur == eos or dec.position() >= self.max_seq_len - 1:
                break
            cur = dec.decode_step(cur)
            generated.append(cur)
            if stream:
                self._out(self.tokenizer.decode([cur], skip_special_tokens=True))
        t2 = time.perf_counter()
        if show_speed:
            self._out(f"\n[prefill: {len(ids)} tok @ {len(ids) / max(t1 - t0, 1e-9):.0f} tok/s | "
                      f"decode: {len(generated)} tok @ {len(generated) / max(t2 - t1, 1e-9):.0f} tok/s | "
                      f"total: {(t2 - t0) * 1e3:.0f}ms]\n")
        return self.tokenizer.decode(generated, skip_special_tokens=True)

    def generate(self, prompt: str, max_new_tokens: int = 100, show_speed: bool = True) -> str:
        return self._run(prompt, max_new_tokens, False, show_speed)

    def generate_stream(self, prompt: str, max_new_tokens: int = 100) -> str:
        """Prints every token as soon as it is decoded and returns the whole answer."""
        return self._run(prompt, max_new_tokens, True, True)

    # ------------------------------------------------------------------ interactive loop
    def chat(self, read=input):
        self._out("\n" + "=" * 60 + "\nQwen3-0.6B Chat (megaqwen_b200, sm_100a kernels)\n" + "=" * 60 + "\n"
                  "Type 'quit' or 'exit' to end the conversation.\nType 'clear' to start a new conversation.\n"
                  + "=" * 60 + "\n\n")
        conversation = []
        while True:
            try:
                user = read("You: ").strip()
            except (KeyboardInterrupt, EOFError):
                self._out("\nGoodbye!\n")
                break
            if not user:
                continue
            if user.lower() in ("quit", "exit"):
                self._out("Goodbye!\n")
                break
            if user.lower() == "clear":
                conversation = []
                self._out("\n[Conversation cleared]\n\n")
                continue
            conversation.append({"role": "user", "content": user})
            self._out("Assistant: ")
            answer = clean_response(self.generate_stream(build_chat_prompt(conversation), max_new_tokens=500))
            self._out(answer + "\n\n")
            conversation.append({"role": "assistant", "content": answer})
        return conversation


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if not argv:
        raise SystemExit("usage: python -m megaqwen_b200.chat <model_dir> [max_seq_len]")
    MegakernelChat(argv[0], int(argv[1]) if len(argv) > 1 else 2048).chat()


if __name__ == "__main__":
    main()
