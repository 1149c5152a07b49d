"""Host logic of the generators, the chat entry point and the weight loader,
run on the CPU against a scripted decoder and a small tokenizer (reference:
csrc/megakernel/megakernel_generators.py:12-193, chat.py:425-731,
megaqwen/safetensors_loader.py:24-83)."""
import json
import os

import pytest
import torch


class StubTokenizer:
    """Characters <-> ids; id 1 is EOS and decodes to nothing with skip_special_tokens."""
    eos_token_id = 1

    def encode(self, text, add_special_tokens=True):
        return [2 + (ord(c) % 200) for c in text]

    def decode(self, ids, skip_special_tokens=False):
        return "".join("" if (skip_special_tokens and i == 1) else ("<eos>" if i == 1 else chr(95 + i % 30)) for i in ids)


class ScriptedDecoder:
    """Plays the decoder's part: the next token is a fixed function of the consumed token."""

    def __init__(self, max_seq_len, eos_after=None):
        self.max_seq_len_, self.position_, self.eos_after, self.consumed = max_seq_len, 0, eos_after, []

    def reset(self):
        self.position_, self.consumed = 0, []

    def position(self):
        return self.position_

    def _next(self, t):
        if self.eos_after is not None and len(self.consumed) >= self.eos_after:
            return 1
        return 2 + (7 * t + 3) % 200

    def decode_step(self, t):
        self.consumed.append(int(t))
        self.position_ += 1
        return self._next(int(t))

    def prefill_step(self, ids):
        ids = [int(x) for x in ids]
        self.consumed = list(ids)
        self.position_ = len(ids)
        return self._next(ids[-1])


def make_generator(cls, decoder, max_seq_len, **extra):
    g = object.__new__(cls)
    g.decoder, g.tokenizer, g.max_seq_len = decoder, StubTokenizer(), max_seq_len
    for k, v in extra.items():
        setattr(g, k, v)
    return g


def expected_chain(first, n):
    out, t = [], first
    for _ in range(n):
        t = 2 + (7 * t + 3) % 200
        out.append(t)
    return out


def test_decode_only_generator_feeds_prompt_and_excludes_stop_token():
    from megaqwen_b200.generators import MegakernelGenerator
    dec = ScriptedDecoder(64)
    g = make_generator(MegakernelGenerator, dec, 64)
    ids = g.tokenizer.encode("hello")
    want = expected_chain(ids[-1], 6)
    assert g.generate_ids(ids, 6) == want
    assert dec.consumed[:len(ids)] == ids                     # the whole prompt went through decode_step
    assert g.generate("hello", max_new_tokens=6) == g.tokenizer.decode(want, skip_special_tokens=True)
    assert list(g.generate_stream("hello", max_new_tokens=3)) == [g.tokenizer.decode([t]) for t in want[:3]]
    # an explicit stop token ends the output before it
    assert g.generate_ids(ids, 6, stop_tokens=[want[2]]) == want[:2]
    # the tokenizer's EOS is the default stop token of generate()
    dec2 = ScriptedDecoder(64, eos_after=len(ids) + 2)
    g2 = make_generator(MegakernelGenerator, dec2, 64)
    assert g2.generate("hello", max_new_tokens=6) == g2.tokenizer.decode(want[:2], skip_special_tokens=True)


def test_generators_stop_one_short_of_max_seq_len():
    from megaqwen_b200.generators import MegakernelGenerator, MegakernelPrefillGenerator
    ids = StubTokenizer().encode("abcdef")
    g = make_generator(MegakernelGenerator, ScriptedDecoder(10), 10)
    out = g.generate_ids(ids, 100)
    assert g.decoder.position() == 9 and len(out) == 9 - (len(ids) - 1)
    p = make_generator(MegakernelPrefillGenerator, ScriptedDecoder(10), 10, max_prefill_len=8)
    out = p.generate_ids(ids, 100)
    assert p.decoder.position() == 9 and out[0] == expected_chain(ids[-1], 1)[0]
    with pytest.raises(ValueError, match="exceeds max prefill length"):
        p.generate_ids(list(range(2, 12)), 4)


def test_prefill_generator_first_token_comes_from_prefill():
    from megaqwen_b200.generators import MegakernelPrefillGenerator
    dec = ScriptedDecoder(64)
    p = make_generator(MegakernelPrefillGenerator, dec, 64, max_prefill_len=32)
    ids = p.tokenizer.encode("prompt")
    want = expected_chain(ids[-1], 5)
    assert p.generate_ids(ids, 5) == want
    assert dec.consumed[:len(ids)] == ids and dec.consumed[len(ids):] == want      # like the reference, the last token is also fed
    assert p.generate_ids(ids, 5, stop_tokens=[want[0]]) == []
    nxt, pos = p.prefill_only("prompt")
    assert nxt == want[0] and pos == len(ids)


def test_chat_prompt_template_and_clean_up():
    from megaqwen_b200.chat import build_chat_prompt, clean_response
    conv = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}, {"role": "user", "content": "2+2?"}]
    assert build_chat_prompt(conv) == (
        "<|im_start|>system\nYou are a helpful assistant. Be concise and direct. /nothink<|im_end|>\n"
        "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\nyo<|im_end|>\n<|im_start|>user\n2+2?<|im_end|>\n"
        "<|im_start|>assistant\n")
    assert clean_response(" 4 <|im_end|> trailing") == "4"
    assert clean_response("<think>hm\nhm</think> 4") == "4"
    assert clean_response("4 <think>unfinished") == "4"
    assert clean_response("<think>only") == "[Model is thinking... try asking more directly]"


def test_chat_generation_loop_with_scripted_decoder():
    from megaqwen_b200.chat import MegakernelChat
    chat = object.__new__(MegakernelChat)
    printed = []
    chat.tokenizer, chat.max_seq_len, chat._out = StubTokenizer(), 32, printed.append
    chat.decoder = ScriptedDecoder(32, eos_after=8)
    ids = chat.tokenizer.encode("hello")
    text = chat.generate("hello", max_new_tokens=10, show_speed=False)
    # first token = prediction after the last prompt token; EOS ends the loop and is not shown
    want = expected_chain(ids[-1], 3)
    assert text == chat.tokenizer.decode(want, skip_special_tokens=True)
    assert chat.decoder.consumed[:len(ids)] == ids and not printed
    # a prompt that leaves no room for max_new_tokens is cut from the left
    chat.decoder = ScriptedDecoder(32)
    chat.generate("x" * 40, max_new_tokens=10, show_speed=False)
    assert len(chat.decoder.consumed) >= 21 and chat.decoder.consumed[:21] == chat.tokenizer.encode("x" * 21)
    assert any("truncating" in s for s in printed)
    # interactive loop: one turn, then 'clear', then 'quit'
    chat.max_seq_len = 1024
    chat.decoder = ScriptedDecoder(1024, eos_after=60)
    script = iter(["hi", "clear", "quit"])
    conv = chat.chat(read=lambda _: next(script))
    assert conv == []
    assert any(s.startswith("Assistant: ") for s in printed)


def write_safetensors(path, tensors):
    from safetensors.torch import save_file
    save_file(tensors, path)


def test_load_tensors_single_file_sharded_and_missing_key(tmp_path):
    from megaqwen_b200.weights import load_tensors
    a, b = torch.arange(6, dtype=torch.float32).reshape(2, 3), torch.ones(4, dtype=torch.bfloat16)
    single = tmp_path / "single"
    single.mkdir()
    write_safetensors(str(single / "model.safetensors"), {"a": a, "b": b})
    t = load_tensors(str(single), ["a", "b"])
    assert torch.equal(t["a"], a) and torch.equal(t["b"], b)
    with pytest.raises(KeyError, match="Missing tensor"):
        load_tensors(str(single), ["a", "nope"])
    assert "nope" not in load_tensors(str(single), ["a", "nope"], optional=("nope",))
    shard = tmp_path / "sharded"
    shard.mkdir()
    write_safetensors(str(shard / "model-00001-of-00002.safetensors"), {"a": a})
    write_safetensors(str(shard / "model-00002-of-00002.safetensors"), {"b": b})
    with open(shard / "model.safetensors.index.json", "w") as fh:
        json.dump({"weight_map": {"a": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}}, fh)
    t = load_tensors(str(shard), ["b", "a"])
    assert torch.equal(t["a"], a) and torch.equal(t["b"], b)
    with pytest.raises(KeyError, match="Missing tensor"):
        load_tensors(str(shard), ["c"])
    with pytest.raises(FileNotFoundError):
        load_tensors(str(tmp_path), ["a"])


def test_load_qwen3_weights_from_a_local_checkpoint(tmp_path):
    """A two-layer checkpoint with the 0.6B block geometry written as HF safetensors loads into
    the reference's dict layout (csrc/megakernel/megakernel_weights.py:424-450)."""
    from megaqwen_b200.spec import QWEN3_TINY
    from megaqwen_b200.synthetic import random_weights
    from megaqwen_b200.weights import _LAYER_KEYS, load_qwen3_weights
    w = random_weights(QWEN3_TINY, 64)
    sd = {"model.embed_tokens.weight": w["embed_weight"], "model.norm.weight": w["final_norm_weight"]}
    for l in range(2):
        for j, k in enumerate(_LAYER_KEYS):
            sd[f"model.layers.{l}.{k}"] = w["layer_weights"][11 * l + j]
    write_safetensors(str(tmp_path / "model.safetensors"), {k: v.contiguous() for k, v in sd.items()})
    with open(tmp_path / "config.json", "w") as fh:
        json.dump({"num_hidden_layers": 2, "vocab_size": 4096, "hidden_size": 1024, "intermediate_size": 3072,
                   "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6,
                   "rope_theta": 1e6, "tie_word_embeddings": True}, fh)
    got = load_qwen3_weights(str(tmp_path), max_seq_len=64, device="cpu")
    assert set(got) >= {"embed_weight", "layer_weights", "final_norm_weight", "lm_head_weight", "cos_table", "sin_table", "tokenizer"}
    assert len(got["layer_weights"]) == 22 and got["lm_head_weight"] is got["embed_weight"]
    assert all(torch.equal(x, y) for x, y in zip(got["layer_weights"], w["layer_weights"]))
    assert torch.equal(got["cos_table"], w["cos_table"]) and torch.equal(got["sin_table"], w["sin_table"])
    os.remove(tmp_path / "config.json")
    with pytest.raises(FileNotFoundError):
        load_qwen3_weights(str(tmp_path), max_seq_len=64, device="cpu")
