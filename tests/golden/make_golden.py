"""Generate the golden vectors under tests/golden/ from the reference's ground
truth, HuggingFace Qwen3ForCausalLM (bf16, CPU), on the synthetic weights and
prompts of megaqwen_b200.synthetic.  Run from the repository root:

    python tests/golden/make_golden.py [tiny] [cfg1] [cfg2] [cfg3]

Each .npz holds the prompt, the greedy tokens HF `generate` produced, and the
teacher-forced HF logits of every step: in full (bf16 bit patterns) for the
tiny model; for the full-size model the top-8 values/indices per step and every
64th vocabulary entry.  Recorded with transformers 5.5.0 / torch 2.11.0.
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
from megaqwen_b200.spec import QWEN3_0_6B, QWEN3_TINY  # noqa: E402
from megaqwen_b200.synthetic import random_prompt, random_weights  # noqa: E402
from oracle.hf_reference import build_hf_model, hf_generate, hf_step_logits  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
STRIDE = 64


def bits(t):
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def pack(name, spec, prompt, tokens, logits, full):
    top = logits.topk(8, -1)
    d = dict(prompt=prompt.numpy().astype(np.int32), tokens=np.asarray(tokens, dtype=np.int32),
             top_vals=bits(top.values), top_idx=top.indices.numpy().astype(np.int32),
             num_layers=spec.num_layers, vocab=spec.vocab_size)
    if full:
        d["logits"] = bits(logits)
    else:
        d["strided"] = bits(logits[:, ::STRIDE])
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **d)
    print(name, "saved", len(tokens), "tokens")


def run(name, spec, model, cfg_idx, prompt_len, n_new, full):
    prompt = random_prompt(spec, prompt_len, cfg_idx, 0)
    tokens = hf_generate(model, prompt, n_new)
    logits = hf_step_logits(model, prompt, tokens[:-1])
    assert logits.argmax(-1).tolist() == tokens, "teacher-forced HF run must reproduce generate()"
    pack(name, spec, prompt, tokens, logits, full)


def main(which):
    torch.manual_seed(0)
    if "tiny" in which:
        w = random_weights(QWEN3_TINY, 2304)
        m = build_hf_model(QWEN3_TINY, w)
        run("tiny_p16_n32", QWEN3_TINY, m, 1, 16, 32, True)
        run("tiny_p300_n24", QWEN3_TINY, m, 2, 300, 24, True)
    if any(c in which for c in ("cfg1", "cfg2", "cfg3")):
        w = random_weights(QWEN3_0_6B, 2304)
        m = build_hf_model(QWEN3_0_6B, w)
        if "cfg1" in which:
            run("full_cfg1_p16_n64", QWEN3_0_6B, m, 1, 16, 64, False)
        if "cfg2" in which:
            run("full_cfg2_p2048_n256", QWEN3_0_6B, m, 2, 2048, 256, False)
        if "cfg3" in which:
            run("full_cfg3_p1024_n32", QWEN3_0_6B, m, 3, 1024, 32, False)


if __name__ == "__main__":
    main(sys.argv[1:] or ["tiny", "cfg1", "cfg2", "cfg3"])
