"""Generate the golden vectors under tests/golden/ from the reference's ground
truth, HuggingFace Qwen3ForCausalLM (bf16, CPU), on the synthetic weights and
prompts of megaqwen_b200.synthetic.  Run from the repository root:

    python tests/golden/make_golden.py [tiny] [cfg1] [cfg2] [cfg3] [cfg4] [cfg5] [selfnoise]

Each .npz holds the prompt, the greedy tokens HF `generate` produced, and the
teacher-forced HF logits of every step: in full (bf16 bit patterns) for the
tiny model; for the full-size model the top-8 values/indices per step and every
64th vocabulary entry.  The batched configurations 4 and 5 are recorded per
sequence (batch 1 each, so no padding enters the numbers): a few of the
batch's prompts, 16 teacher-forced steps each.  ``selfnoise`` records how far
HF's own logits move when the same prompt is fed in one forward or token by
token (the band no implementation can be expected to beat).  Recorded with
transformers 5.5.0 / torch 2.11.0.
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
from megaqwen_b200.spec import QWEN3_0_6B, QWEN3_TINY  # noqa: E402
from megaqwen_b200.synthetic import random_lengths, random_prompt, random_weights  # noqa: E402
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


# sequences of the batched configurations that get a fixture: (index in the batch, prompt length)
CFG4_SEQS = (0, 9, 18, 31)
CFG5_SEQS = (0, 63)
BATCH_STEPS = 16


def run(name, spec, model, cfg_idx, prompt_len, n_new, full, seq_idx=0):
    prompt = random_prompt(spec, prompt_len, cfg_idx, seq_idx)
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
    if any(c in which for c in ("cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "selfnoise")):
        w = random_weights(QWEN3_0_6B, 2304)
        m = build_hf_model(QWEN3_0_6B, w)
        if "cfg1" in which:
            run("full_cfg1_p16_n64", QWEN3_0_6B, m, 1, 16, 64, False)
        if "cfg2" in which:
            run("full_cfg2_p2048_n256", QWEN3_0_6B, m, 2, 2048, 256, False)
        if "cfg3" in which:
            run("full_cfg3_p1024_n32", QWEN3_0_6B, m, 3, 1024, 32, False)
        if "cfg4" in which:
            lens = random_lengths(32, 256, 512)
            for b in CFG4_SEQS:
                run(f"full_cfg4_seq{b}_n{BATCH_STEPS}", QWEN3_0_6B, m, 4, lens[b], BATCH_STEPS, False, seq_idx=b)
        if "cfg5" in which:
            for b in CFG5_SEQS:
                run(f"full_cfg5_seq{b}_n{BATCH_STEPS}", QWEN3_0_6B, m, 5, 1024, BATCH_STEPS, False, seq_idx=b)
        if "selfnoise" in which:
            # HF against itself on config 1: prompt in one forward vs one token at a time
            g = np.load(os.path.join(HERE, "full_cfg1_p16_n64.npz"))
            prompt, tokens = torch.from_numpy(g["prompt"]), g["tokens"].tolist()
            a = hf_step_logits(m, prompt, tokens[:-1])
            b = hf_step_logits(m, prompt, tokens[:-1], token_by_token_prompt=True)
            d = (a - b).abs()
            top = b.topk(8, -1)
            np.savez_compressed(os.path.join(HERE, "full_cfg1_hf_token_by_token.npz"),
                                top_vals=bits(torch.gather(b, 1, torch.from_numpy(g["top_idx"]).long())),
                                strided=bits(b[:, ::STRIDE]), argmax=b.argmax(-1).numpy().astype(np.int32),
                                max_abs=np.float32(d.max()), mean_abs=np.float32(d.mean()),
                                frac_2e2=np.float32((d <= 2e-2).float().mean()))
            print("HF self-noise cfg1: max", float(d.max()), "mean", float(d.mean()),
                  "frac<=2e-2", float((d <= 2e-2).float().mean()),
                  "argmax agree", float((a.argmax(-1) == b.argmax(-1)).float().mean()))


if __name__ == "__main__":
    main(sys.argv[1:] or ["tiny", "cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "selfnoise"])
