"""How far the reference's own ground truth moves under a change that alters no
arithmetic on paper: HF Qwen3ForCausalLM (bf16, CPU) fed the same config-1 prompt
in one forward (the golden fixture) or one token at a time (run here).  Both are
"the oracle"; their distance is the band below which a per-logit bound cannot
separate an implementation error from bf16 re-rounding, and it is what the
tolerances in helpers.py are derived from.
"""
import numpy as np
import torch

from helpers import LOGIT_MAX_TOL, LOGIT_TARGET, GOLDEN, bf16_bits_to_f32, load_golden
from megaqwen_b200.spec import QWEN3_0_6B
from megaqwen_b200.synthetic import random_weights
from oracle.hf_reference import build_hf_model, hf_step_logits


def test_hf_is_not_self_consistent_to_2e2():
    g = load_golden("full_cfg1_p16_n64")
    model = build_hf_model(QWEN3_0_6B, random_weights(QWEN3_0_6B, 128))
    lg = hf_step_logits(model, g["prompt"], g["tokens"][:-1], token_by_token_prompt=True)
    strided = lg[:, ::64]
    top = torch.gather(lg, 1, g["top_idx"])
    d = torch.cat([(strided - g["strided"]).abs().flatten(), (top - g["top_vals"]).abs().flatten()])
    worst, mean, frac = float(d.max()), float(d.mean()), float((d <= LOGIT_TARGET).float().mean())
    agree = float((lg.argmax(-1) == torch.tensor(g["tokens"])).float().mean())
    print(f"HF one-forward vs token-by-token, config 1, 64 steps: max {worst:.4f} mean {mean:.4f} "
          f"within 2e-2 {frac:.4f} arg-max agreement {agree:.4f}")
    # the oracle's own noise exceeds the 2e-2 target (measured 0.047 over all logits, 0.0391 on this subset) ...
    assert worst > LOGIT_TARGET
    assert worst >= 0.035 and mean >= 5e-3 and frac < 0.995
    # ... and the bound the GPU tests use is this band plus a margin, not a multiple of it
    assert LOGIT_MAX_TOL <= 1.5 * worst
    # the run is deterministic: it reproduces the recorded token-by-token logits bit for bit
    z = np.load(GOLDEN + "/full_cfg1_hf_token_by_token.npz")
    assert torch.equal(bf16_bits_to_f32(z["strided"]), strided)
    assert torch.equal(bf16_bits_to_f32(z["top_vals"]), top)
    assert z["argmax"].tolist() == lg.argmax(-1).tolist()
    assert abs(float(z["max_abs"]) - 0.0471) < 1e-3      # over all 151 936 logits per step
