"""Pin the CPU restatement (oracle/qwen3_restatement.py) to the golden vectors
recorded from the reference's ground truth (HF Qwen3ForCausalLM bf16 on CPU,
tests/golden/make_golden.py)."""
import pytest
import torch

from helpers import assert_logits_close, assert_tokens_match, load_golden
from megaqwen_b200.spec import QWEN3_0_6B, QWEN3_TINY
from megaqwen_b200.synthetic import random_prompt, random_weights
from oracle.qwen3_restatement import RestatedQwen3


def margins(g):
    return (g["top_vals"][:, 0] - g["top_vals"][:, 1]).tolist()


@pytest.mark.parametrize("name,cfg,plen", [("tiny_p16_n32", 1, 16), ("tiny_p300_n24", 2, 300)])
def test_restatement_matches_hf_golden_tiny(name, cfg, plen):
    g = load_golden(name)
    assert torch.equal(g["prompt"], random_prompt(QWEN3_TINY, plen, cfg, 0))
    w = random_weights(QWEN3_TINY, 2304)
    r = RestatedQwen3(QWEN3_TINY, w, 512)
    lg = r.step_logits(g["prompt"], g["tokens"][:-1])
    assert_logits_close(lg, g["logits"], name)
    assert_tokens_match(lg.argmax(-1).tolist(), g["tokens"], margins(g), name)
    # decode-style feeding (one token at a time) stays inside the same band
    lg2 = r.step_logits(g["prompt"], g["tokens"][:-1], token_by_token_prompt=True)
    assert_logits_close(lg2, g["logits"], name + " token-by-token")


def test_restatement_matches_hf_golden_full_cfg1():
    g = load_golden("full_cfg1_p16_n64")
    w = random_weights(QWEN3_0_6B, 2304)
    r = RestatedQwen3(QWEN3_0_6B, w, 128)
    lg = r.step_logits(g["prompt"], g["tokens"][:-1])
    assert_logits_close(lg[:, ::64], g["strided"], "full cfg1 strided logits")
    got_top = torch.gather(lg, 1, g["top_idx"])
    assert_logits_close(got_top, g["top_vals"], "full cfg1 top-8 logits")
    assert_tokens_match(lg.argmax(-1).tolist(), g["tokens"], margins(g), "full cfg1")


def test_golden_files_are_self_consistent():
    for name in ("tiny_p16_n32", "tiny_p300_n24", "full_cfg1_p16_n64", "full_cfg2_p2048_n256", "full_cfg3_p1024_n32"):
        g = load_golden(name)
        # the greedy token carries the maximum logit (ties: any index holding it)
        for i, t in enumerate(g["tokens"]):
            holders = g["top_idx"][i][g["top_vals"][i] == g["top_vals"][i, 0]].tolist()
            assert t in holders, (name, i)
        assert (g["top_vals"][:, 0] >= g["top_vals"][:, 1]).all()
