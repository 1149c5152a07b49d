"""Host-side logic that needs no GPU: byte model, synthetic inputs, errors."""
import pytest
import torch

from megaqwen_b200.spec import QWEN3_0_6B, QWEN3_TINY
from megaqwen_b200.synthetic import random_lengths, random_prompt, random_weights, rope_tables


def test_decode_byte_model():
    # weights 1 192 101 888 B, 114 688 B of K+V per cached position
    assert QWEN3_0_6B.weight_bytes() == 1_192_101_888
    assert QWEN3_0_6B.kv_bytes_per_position() == 114_688
    assert QWEN3_0_6B.decode_bytes(2048) == 1_192_101_888 + 114_688 * 2049
    assert abs(QWEN3_0_6B.prefill_flops(1024) / 1e12 - 1.0225) < 2e-3


def test_synthetic_weights_are_deterministic_and_laid_out_like_the_reference():
    a = random_weights(QWEN3_TINY, 64)
    b = random_weights(QWEN3_TINY, 64)
    assert len(a["layer_weights"]) == 11 * QWEN3_TINY.num_layers
    assert a["lm_head_weight"] is a["embed_weight"]
    for x, y in zip(a["layer_weights"], b["layer_weights"]):
        assert torch.equal(x, y)
    shapes = [tuple(t.shape) for t in a["layer_weights"][:11]]
    assert shapes == [(1024,), (2048, 1024), (1024, 1024), (1024, 1024), (128,), (128,), (1024, 2048), (1024,),
                      (3072, 1024), (3072, 1024), (1024, 3072)]
    assert all(t.dtype == torch.bfloat16 for t in a["layer_weights"])
    assert float(a["layer_weights"][0].float().min()) == 1.0
    std = float(a["layer_weights"][1].float().std())
    assert 0.019 < std < 0.021


def test_prompts_and_lengths():
    p = random_prompt(QWEN3_0_6B, 2048, 2, 0)
    assert p.dtype == torch.int32 and p.numel() == 2048 and int(p.max()) < 151936 and int(p.min()) >= 0
    assert torch.equal(p, random_prompt(QWEN3_0_6B, 2048, 2, 0))
    assert not torch.equal(p, random_prompt(QWEN3_0_6B, 2048, 2, 1))
    ls = random_lengths(32, 256, 512)
    assert len(ls) == 32 and min(ls) >= 256 and max(ls) <= 512


def test_rope_tables_duplicate_halves():
    cos, sin = rope_tables(32, 1e6, 128)
    assert cos.shape == (32, 128) and cos.dtype == torch.bfloat16
    assert torch.equal(cos[:, :64], cos[:, 64:]) and torch.equal(sin[:, :64], sin[:, 64:])
    assert float(cos[0, 0]) == 1.0 and float(sin[0, 0]) == 0.0


def test_decoder_refuses_to_run_without_cuda():
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    from megaqwen_b200.decoder import MegakernelDecoder
    w = random_weights(QWEN3_TINY, 64)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        MegakernelDecoder(w["embed_weight"], w["layer_weights"], w["final_norm_weight"], w["lm_head_weight"],
                          w["cos_table"], w["sin_table"], 2, 64)
