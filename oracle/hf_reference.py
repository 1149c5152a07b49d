"""The reference's ground truth: HuggingFace ``Qwen3ForCausalLM`` in bf16 on CPU.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

The reference checks its CUDA path against ``AutoModelForCausalLM`` greedy
generation (verify_correctness.py:11-34, benchmark_suite.py:48-69,
experiments/framework_bench/quality_metrics.py:109-133).  The arithmetic lives
in the third-party ``transformers`` package (requirements.txt:2 pins only
``transformers>=4.40.0``; this image has 5.5.0), which is not vendored in the
reference tree.  This module builds that model from a weight dict in the
reference's layout (csrc/megakernel/megakernel_weights.py:109-128) instead of a
checkpoint and runs it exactly as those scripts do, on the host cores.
"""
from __future__ import annotations

import time

import torch


def build_hf_model(spec, weights: dict):
    """Qwen3ForCausalLM (bf16, eval, CPU) holding ``weights``."""
    from transformers import Qwen3Config, Qwen3ForCausalLM

    cfg = Qwen3Config(
        vocab_size=spec.vocab_size,
        hidden_size=spec.hidden_size,
        intermediate_size=spec.intermediate_size,
        num_hidden_layers=spec.num_layers,
        num_attention_heads=spec.num_q_heads,
        num_key_value_heads=spec.num_kv_heads,
        head_dim=spec.head_dim,
        rms_norm_eps=spec.rms_eps,
        rope_theta=spec.rope_theta,
        rope_parameters={"rope_type": "default", "rope_theta": spec.rope_theta},
        max_position_embeddings=40960,
        tie_word_embeddings=True,
        attention_bias=False,
        use_sliding_window=False,
    )
    with torch.device("meta"):
        model = Qwen3ForCausalLM(cfg)
    sd = {"model.embed_tokens.weight": weights["embed_weight"].cpu(),
          "model.norm.weight": weights["final_norm_weight"].cpu(),
          "lm_head.weight": weights["embed_weight"].cpu()}
    names = ["input_layernorm", "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj",
             "self_attn.q_norm", "self_attn.k_norm", "self_attn.o_proj",
             "post_attention_layernorm", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"]
    flat = weights["layer_weights"]
    for layer in range(spec.num_layers):
        for j, n in enumerate(names):
            sd[f"model.layers.{layer}.{n}.weight"] = flat[11 * layer + j].cpu()
    missing, unexpected = model.load_state_dict(sd, strict=False, assign=True)
    assert not unexpected, unexpected
    assert all("rotary" in m or "inv_freq" in m for m in missing), missing
    model.tie_weights()
    model = model.to(torch.bfloat16).eval()
    # The rotary inv_freq buffer was created on the meta device and needs real
    # storage; it must stay fp32 as it does under from_pretrained(dtype=bf16)
    # (a module-wide .to(bf16) would round the frequencies), so it is rebuilt
    # after the cast.
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RotaryEmbedding
    model.model.rotary_emb = Qwen3RotaryEmbedding(cfg)
    assert model.model.rotary_emb.inv_freq.dtype == torch.float32
    assert model.lm_head.weight.data_ptr() == model.model.embed_tokens.weight.data_ptr()
    return model


@torch.no_grad()
def hf_generate(model, prompt_ids, max_new_tokens: int):
    """Greedy ``generate`` exactly as the reference scripts call it; returns the
    new token ids (list of int)."""
    ids = torch.as_tensor(prompt_ids, dtype=torch.long).view(1, -1)
    out = model.generate(ids, max_new_tokens=max_new_tokens, min_new_tokens=max_new_tokens,
                         do_sample=False, use_cache=True,
                         pad_token_id=0, eos_token_id=None)
    return out[0, ids.shape[1]:].tolist()


@torch.no_grad()
def hf_step_logits(model, prompt_ids, forced_tokens, token_by_token_prompt: bool = False):
    """Teacher-forced run: feed the prompt (one forward, or one token at a time
    as the reference's decode-only generator does,
    csrc/megakernel/megakernel_generators.py:29-46), then ``forced_tokens`` one
    at a time.  Returns fp32 logits [1 + len(forced_tokens), V]: row 0 follows
    the prompt, row i follows forced_tokens[i-1]."""
    from transformers import DynamicCache

    cache = DynamicCache(config=model.config)
    ids = torch.as_tensor(prompt_ids, dtype=torch.long).view(1, -1)
    rows = []
    if token_by_token_prompt:
        for i in range(ids.shape[1]):
            out = model(input_ids=ids[:, i:i + 1], past_key_values=cache, use_cache=True)
    else:
        out = model(input_ids=ids, past_key_values=cache, use_cache=True)
    rows.append(out.logits[0, -1].float())
    for t in forced_tokens:
        out = model(input_ids=torch.tensor([[int(t)]]), past_key_values=cache, use_cache=True)
        rows.append(out.logits[0, -1].float())
    return torch.stack(rows)


@torch.no_grad()
def time_hf_decode(model, prompt_ids, max_new_tokens: int):
    """(decode tok/s, prefill seconds).  The prompt goes through one forward into a
    DynamicCache (timed: the prefill), then ``max_new_tokens`` greedy single-token
    forwards are timed directly, which is the loop ``generate`` runs for the reference's
    scripts (benchmark_suite.py:48-69) without subtracting two nearly equal durations."""
    from transformers import DynamicCache

    ids = torch.as_tensor(prompt_ids, dtype=torch.long).view(1, -1)
    cache = DynamicCache(config=model.config)
    t0 = time.perf_counter()
    out = model(input_ids=ids, past_key_values=cache, use_cache=True)
    tok = out.logits[0, -1].argmax().view(1, 1)
    t1 = time.perf_counter()
    for _ in range(max_new_tokens):
        out = model(input_ids=tok, past_key_values=cache, use_cache=True)
        tok = out.logits[0, -1].argmax().view(1, 1)
    t2 = time.perf_counter()
    return max_new_tokens / max(t2 - t1, 1e-9), t1 - t0
