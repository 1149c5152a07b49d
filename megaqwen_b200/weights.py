"""Weight loading in the reference's dict layout.

``load_qwen3_weights(model_name, max_seq_len)`` returns the dict the
reference's loader returns (csrc/megakernel/megakernel_weights.py:220-505):
``embed_weight, layer_weights (flat, 11 per layer), final_norm_weight,
lm_head_weight, cos_table, sin_table, tokenizer``.  ``model_name`` is either a
local directory holding HF safetensors of a Qwen3 model with the 0.6B block
geometry (single file or sharded with an index, as
megaqwen/safetensors_loader.py:24-83 accepts) or the string
``"synthetic"`` / ``"synthetic-tiny"`` for deterministic random-init weights.
"""
from __future__ import annotations

import json
import os

import torch

from .spec import QWEN3_0_6B, QWEN3_TINY, ModelSpec
from .synthetic import random_weights, rope_tables

_LAYER_KEYS = ["input_layernorm.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight",
               "self_attn.v_proj.weight", "self_attn.q_norm.weight", "self_attn.k_norm.weight",
               "self_attn.o_proj.weight", "post_attention_layernorm.weight", "mlp.gate_proj.weight",
               "mlp.up_proj.weight", "mlp.down_proj.weight"]


def load_tensors(model_dir: str, keys, optional=()) -> dict:
    """Read the named tensors from model.safetensors or from the shards listed in
    model.safetensors.index.json.  A key that the checkpoint does not hold raises
    KeyError (reference: megaqwen/safetensors_loader.py:50-52) unless it is listed
    in ``optional``."""
    from safetensors import safe_open

    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    out = {}
    if os.path.exists(single):
        with safe_open(single, framework="pt", device="cpu") as f:
            names = set(f.keys())
            for k in keys:
                if k in names:
                    out[k] = f.get_tensor(k)
                elif k not in optional:
                    raise KeyError(f"Missing tensor key in safetensors: {k}")
        return out
    if not os.path.exists(index):
        raise FileNotFoundError(f"no model.safetensors or model.safetensors.index.json in {model_dir}")
    with open(index) as fh:
        weight_map = json.load(fh)["weight_map"]
    by_file = {}
    for k in keys:
        if k in weight_map:
            by_file.setdefault(weight_map[k], []).append(k)
        elif k not in optional:
            raise KeyError(f"Missing tensor key in safetensors index: {k}")
    for fname, ks in by_file.items():
        with safe_open(os.path.join(model_dir, fname), framework="pt", device="cpu") as f:
            for k in ks:
                out[k] = f.get_tensor(k)
    return out


def _bf16(t, device):
    return t.to(torch.bfloat16).contiguous().to(device)


def load_qwen3_weights(model_name="Qwen/Qwen3-0.6B", max_seq_len=2048, device="cuda", spec: ModelSpec | None = None, seed: int = 0) -> dict:
    if model_name in ("synthetic", "synthetic-tiny"):
        spec = spec or (QWEN3_TINY if model_name == "synthetic-tiny" else QWEN3_0_6B)
        w = random_weights(spec, max_seq_len, seed=seed, device="cpu")
        w["layer_weights"] = [t.to(device) for t in w["layer_weights"]]
        for k in ("embed_weight", "final_norm_weight", "cos_table", "sin_table"):
            w[k] = w[k].to(device)
        w["lm_head_weight"] = w["embed_weight"]
        w["spec"] = spec
        return w
    if not os.path.isdir(model_name):
        raise FileNotFoundError(
            f"{model_name!r} is not a local directory; this engine loads local safetensors only (no network)")
    with open(os.path.join(model_name, "config.json")) as fh:
        cfg = json.load(fh)
    cfg = cfg.get("text_config", cfg)
    spec = ModelSpec(num_layers=cfg["num_hidden_layers"], vocab_size=cfg["vocab_size"],
                     rms_eps=cfg.get("rms_norm_eps", 1e-6), rope_theta=cfg.get("rope_theta", 1e6))
    geom = (cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
            cfg.get("head_dim", 128))
    if geom != (1024, 3072, 16, 8, 128):
        raise RuntimeError(f"unsupported block geometry {geom}; the kernels are built for (1024, 3072, 16, 8, 128)")
    prefix = "model."
    keys = [prefix + "embed_tokens.weight", prefix + "norm.weight", "lm_head.weight"]
    for l in range(spec.num_layers):
        keys += [f"{prefix}layers.{l}.{k}" for k in _LAYER_KEYS]
    t = load_tensors(model_name, keys, optional=("lm_head.weight",))
    embed = _bf16(t[prefix + "embed_tokens.weight"], device)
    lm_head = embed if "lm_head.weight" not in t or cfg.get("tie_word_embeddings", True) else _bf16(t["lm_head.weight"], device)
    layer_weights = [_bf16(t[f"{prefix}layers.{l}.{k}"], device) for l in range(spec.num_layers) for k in _LAYER_KEYS]
    cos, sin = rope_tables(max_seq_len, spec.rope_theta, spec.head_dim, device)
    tokenizer = None
    try:
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(model_name, local_files_only=True)
    except Exception:
        tokenizer = None
    return {"embed_weight": embed, "layer_weights": layer_weights, "final_norm_weight": _bf16(t[prefix + "norm.weight"], device),
            "lm_head_weight": lm_head, "cos_table": cos, "sin_table": sin, "tokenizer": tokenizer, "spec": spec}
