"""State-dict key map between this package's checkpoints and the HuggingFace ``Imu1ForCausalLM`` layout.

Same names as the reference converters use (scripts/hf/convert_imu1_checkpoint.py:163-264), expressed as one table
so that both directions come from a single source.  ``lm_head.weight`` (the inert alias stored when ``weight_tying``
is set) is dropped on the way out and re-created on the way back; ``position_scale`` and RoPE cache buffers of the
HF model are ignored on the way back.
"""

from __future__ import annotations

import re
from typing import Any

import torch

TOP_LEVEL = {
    "embedding.weight": "model.embed_tokens.weight",
    "final_norm.gain": "model.norm.weight",
    "lm_head.linear.weight": "lm_head.weight",
}
PER_LAYER = {
    "ln1.gain": "input_layernorm.weight",
    "ln2.gain": "post_attention_layernorm.weight",
    "attn.qkv.linear.weight": "self_attn.qkv_proj.weight",
    "attn.out.linear.weight": "self_attn.o_proj.weight",
    "attn.attn_gate.linear.weight": "self_attn.attn_gate.weight",
    "attn.sdpa_qknorm.gain": "self_attn.qk_norm.gain",
    "attn.alpha1": "self_attn.alpha1",
    "attn.alpha2": "self_attn.alpha2",
    "attn.scale": "self_attn.value_scale",
    "ffn.up.linear.weight": "mlp.up_proj.weight",
    "ffn.down.linear.weight": "mlp.down_proj.weight",
}
_PER_LAYER_REV = {v: k for k, v in PER_LAYER.items()}
_PER_LAYER_REV.update({"input_layernorm.rms_norm.weight": "ln1.gain", "post_attention_layernorm.rms_norm.weight": "ln2.gain"})
_TOP_REV = {v: k for k, v in TOP_LEVEL.items()}
_IGNORED_HF = re.compile(r"(position_scale|rotary_emb\.(cos|sin)_cached|inv_freq)$")


def rename_to_hf(name: str) -> str | None:
    if name == "lm_head.weight":
        return None
    if name in TOP_LEVEL:
        return TOP_LEVEL[name]
    m = re.match(r"blocks\.(\d+)\.(.+)$", name)
    if m and m.group(2) in PER_LAYER:
        return f"model.layers.{m.group(1)}.{PER_LAYER[m.group(2)]}"
    raise KeyError(f"Unhandled parameter name: {name}")


def to_hf_state_dict(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        nk = rename_to_hf(k)
        if nk is not None:
            out[nk] = v
    return out


def from_hf_state_dict(sd: dict[str, torch.Tensor], weight_tying_alias: bool = True) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    for k, v in sd.items():
        if _IGNORED_HF.search(k):
            continue
        if k in _TOP_REV:
            out[_TOP_REV[k]] = v
            continue
        m = re.match(r"model\.layers\.(\d+)\.(.+)$", k)
        if m and m.group(2) in _PER_LAYER_REV:
            out[f"blocks.{m.group(1)}.{_PER_LAYER_REV[m.group(2)]}"] = v
            continue
        raise KeyError(f"Unhandled converted key: {k}")
    if weight_tying_alias and "embedding.weight" in out:
        out["lm_head.weight"] = out["embedding.weight"]
    return out


def ordered_native_state_dict(sd: dict[str, torch.Tensor], n_layers: int) -> dict[str, torch.Tensor]:
    """Keys in the module-tree order of ``models.Transformer`` (what ``load_state_dict`` and readers expect)."""
    order = ["embedding.weight"]
    per = ["ln1.gain", "attn.alpha1", "attn.alpha2", "attn.scale", "attn.qkv.linear.weight", "attn.out.linear.weight",
           "attn.sdpa_qknorm.gain", "attn.attn_gate.linear.weight", "ln2.gain", "ffn.up.linear.weight", "ffn.down.linear.weight"]
    for i in range(n_layers):
        order += [f"blocks.{i}.{s}" for s in per]
    order += ["final_norm.gain", "lm_head.weight", "lm_head.linear.weight"]
    return {k: sd[k] for k in order if k in sd}


def hf_config_dict(cfg: dict[str, Any], bos_id=None, eos_id=256, pad_id=None, tie_word_embeddings=None) -> dict[str, Any]:
    """``config.json`` of the HF model from the checkpoint's config (dict form)."""
    m, d = cfg["model"], cfg.get("data", {})
    return {
        "architectures": ["Imu1ForCausalLM"],
        "model_type": "imu_1",
        "vocab_size": m["vocab_size"],
        "hidden_size": m["d_model"],
        "intermediate_size": m["d_ff"],
        "num_hidden_layers": m["n_layers"],
        "num_attention_heads": m["n_heads"],
        "num_key_value_heads": m.get("n_kv_heads") or m["n_heads"],
        "hidden_act": "silu",
        "max_position_embeddings": max(8192, d.get("context_length", 0), m.get("max_seq_len", 0)),
        "rms_norm_eps": 1e-5,
        "rope_theta": m.get("theta", 10000),
        "attn_qknorm": m.get("attn_qknorm", True),
        "attn_val_residual": m.get("attn_val_residual", True),
        "attn_gating": m.get("attn_gating", False),
        "layernorm_scaling": m.get("layernorm_scaling", False),
        "tie_word_embeddings": m.get("weight_tying", False) if tie_word_embeddings is None else tie_word_embeddings,
        "pad_token_id": d.get("pad_token_id", pad_id),
        "bos_token_id": bos_id,
        "eos_token_id": eos_id,
        "torch_dtype": "float32",
    }


def native_model_config(hf: dict[str, Any]) -> dict[str, Any]:
    """Minimal ``model`` section of a native config from an HF ``config.json``."""
    return {
        "vocab_size": hf["vocab_size"], "d_model": hf["hidden_size"], "d_ff": hf["intermediate_size"],
        "n_layers": hf["num_hidden_layers"], "n_heads": hf["num_attention_heads"],
        "n_kv_heads": hf.get("num_key_value_heads", hf["num_attention_heads"]), "theta": hf.get("rope_theta", 10000),
        "weight_tying": hf.get("tie_word_embeddings", False), "attn_qknorm": hf.get("attn_qknorm", False),
        "attn_val_residual": hf.get("attn_val_residual", False), "attn_gating": hf.get("attn_gating", False),
        "layernorm_scaling": hf.get("layernorm_scaling", False),
    }
