"""HuggingFace ``Imu1ForCausalLM`` directory -> native ``.pt`` checkpoint (``iteration: 0``, no optimizer state).
Counterpart of scripts/hf/convert_hf_to_imu.py of the reference."""

from __future__ import annotations

import json
from argparse import ArgumentParser
from pathlib import Path

import torch

from sample_efficient_gpt_b200.scripts.hf.keymap import from_hf_state_dict, native_model_config, ordered_native_state_dict


def load_hf_state_dict(model_dir: Path) -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    sd: dict[str, torch.Tensor] = {}
    files = sorted(model_dir.glob("*.safetensors"))
    if files:
        for f in files:
            sd.update(load_file(str(f)))
        return sd
    for f in sorted(model_dir.glob("pytorch_model*.bin")):
        sd.update(torch.load(f, map_location="cpu", weights_only=True))
    if not sd:
        raise FileNotFoundError(f"no weights under {model_dir}")
    return sd


def convert(model_dir, out_path, context_length: int = 1024) -> Path:
    from sample_efficient_gpt_b200.config_schema import default_cfg
    from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, save_config

    model_dir = Path(model_dir)
    hf_cfg = json.loads((model_dir / "config.json").read_text())
    mcfg = native_model_config(hf_cfg)
    hf_sd = load_hf_state_dict(model_dir)
    if "lm_head.weight" not in hf_sd and hf_cfg.get("tie_word_embeddings"):
        hf_sd["lm_head.weight"] = hf_sd["model.embed_tokens.weight"].clone()
    sd = from_hf_state_dict({k: v.float() for k, v in hf_sd.items()}, weight_tying_alias=mcfg["weight_tying"])
    sd = ordered_native_state_dict(sd, mcfg["n_layers"])
    cfg = apply_overrides(default_cfg, {f"model.{k}": v for k, v in mcfg.items()})
    cfg = apply_overrides(cfg, {"data.context_length": context_length})
    out_path = Path(out_path)
    out_path.parent.mkdir(parents=True, exist_ok=True)
    torch.save({"config": save_config(cfg), "model": sd, "optimizer": None, "iteration": 0, "run_id": None,
                "hf_metadata": {"source": str(model_dir), "architectures": hf_cfg.get("architectures")}}, out_path)
    return out_path


if __name__ == "__main__":
    p = ArgumentParser()
    p.add_argument("--model-dir", required=True)
    p.add_argument("--output", required=True)
    p.add_argument("--context-length", type=int, default=1024)
    a = p.parse_args()
    print(convert(a.model_dir, a.output, a.context_length))
