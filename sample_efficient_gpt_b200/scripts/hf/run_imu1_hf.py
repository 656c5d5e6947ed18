"""Sampling sanity check of a converted HF directory (scripts/hf/run_imu1_hf.py of the reference).

Uses ``transformers`` when it knows the ``imu_1`` model type; otherwise loads the safetensors back into this package's
model through the key map, so the check also works without the model class."""

from __future__ import annotations

import json
from argparse import ArgumentParser
from pathlib import Path

import torch


def load_native_from_hf(model_dir: Path):
    from sample_efficient_gpt_b200.config_schema import ModelConfig
    from sample_efficient_gpt_b200.models import build_model
    from sample_efficient_gpt_b200.scripts.hf.convert_hf_to_imu import load_hf_state_dict
    from sample_efficient_gpt_b200.scripts.hf.keymap import from_hf_state_dict, native_model_config

    hf = json.loads((model_dir / "config.json").read_text())
    mcfg = native_model_config(hf)
    model = build_model(ModelConfig(**mcfg))
    sd = from_hf_state_dict({k: v.float() for k, v in load_hf_state_dict(model_dir).items()}, mcfg["weight_tying"])
    model.load_state_dict(sd)
    return model.eval(), hf


def main():
    p = ArgumentParser()
    p.add_argument("--model-dir", required=True)
    p.add_argument("--prompt", default="Once upon a time")
    p.add_argument("--max-new-tokens", type=int, default=64)
    p.add_argument("--temperature", type=float, default=0.7)
    p.add_argument("--top-p", type=float, default=0.9)
    a = p.parse_args()
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(a.model_dir)
    ids = torch.tensor([tok.encode(a.prompt)])
    try:
        from transformers import AutoModelForCausalLM

        model = AutoModelForCausalLM.from_pretrained(a.model_dir)
        out = model.generate(ids, max_new_tokens=a.max_new_tokens, do_sample=a.temperature > 0, temperature=a.temperature, top_p=a.top_p)
    except Exception:
        model, hf = load_native_from_hf(Path(a.model_dir))
        out, _ = model.generate(ids, hf.get("eos_token_id") or 0, top_p=a.top_p, temperature=a.temperature, max_steps=a.max_new_tokens)
    print(tok.decode(out[0].tolist()))


if __name__ == "__main__":
    main()
