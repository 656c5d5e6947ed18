"""``.pt`` checkpoint -> HuggingFace directory (``model.safetensors``, ``config.json``, ``generation_config.json``,
optionally the tokenizer with a chat template).  Counterpart of scripts/hf/convert_imu1_checkpoint.py of the reference.

``--test`` checks that the key mapping is lossless: logits of the native model from the original weights and from the
weights after a round trip through HF names agree to 1e-5 on random tokens (CPU, fp32).
"""

from __future__ import annotations

import json
import shutil
from argparse import ArgumentParser
from pathlib import Path

import torch

from sample_efficient_gpt_b200.scripts.hf.keymap import from_hf_state_dict, hf_config_dict, ordered_native_state_dict, to_hf_state_dict

CHAT_TEMPLATE = (
    "{% for message in messages %}{{ '<|im_start|>' + message['role'] + '\n' + message['content'] + '<|im_end|>\n' }}"
    "{% endfor %}{% if add_generation_prompt %}{{ '<|im_start|>assistant\n' }}{% endif %}"
)


def load_checkpoint(path) -> dict:
    ckpt = torch.load(path, map_location="cpu", weights_only=False)
    if "model" not in ckpt or "config" not in ckpt:
        raise ValueError("Checkpoint does not contain expected keys 'model'/'config'.")
    if isinstance(ckpt["config"], str):
        ckpt["config"] = json.loads(ckpt["config"])
    return ckpt


def resolve_special_ids(tokenizer_dir: Path | None):
    bos, eos, pad = None, 256, None
    if tokenizer_dir is not None:
        try:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(tokenizer_dir, local_files_only=True)
            bos = tok.bos_token_id
            eos = tok.eos_token_id or tok.convert_tokens_to_ids("<|endoftext|>")
            pad = tok.pad_token_id
        except Exception as exc:
            print(f"warning: tokenizer at {tokenizer_dir} not loadable: {exc}")
    return bos, eos, pad


def native_logits(cfg: dict, state_dict: dict, tokens: torch.Tensor) -> torch.Tensor:
    from sample_efficient_gpt_b200.models import build_model
    from sample_efficient_gpt_b200.utils.config_tools import load_config

    model = build_model(load_config(cfg).model)
    model.load_state_dict(state_dict)
    model.eval()
    with torch.no_grad():
        return model(tokens)[0]


def convert(ckpt_path, out_dir, tokenizer_dir=None, tie_word_embeddings=None, dtype: str = "float32") -> Path:
    from safetensors.torch import save_file

    ckpt = load_checkpoint(ckpt_path)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    bos, eos, pad = resolve_special_ids(Path(tokenizer_dir) if tokenizer_dir else None)
    cfg = hf_config_dict(ckpt["config"], bos, eos, pad, tie_word_embeddings)
    cfg["torch_dtype"] = dtype
    td = getattr(torch, dtype)
    hf_sd = {k: v.detach().to(td).contiguous().clone() for k, v in to_hf_state_dict(ckpt["model"]).items()}
    save_file(hf_sd, str(out / "model.safetensors"), metadata={"format": "pt"})
    (out / "config.json").write_text(json.dumps(cfg, indent=2))
    (out / "generation_config.json").write_text(json.dumps({"bos_token_id": bos, "eos_token_id": eos, "pad_token_id": pad}, indent=2))
    if tokenizer_dir:
        for f in Path(tokenizer_dir).glob("*"):
            if f.is_file():
                shutil.copy(f, out / f.name)
        tc = out / "tokenizer_config.json"
        if tc.exists():
            d = json.loads(tc.read_text())
            d.setdefault("chat_template", CHAT_TEMPLATE)
            tc.write_text(json.dumps(d, indent=2))
    return out


def self_test(ckpt_path) -> float:
    ckpt = load_checkpoint(ckpt_path)
    cfg, sd = ckpt["config"], ckpt["model"]
    back = ordered_native_state_dict(from_hf_state_dict(to_hf_state_dict(sd), "lm_head.weight" in sd), cfg["model"]["n_layers"])
    assert list(back) == list(sd), "key order changed in the round trip"
    tokens = torch.randint(0, cfg["model"]["vocab_size"], (2, 16), generator=torch.Generator().manual_seed(0))
    diff = (native_logits(cfg, sd, tokens) - native_logits(cfg, back, tokens)).abs().max().item()
    assert diff <= 1e-5, f"round-trip logits differ by {diff}"
    return diff


def main():
    p = ArgumentParser()
    p.add_argument("--checkpoint", required=True)
    p.add_argument("--output-dir", required=True)
    p.add_argument("--tokenizer-dir", default=None)
    p.add_argument("--dtype", default="float32", choices=["float32", "bfloat16", "float16"])
    p.add_argument("--tie-word-embeddings", default=None, type=lambda s: s.lower() in ("1", "true"))
    p.add_argument("--test", action="store_true")
    a = p.parse_args()
    if a.test:
        print(f"round-trip max |dlogits| = {self_test(a.checkpoint):.2e}")
    print(convert(a.checkpoint, a.output_dir, a.tokenizer_dir, a.tie_word_embeddings, a.dtype))


if __name__ == "__main__":
    main()
