"""Initialise an IMU-format checkpoint from a Llama-style HF model (SmolLM2), optionally widening it.

Counterpart of scripts/hf/convert_smollm2_to_imu.py of the reference.  Packing: ``q_proj | k_proj | v_proj`` rows become
the packed ``qkv`` matrix, ``gate_proj | up_proj`` rows the packed SwiGLU ``up`` matrix.  Widening modes for the parts of
a larger target that the source does not cover:
  * ``noise``         : keep the target's fresh init there, scaled by ``--init-multiplier``;
  * ``preserve``      : zeros there, so the widened network computes the source function on the old coordinates;
  * ``preserve-norm`` : like ``preserve`` for matrices, and RMSNorm gains of the new coordinates are set to 1.
``--ffn-net2wider`` / ``--attn-net2wider`` grow the FFN width / the number of heads by repeating units and dividing the
consuming matrix by the repeat count (function preserving), with optional zero-sum noise to break the symmetry.
Extras of the IMU architecture start as no-ops: gate weights zero (gate = 2*sigmoid(0) = 1), value-residual
``alpha1=1, alpha2=0, scale=1``; ``--qk-gain`` sets the QK-norm gain.
The result is ``{"model", "config", "iteration": 0, "optimizer": None, "hf_metadata"}``.
"""

from __future__ import annotations

import json
from argparse import ArgumentParser
from pathlib import Path

import torch

from sample_efficient_gpt_b200.scripts.hf.convert_hf_to_imu import load_hf_state_dict


def resize_like(fresh: torch.Tensor, src: torch.Tensor, mode: str, init_multiplier: float) -> torch.Tensor:
    """``fresh``-shaped tensor holding ``src`` on the overlap; the rest by ``mode``."""
    out = torch.zeros_like(fresh) if mode in ("preserve", "preserve-norm") else fresh.detach().clone() * init_multiplier
    idx = tuple(slice(0, min(a, b)) for a, b in zip(out.shape, src.shape))
    out[idx] = src[idx].to(out.dtype)
    return out


def repeat_map(src_units: int, dst_units: int) -> tuple[torch.Tensor, torch.Tensor]:
    """new unit -> old unit (each old unit repeated dst//src times, the first dst%src once more) and the repeat counts."""
    counts = torch.full((src_units,), dst_units // src_units, dtype=torch.long)
    counts[: dst_units % src_units] += 1
    return torch.arange(src_units).repeat_interleave(counts), counts


def zero_sum_noise(block: torch.Tensor, counts: torch.Tensor, std: float, gen: torch.Generator, width: int = 1) -> torch.Tensor:
    """Noise on the columns of repeated units that sums to zero over each unit's copies (keeps the function).  A unit is
    ``width`` adjacent columns (1 for FFN channels, head_dim for attention heads); its copies follow one another."""
    if std <= 0:
        return block
    pos = 0
    for c in counts.tolist():
        if c > 1:
            span = block[:, pos : pos + c * width]
            n = torch.randn(block.size(0), c, width, generator=gen) * std * span.std() / c
            span += (n - n.mean(dim=1, keepdim=True)).reshape(block.size(0), c * width)
        pos += c * width
    return block


def net2wider_ffn(gate, up, down, dst_dff: int, noise_std: float, gen) -> tuple[torch.Tensor, torch.Tensor]:
    old, counts = repeat_map(gate.size(0), dst_dff)
    packed = torch.cat([gate[old], up[old]], dim=0)
    down_new = zero_sum_noise(down[:, old] / counts[old].to(down.dtype)[None, :], counts, noise_std, gen)
    return packed, down_new


def net2wider_heads(q, k, v, o, src_heads, src_kv, dst_heads, dst_kv, hd, noise_std, gen):
    """Repeat whole heads (query heads and KV heads by the same map within a group) and split the output projection."""
    oldq, cq = repeat_map(src_heads, dst_heads)
    oldkv, _ = repeat_map(src_kv, dst_kv)
    rows = lambda idx: (idx[:, None] * hd + torch.arange(hd)[None, :]).reshape(-1)  # noqa: E731
    qn, kn, vn = q[rows(oldq)], k[rows(oldkv)], v[rows(oldkv)]
    cols = rows(oldq)
    denom = cq[oldq].repeat_interleave(hd).to(o.dtype)
    on = o[:, cols] / denom[None, :]
    on = zero_sum_noise(on, cq, noise_std, gen, width=hd)  # copies of a head see the same attention output: their noise cancels
    return qn, kn, vn, on


def convert(model_dir, out_path, target: dict | None = None, mode: str = "noise", init_multiplier: float = 1.0,
            ffn_net2wider: bool = False, attn_net2wider: bool = False, noise_std: float = 0.0, qk_gain: float | None = None,
            seed: int = 0) -> Path:
    from sample_efficient_gpt_b200.config_schema import default_cfg
    from sample_efficient_gpt_b200.models import build_model
    from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, save_config

    model_dir = Path(model_dir)
    hf = json.loads((model_dir / "config.json").read_text())
    src = {k: v.float() for k, v in load_hf_state_dict(model_dir).items()}
    sH, sKV = hf["num_attention_heads"], hf.get("num_key_value_heads", hf["num_attention_heads"])
    s_d, s_ff, L = hf["hidden_size"], hf["intermediate_size"], hf["num_hidden_layers"]
    hd = s_d // sH
    t = dict(d_model=s_d, d_ff=s_ff, n_layers=L, n_heads=sH, n_kv_heads=sKV, vocab_size=hf["vocab_size"], theta=hf.get("rope_theta", 10000),
             attn_qknorm=True, attn_val_residual=True, attn_gating="per-head", layernorm_scaling=True,
             weight_tying=hf.get("tie_word_embeddings", False))
    t.update(target or {})
    assert t["d_model"] // t["n_heads"] == hd, "head_dim must stay the same when widening"
    cfg = apply_overrides(default_cfg, {f"model.{k}": v for k, v in t.items()})
    torch.manual_seed(seed)
    gen = torch.Generator().manual_seed(seed)
    model = build_model(cfg.model)
    sd = model.state_dict()
    new = {}
    fit = lambda name, s: resize_like(sd[name], s, mode, init_multiplier)  # noqa: E731
    new["embedding.weight"] = fit("embedding.weight", src["model.embed_tokens.weight"])
    head_src = src.get("lm_head.weight", src["model.embed_tokens.weight"])
    new["lm_head.linear.weight"] = fit("lm_head.linear.weight", head_src)
    gain_fill = 1.0 if mode == "preserve-norm" else None
    for i in range(t["n_layers"]):
        si = min(i, L - 1)
        pre, spre = f"blocks.{i}.", f"model.layers.{si}."
        q, k, v = (src[spre + f"self_attn.{n}_proj.weight"] for n in "qkv")
        o = src[spre + "self_attn.o_proj.weight"]
        if attn_net2wider and (t["n_heads"] != sH or t["n_kv_heads"] != sKV):
            q, k, v, o = net2wider_heads(q, k, v, o, sH, sKV, t["n_heads"], t["n_kv_heads"], hd, noise_std, gen)
        qkv_fresh = sd[pre + "attn.qkv.linear.weight"]
        qo, ko = t["n_heads"] * hd, t["n_kv_heads"] * hd
        parts = [resize_like(qkv_fresh[:qo], q, mode, init_multiplier), resize_like(qkv_fresh[qo : qo + ko], k, mode, init_multiplier),
                 resize_like(qkv_fresh[qo + ko :], v, mode, init_multiplier)]
        new[pre + "attn.qkv.linear.weight"] = torch.cat(parts, dim=0)
        new[pre + "attn.out.linear.weight"] = fit(pre + "attn.out.linear.weight", o)
        gate, up, down = (src[spre + f"mlp.{n}_proj.weight"] for n in ("gate", "up", "down"))
        dff = sd[pre + "ffn.down.linear.weight"].size(1)
        if ffn_net2wider and dff > s_ff:
            packed, down = net2wider_ffn(gate, up, down, dff, noise_std, gen)
            gate, up = packed[:dff], packed[dff:]
        up_fresh = sd[pre + "ffn.up.linear.weight"]
        new[pre + "ffn.up.linear.weight"] = torch.cat([resize_like(up_fresh[:dff], gate, mode, init_multiplier),
                                                       resize_like(up_fresh[dff:], up, mode, init_multiplier)], dim=0)
        new[pre + "ffn.down.linear.weight"] = fit(pre + "ffn.down.linear.weight", down)
        for ours, theirs in (("ln1.gain", "input_layernorm.weight"), ("ln2.gain", "post_attention_layernorm.weight")):
            g = sd[pre + ours].clone() if gain_fill is None else torch.full_like(sd[pre + ours], gain_fill)
            s = src[spre + theirs]
            g[: min(len(g), len(s))] = s[: len(g)]
            new[pre + ours] = g
        if pre + "attn.attn_gate.linear.weight" in sd:
            new[pre + "attn.attn_gate.linear.weight"] = torch.zeros_like(sd[pre + "attn.attn_gate.linear.weight"])
        if pre + "attn.sdpa_qknorm.gain" in sd:
            new[pre + "attn.sdpa_qknorm.gain"] = torch.full_like(sd[pre + "attn.sdpa_qknorm.gain"], 1.0 if qk_gain is None else qk_gain)
        for nm, val in (("alpha1", 1.0), ("alpha2", 0.0), ("scale", 1.0)):
            if pre + f"attn.{nm}" in sd:
                new[pre + f"attn.{nm}"] = torch.full_like(sd[pre + f"attn.{nm}"], val)
    fn = sd["final_norm.gain"].clone() if gain_fill is None else torch.full_like(sd["final_norm.gain"], gain_fill)
    s = src["model.norm.weight"]
    fn[: min(len(fn), len(s))] = s[: len(fn)]
    new["final_norm.gain"] = fn
    if "lm_head.weight" in sd:
        new["lm_head.weight"] = new["embedding.weight"]
    missing = set(sd) - set(new)
    assert not missing, f"unfilled parameters: {sorted(missing)[:5]}"
    ordered = {k: new[k] for k in sd}
    out_path = Path(out_path)
    out_path.parent.mkdir(parents=True, exist_ok=True)
    torch.save({"config": save_config(cfg), "model": ordered, "optimizer": None, "iteration": 0, "run_id": None,
                "hf_metadata": {"source": str(model_dir), "mode": mode, "ffn_net2wider": ffn_net2wider, "attn_net2wider": attn_net2wider}},
               out_path)
    return out_path


def main():
    p = ArgumentParser()
    p.add_argument("--model-dir", required=True)
    p.add_argument("--output", required=True)
    p.add_argument("--width", type=int, default=None)
    p.add_argument("--n-heads", type=int, default=None)
    p.add_argument("--n-kv-heads", type=int, default=None)
    p.add_argument("--d-ff", type=int, default=None)
    p.add_argument("--n-layers", type=int, default=None)
    p.add_argument("--widening-mode", default="noise", choices=["noise", "preserve", "preserve-norm"])
    p.add_argument("--init-multiplier", type=float, default=1.0)
    p.add_argument("--ffn-net2wider", action="store_true")
    p.add_argument("--attn-net2wider", action="store_true")
    p.add_argument("--noise-std", type=float, default=0.0)
    p.add_argument("--qk-gain", type=float, default=None)
    p.add_argument("--seed", type=int, default=0)
    a = p.parse_args()
    target = {k: v for k, v in dict(d_model=a.width, n_heads=a.n_heads, n_kv_heads=a.n_kv_heads, d_ff=a.d_ff, n_layers=a.n_layers).items()
              if v is not None}
    print(convert(a.model_dir, a.output, target, a.widening_mode, a.init_multiplier, a.ffn_net2wider, a.attn_net2wider, a.noise_std,
                  a.qk_gain, a.seed))


if __name__ == "__main__":
    main()
