import json

import pytest
import torch

from sample_efficient_gpt_b200.models import Transformer
from sample_efficient_gpt_b200.scripts.hf import keymap
from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, save_config
from sample_efficient_gpt_b200.config_schema import default_cfg

MODEL = dict(vocab_size=200, d_model=64, d_ff=128, n_layers=2, n_heads=4, n_kv_heads=2, attn_qknorm=True, attn_val_residual=True,
             attn_gating="per-head", layernorm_scaling=True, weight_tying=True)


def _ckpt(tmp_path):
    cfg = apply_overrides(default_cfg, {f"model.{k}": v for k, v in MODEL.items()})
    torch.manual_seed(0)
    from sample_efficient_gpt_b200.models import build_model

    m = build_model(cfg.model)
    path = tmp_path / "10.pt"
    torch.save({"config": save_config(cfg), "model": m.state_dict(), "optimizer": None, "iteration": 10, "run_id": None}, path)
    return path, m, cfg


def test_key_map_matches_reference_names_and_round_trips(tmp_path):
    path, m, cfg = _ckpt(tmp_path)
    sd = m.state_dict()
    hf = keymap.to_hf_state_dict(sd)
    assert "lm_head.weight" in hf and hf["lm_head.weight"].data_ptr() == sd["lm_head.linear.weight"].data_ptr()
    want = {"model.embed_tokens.weight", "model.norm.weight", "model.layers.0.input_layernorm.weight",
            "model.layers.0.self_attn.qkv_proj.weight", "model.layers.0.self_attn.o_proj.weight", "model.layers.0.self_attn.attn_gate.weight",
            "model.layers.0.self_attn.qk_norm.gain", "model.layers.0.self_attn.alpha1", "model.layers.0.self_attn.alpha2",
            "model.layers.0.self_attn.value_scale", "model.layers.1.post_attention_layernorm.weight", "model.layers.1.mlp.up_proj.weight",
            "model.layers.1.mlp.down_proj.weight"}
    assert want <= set(hf) and len(hf) == len(sd) - 1
    back = keymap.ordered_native_state_dict(keymap.from_hf_state_dict(hf), 2)
    assert list(back) == list(sd) and all(torch.equal(back[k], sd[k]) for k in sd)
    with pytest.raises(KeyError):
        keymap.rename_to_hf("blocks.0.nope")
    extra = dict(hf)
    extra["model.layers.0.input_layernorm.position_scale"] = torch.ones(())
    extra["model.rotary_emb.cos_cached"] = torch.ones(2)
    assert set(keymap.from_hf_state_dict(extra)) == set(sd)


def test_pt_to_hf_and_back(tmp_path):
    pytest.importorskip("safetensors")
    from sample_efficient_gpt_b200.scripts.hf.convert_hf_to_imu import convert as to_pt
    from sample_efficient_gpt_b200.scripts.hf.convert_imu1_checkpoint import convert as to_hf, self_test

    path, m, cfg = _ckpt(tmp_path)
    assert self_test(path) <= 1e-5
    out = to_hf(path, tmp_path / "hf")
    c = json.loads((out / "config.json").read_text())
    assert c["model_type"] == "imu_1" and c["hidden_size"] == 64 and c["num_key_value_heads"] == 2 and c["eos_token_id"] == 256
    back = to_pt(out, tmp_path / "back.pt")
    blob = torch.load(back, map_location="cpu", weights_only=False)
    assert blob["iteration"] == 0 and blob["optimizer"] is None
    assert list(blob["model"]) == list(m.state_dict())
    m2 = Transformer(2, 200, 64, 4, 128, **{k: v for k, v in MODEL.items() if k.startswith("attn") or k in ("layernorm_scaling", "weight_tying", "n_kv_heads")})
    m2.load_state_dict(blob["model"])
    ids = torch.randint(0, 200, (1, 9))
    assert torch.allclose(m(ids)[0], m2(ids)[0], atol=1e-6)


def _fake_llama(tmp_path, d=32, ff=64, L=2, H=4, KV=2, V=100):
    from safetensors.torch import save_file

    torch.manual_seed(1)
    hd = d // H
    sd = {"model.embed_tokens.weight": torch.randn(V, d) * 0.1, "model.norm.weight": torch.rand(d) + 0.5}
    for i in range(L):
        p = f"model.layers.{i}."
        sd[p + "self_attn.q_proj.weight"] = torch.randn(H * hd, d) * 0.1
        sd[p + "self_attn.k_proj.weight"] = torch.randn(KV * hd, d) * 0.1
        sd[p + "self_attn.v_proj.weight"] = torch.randn(KV * hd, d) * 0.1
        sd[p + "self_attn.o_proj.weight"] = torch.randn(d, d) * 0.1
        sd[p + "mlp.gate_proj.weight"] = torch.randn(ff, d) * 0.1
        sd[p + "mlp.up_proj.weight"] = torch.randn(ff, d) * 0.1
        sd[p + "mlp.down_proj.weight"] = torch.randn(d, ff) * 0.1
        sd[p + "input_layernorm.weight"] = torch.rand(d) + 0.5
        sd[p + "post_attention_layernorm.weight"] = torch.rand(d) + 0.5
    mdir = tmp_path / "llama"
    mdir.mkdir()
    save_file(sd, str(mdir / "model.safetensors"))
    (mdir / "config.json").write_text(json.dumps(dict(hidden_size=d, intermediate_size=ff, num_hidden_layers=L, num_attention_heads=H,
                                                       num_key_value_heads=KV, vocab_size=V, rope_theta=10000, tie_word_embeddings=True)))
    return mdir, sd


def test_smollm2_init_packing_and_function_preserving_ffn_widening(tmp_path):
    pytest.importorskip("safetensors")
    from sample_efficient_gpt_b200.scripts.hf.convert_smollm2_to_imu import convert, repeat_map

    mdir, src = _fake_llama(tmp_path)
    same = torch.load(convert(mdir, tmp_path / "same.pt"), weights_only=False)
    sd = same["model"]
    q, k, v = (src[f"model.layers.0.self_attn.{n}_proj.weight"] for n in "qkv")
    assert torch.equal(sd["blocks.0.attn.qkv.linear.weight"], torch.cat([q, k, v]))
    assert torch.equal(sd["blocks.1.ffn.up.linear.weight"], torch.cat([src["model.layers.1.mlp.gate_proj.weight"], src["model.layers.1.mlp.up_proj.weight"]]))
    assert float(sd["blocks.0.attn.attn_gate.linear.weight"].abs().sum()) == 0 and float(sd["blocks.0.attn.alpha2"]) == 0
    assert json.loads(same["config"])["model"]["n_kv_heads"] == 2 and same["iteration"] == 0
    old, counts = repeat_map(3, 8)
    assert old.tolist() == [0, 0, 0, 1, 1, 1, 2, 2] and counts.tolist() == [3, 3, 2]
    wide = torch.load(convert(mdir, tmp_path / "wide.pt", target={"d_ff": 128}, ffn_net2wider=True, noise_std=0.1), weights_only=False)["model"]
    x = torch.randn(5, 32)

    def ffn(up_w, down_w):
        g, u = (x @ up_w.t()).chunk(2, dim=-1)
        return (torch.nn.functional.silu(g) * u) @ down_w.t()

    a = ffn(sd["blocks.0.ffn.up.linear.weight"], sd["blocks.0.ffn.down.linear.weight"])
    b = ffn(wide["blocks.0.ffn.up.linear.weight"], wide["blocks.0.ffn.down.linear.weight"])
    assert wide["blocks.0.ffn.down.linear.weight"].shape == (32, 128) and torch.allclose(a, b, atol=1e-5)
    wider = torch.load(convert(mdir, tmp_path / "w2.pt", target={"d_model": 64, "n_heads": 8, "n_kv_heads": 4, "d_ff": 128}, mode="preserve"),
                       weights_only=False)["model"]
    assert wider["embedding.weight"].shape == (100, 64) and float(wider["embedding.weight"][:, 32:].abs().sum()) == 0


def test_head_widening_noise_breaks_symmetry_and_keeps_the_function():
    from sample_efficient_gpt_b200.scripts.hf.convert_smollm2_to_imu import net2wider_heads

    torch.manual_seed(0)
    d, H, KV, hd = 32, 4, 2, 8
    q, k, v, o = torch.randn(H * hd, d), torch.randn(KV * hd, d), torch.randn(KV * hd, d), torch.randn(d, H * hd)
    x = torch.randn(6, d)

    def attn_out(q, k, v, o, heads, kv):
        qh = (x @ q.t()).view(6, heads, hd)
        kh = (x @ k.t()).view(6, kv, hd).repeat_interleave(heads // kv, dim=1)
        vh = (x @ v.t()).view(6, kv, hd).repeat_interleave(heads // kv, dim=1)
        att = torch.einsum("thd,shd->hts", qh, kh).div(hd**0.5).softmax(-1)
        return torch.einsum("hts,shd->thd", att, vh).reshape(6, heads * hd) @ o.t()

    want = attn_out(q, k, v, o, H, KV)
    gen = torch.Generator().manual_seed(1)
    q0, k0, v0, o0 = net2wider_heads(q, k, v, o.clone(), H, KV, 8, 4, hd, 0.0, gen)
    q1, k1, v1, o1 = net2wider_heads(q, k, v, o.clone(), H, KV, 8, 4, hd, 0.5, gen)
    assert torch.allclose(attn_out(q0, k0, v0, o0, 8, 4), want, atol=1e-5)
    assert torch.allclose(attn_out(q1, k1, v1, o1, 8, 4), want, atol=1e-4), "zero-sum noise must keep the function"
    assert torch.equal(o0[:, :hd], o0[:, hd : 2 * hd]), "without noise the copies of a head are exact duplicates"
    assert not torch.allclose(o1[:, :hd], o1[:, hd : 2 * hd]), "--noise-std must perturb the copies"


def test_posthoc_ema(tmp_path):
    from sample_efficient_gpt_b200.scripts.ema_posthoc import ema_of, list_checkpoints

    for it, val in ((1, 1.0), (2, 2.0), (10, 3.0)):
        torch.save({"config": "{}", "model": {"w": torch.full((2,), val)}, "optimizer": None, "iteration": it, "run_id": None}, tmp_path / f"{it}.pt")
    torch.save({}, tmp_path / "2_ema.pt")
    paths = list_checkpoints(tmp_path)
    assert [p.name for p in paths] == ["1.pt", "2.pt", "10.pt"]
    out = ema_of(paths, 0.8)
    assert out["iteration"] == 10 and out["optimizer"] is None
    assert torch.allclose(out["model"]["w"], torch.full((2,), 0.8 * (0.8 * 1 + 0.2 * 2) + 0.2 * 3))
