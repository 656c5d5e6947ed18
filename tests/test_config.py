import json

import pytest

from sample_efficient_gpt_b200.utils.config_tools import (
    apply_overrides, load_cfg, load_config, render_template, save_config, set_by_dotted,
)


def test_imu1_stages_resolve_like_the_reference():
    st = load_cfg("imu1_base.yaml", "stable")
    assert (st.data.batch_size, st.data.val_batch_size, st.data.context_length, st.data.seed) == (384, 32, 768, 42)
    assert st.model.d_model == 1152 and st.model.n_layers == 30 and st.model.n_heads == 18 and st.model.n_kv_heads == 6
    assert st.model.attn_gating == "per-head" and st.model.weight_tying and st.model.layernorm_scaling
    assert st.optim.lr == pytest.approx(6e-3) and st.optim.muon_lr == pytest.approx(0.011) and st.optim.muon_wd == 0.1
    assert st.optim.betas == (0.95, 0.99) and st.optim.scheduler == "wsd" and st.optim.use_muon
    assert st.optim.zero_lr_steps == 500 and st.optim.warmup_steps == 2500 and st.optim.wd == 0.0
    assert st.trainer.dtype == "bfloat16" and st.trainer.gradient_accumulation_steps == 2
    assert st.trainer.max_steps == 100000 and st.trainer.save_every == 2500 and st.trainer.val_every == 5000
    assert st.trainer.log_every == 50
    dc = load_cfg("imu1_base.yaml", "decay")
    assert (dc.data.batch_size, dc.data.context_length, dc.data.seed, dc.data.val_batch_size) == (312, 896, 43, 192)
    assert dc.optim.lr_min_coeff == 0.25 and dc.optim.wsd_phase == "decay" and dc.optim.wsd_decay_step == 100000
    mt = load_cfg("imu1_base.yaml", "midtrain")
    assert (mt.data.batch_size, mt.data.context_length, mt.data.val_batch_size) == (192, 1152, 8)
    assert mt.optim.lr == 0.002 and mt.optim.muon_lr == 0.003 and mt.optim.lr_min_coeff == 0.33 and mt.trainer.max_steps == 265000


def test_yaml_needs_key_and_rejects_unknown(tmp_path):
    with pytest.raises(ValueError):
        load_cfg("imu1_base.yaml", None)
    with pytest.raises(KeyError):
        load_cfg("imu1_base.yaml", "nope")
    bad = tmp_path / "bad.yaml"
    bad.write_text("model:\n  not_a_field: 3\n")
    with pytest.raises(TypeError):
        load_cfg(str(bad))


def test_overrides_and_roundtrip():
    cfg = load_cfg("gpt_small_faster")
    cfg2 = apply_overrides(cfg, {"optim.lr": 1e-3, "model.d_model": 512, "trainer.run_name": "x"})
    assert cfg2.optim.lr == 1e-3 and cfg2.model.d_model == 512 and cfg.model.d_model == 768
    with pytest.raises(TypeError):
        set_by_dotted(cfg, "optim.nope", 1)
    s = save_config(cfg2)
    assert isinstance(json.loads(s)["trainer"]["save_dir"], str)
    back = load_config(s)
    assert save_config(back) == s
    d = json.loads(s)
    d["model"]["from_the_future"] = 1  # unknown keys in a checkpoint config are ignored
    assert load_config(d).model.d_model == 512


def test_all_packaged_configs_load():
    for name in ("base", "gpt_small_faster", "gpt_126m"):
        load_cfg(name)
    for y, k in (("smollm2_wide.yaml", "stable"), ("tiny_cpu.yaml", None), ("imu1_moe.yaml", None), ("dense_1p5b.yaml", None),
                 ("imu1_base.yaml", "bench")):
        load_cfg(y, k)


def test_run_name_template():
    cfg = load_cfg("gpt_small_faster")
    name = render_template("{date}_{optim.lr}_{nope}", cfg)
    assert name.endswith("_0.007_NA") and len(name.split("_")[0]) == 4


def test_cli_resolve(tmp_path):
    from sample_efficient_gpt_b200.train import parse_args, resolve

    args = parse_args(["--config", "gpt_small_faster", "--train-path", "a", "--validation-path", "b",
                       "--override", '{"optim.lr": 0.001, "optim.seesaw_steps": "(10, 20)"}'])
    cfg, run_name = resolve(load_cfg(args.config), args)
    assert cfg.optim.lr == 0.001 and cfg.optim.seesaw_steps == (10, 20)
    assert cfg.optim.cosine_steps == cfg.trainer.max_steps
    assert cfg.data.train_path == "a" and str(cfg.trainer.save_dir).endswith(run_name) and "lr=0.00" in run_name


def test_loss_parity_compare_reports_window_differences(tmp_path):
    """``loss_parity.py --compare``: per-step and 50-step-window differences of two recorded loss curves."""
    import importlib.util
    import json
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("loss_parity", Path(__file__).resolve().parents[1] / "loss_parity.py")
    lp = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(lp)
    a = [5.0 - 0.01 * i for i in range(200)]
    b = [x + (0.02 if i >= 100 else 0.0) for i, x in enumerate(a)]
    for name, losses in (("a.json", a), ("b.json", b)):
        (tmp_path / name).write_text(json.dumps({"impl": "ours", "steps": 100, "losses": losses}))
    out = lp.compare(str(tmp_path / "a.json"), str(tmp_path / "b.json"))
    assert out["micro_steps"] == 200
    assert abs(out["max_abs_diff"] - 0.02) < 1e-5 and abs(out["max_abs_diff_of_50_step_means"] - 0.02) < 1e-5
    assert abs(out["mean_abs_diff"] - 0.01) < 1e-5
    assert len(out["windows"]) == 4 and abs(out["windows"][0][0] - out["windows"][0][1]) < 1e-5
