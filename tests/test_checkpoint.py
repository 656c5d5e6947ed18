import json

import numpy as np
import torch

from sample_efficient_gpt_b200.optim import WeightEMA
from sample_efficient_gpt_b200.training.checkpoint import find_latest, load_model, load_optimizer, save_checkpoint
from sample_efficient_gpt_b200.training.trainer import Trainer
from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, load_cfg


def _cfg(tmp_path, **over):
    rng = np.random.default_rng(0)
    d = tmp_path / "train"
    d.mkdir(exist_ok=True)
    np.save(d / "a.npy", rng.integers(0, 512, 20_000).astype(np.uint16))
    np.save(tmp_path / "val.npy", rng.integers(0, 512, 3_000).astype(np.uint16))
    cfg = load_cfg("tiny_cpu.yaml")
    base = {"data.train_path": str(d), "data.validation_path": str(tmp_path / "val.npy"), "trainer.save_dir": str(tmp_path / "ck"),
            "model.vocab_size": 512, "model.n_layers": 2, "model.d_model": 64, "model.d_ff": 128, "model.n_heads": 2, "model.n_kv_heads": 1,
            "data.context_length": 32, "data.batch_size": 4, "trainer.max_steps": 4, "trainer.save_every": 2, "trainer.ema_every": 1,
            "model.weight_tying": True}
    base.update(over)
    return apply_overrides(cfg, base)


def test_train_save_resume_layout(tmp_path):
    cfg = _cfg(tmp_path)
    tr = Trainer(cfg)
    tr.train()
    ck = tmp_path / "ck"
    assert sorted(p.name for p in ck.iterdir()) == ["0.pt", "0_ema.pt", "2.pt", "2_ema.pt", "4.pt", "4_ema.pt", "latest"]
    assert find_latest(ck).name == "4.pt"
    blob = torch.load(ck / "4.pt", map_location="cpu", weights_only=False)
    assert set(blob) == {"config", "model", "optimizer", "iteration", "run_id"} and blob["iteration"] == 4
    assert isinstance(blob["config"], str) and json.loads(blob["config"])["model"]["d_model"] == 64
    assert "lm_head.weight" in blob["model"] and "lm_head.linear.weight" in blob["model"]
    adamw_sd, muon_sd = blob["optimizer"]
    st = adamw_sd["state"][0]
    assert set(st) == {"t", "m", "v"} and st["t"] == 5
    mst = next(iter(muon_sd["state"].values()))
    assert set(mst) == {"momentum_buffer", "second_momentum_buffer"}
    ema = torch.load(ck / "4_ema.pt", map_location="cpu", weights_only=False)
    assert ema["optimizer"] is None and list(ema["model"]) == list(blob["model"])
    # resume: weights, iteration and optimizer state come back; a further step then matches a continued run
    tr2 = Trainer(_cfg(tmp_path, **{"trainer.load_from": str(ck / "4.pt"), "trainer.max_steps": 6}))
    assert tr2.iteration == 4
    for a, b in zip(tr.model.parameters(), tr2.model.parameters()):
        assert torch.equal(a, b)
    p0 = tr.optimizers[1].param_groups[0]["params"][0]
    q0 = tr2.optimizers[1].param_groups[0]["params"][0]
    assert torch.allclose(tr.optimizers[1].state[p0]["momentum_buffer"], tr2.optimizers[1].state[q0]["momentum_buffer"])
    x = torch.randint(0, 512, (4, 32)); y = torch.randint(0, 512, (4, 32))
    tr.cfg.trainer.max_steps = 6
    tr.train_step(x, y); tr2.train_step(x, y)
    for a, b in zip(tr.model.parameters(), tr2.model.parameters()):
        assert torch.allclose(a, b, atol=1e-6)


def test_load_optimizer_tolerates_missing_state(tmp_path):
    cfg = _cfg(tmp_path)
    tr = Trainer(cfg)
    save_checkpoint(tmp_path / "x.pt", cfg, tr.model, None, iteration=7, run_id="abc")
    it, rid = load_model(tmp_path / "x.pt", cfg, tr.model)
    assert (it, rid) == (7, "abc")
    load_optimizer(tmp_path / "x.pt", cfg, tr.model, tr.optimizers)  # no optimizer in the file: silently kept fresh
    assert not (tmp_path / "latest").exists()  # only <iteration>.pt files move the pointer


def test_ema_recurrence():
    m = torch.nn.Linear(4, 4, bias=False)
    ema = WeightEMA(m, decay=0.8, every=2)
    w0 = m.weight.detach().clone()
    with torch.no_grad():
        m.weight.add_(1.0)
    assert not ema.maybe_update() and ema.maybe_update()
    assert torch.allclose(ema.state_dict()["weight"], 0.8 * w0 + 0.2 * (w0 + 1.0))


def test_failed_kernel_wait_stops_training_before_the_next_checkpoint(tmp_path):
    """A status word that reports an expired wait (here through an injected probe - on a GPU the probes read the kernels'
    device words) makes train() raise at the next logging step, and no checkpoint is written after that."""
    import pytest

    from sample_efficient_gpt_b200.parallel.symm import CommTimeout

    cfg = _cfg(tmp_path, **{"trainer.max_steps": 6, "trainer.save_every": 3, "trainer.log_every": 1})
    tr = Trainer(cfg)
    state = {"calls": 0}

    def probe():
        state["calls"] += 1
        return 4 if tr.iteration >= 4 else 0

    tr.status_probes.append(("a test probe", probe))
    with pytest.raises(CommTimeout):
        tr.train()
    assert tr.iteration == 4 and state["calls"] >= 4
    names = sorted(p.name for p in (tmp_path / "ck").iterdir() if p.name.endswith(".pt") and "ema" not in p.name)
    assert names == ["0.pt", "3.pt"], names  # nothing from iteration 4 on
    with pytest.raises(CommTimeout):
        tr.save_state()  # a save attempt after the failure is refused as well


def test_prefetch_thread_failure_reaches_the_consumer(tmp_path):
    import pytest

    from sample_efficient_gpt_b200.training.data import MemoryMappedDataset

    cfg = _cfg(tmp_path)
    ds = MemoryMappedDataset(cfg.data.train_path, 32, torch.device("cpu"), 0)
    ds._get_batch_internal = lambda bs: (_ for _ in ()).throw(OSError("disk went away"))
    with pytest.raises(RuntimeError, match="prefetch thread failed"):
        ds.get_batch(4)
    with pytest.raises(RuntimeError, match="prefetch thread failed"):
        ds.get_batch(4)
