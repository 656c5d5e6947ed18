"""Checkpoint files.

Layout (training/checkpoint.py:22-88 of the reference, kept so its converters load our files):
``{"config": <json str>, "model": state_dict, "optimizer": [sd, ...] | None, "iteration": int,
"run_id": str | None}`` saved with ``torch.save`` to ``<save_dir>/<iteration>.pt``.
Additions: the write is atomic (temporary file + rename), a ``latest`` pointer file is kept next to
the checkpoints and ``find_latest`` returns the newest complete one.
"""

from __future__ import annotations

import os
import re
from pathlib import Path

import torch
import torch.nn as nn
from torch.optim import Optimizer

from sample_efficient_gpt_b200.utils.config_tools import save_config
from sample_efficient_gpt_b200.utils.logger import logger


def _to_device(x, device):
    if torch.is_tensor(x):
        return x.to(device, non_blocking=True)
    if isinstance(x, (list, tuple)):
        return type(x)(_to_device(v, device) for v in x)
    if isinstance(x, dict):
        return {k: _to_device(v, device) for k, v in x.items()}
    return x


def atomic_torch_save(obj, fpath: str | Path):
    fpath = Path(fpath)
    fpath.parent.mkdir(parents=True, exist_ok=True)
    tmp = fpath.with_name(fpath.name + f".tmp{os.getpid()}")
    torch.save(obj, tmp)
    os.replace(tmp, fpath)


def save_checkpoint(
    fpath: str | Path,
    cfg,
    model: nn.Module | dict,
    optimizers: list[Optimizer] | None,
    iteration: int = 0,
    run_id: str | None = None,
    extra: dict | None = None,
):
    model_sd = model if isinstance(model, dict) else model.state_dict()
    payload = {
        "config": save_config(cfg) if cfg is not None else None,
        "model": model_sd,
        "optimizer": [o.state_dict() for o in optimizers] if optimizers is not None else None,
        "iteration": iteration,
        "run_id": run_id,
    }
    if extra:
        payload.update(extra)
    atomic_torch_save(payload, fpath)
    fpath = Path(fpath)
    if re.fullmatch(r"\d+\.pt", fpath.name):
        latest = fpath.parent / "latest"
        tmp = latest.with_name(f"latest.tmp{os.getpid()}")
        tmp.write_text(fpath.name)
        os.replace(tmp, latest)


def find_latest(save_dir: str | Path) -> Path | None:
    """Newest complete ``<iteration>.pt`` in ``save_dir`` (pointer file first, directory scan otherwise)."""
    save_dir = Path(save_dir)
    pointer = save_dir / "latest"
    if pointer.exists():
        cand = save_dir / pointer.read_text().strip()
        if cand.exists():
            return cand
    best = None
    for fp in save_dir.glob("*.pt"):
        if re.fullmatch(r"\d+\.pt", fp.name) and (best is None or int(fp.stem) > int(best.stem)):
            best = fp
    return best


def load_model(fpath: str | Path, cfg, model: nn.Module) -> tuple[int, str | None]:
    ckpt = torch.load(fpath, map_location="cpu", weights_only=False)
    model.load_state_dict(ckpt["model"])
    return ckpt.get("iteration", 0), ckpt.get("run_id")


def load_optimizer(fpath: str | Path, cfg, model, optimizers: list[Optimizer] | None) -> None:
    """Restore optimizer state when the file has it and its structure matches; otherwise keep fresh state."""
    if not optimizers or optimizers[0] is None:
        return
    ckpt = torch.load(fpath, map_location="cpu", weights_only=False)
    saved = ckpt.get("optimizer")
    if saved is None or (isinstance(saved, list) and (not saved or saved[0] is None)):
        logger.info("no optimizers detected in the checkpoint, skipping...")
        return
    for idx, (opt, opt_sd) in enumerate(zip(optimizers, saved)):
        cur = opt.state_dict()
        if len(cur["param_groups"]) != len(opt_sd["param_groups"]):
            logger.info(f"optimizer {idx}: param_groups count mismatch, skipping optimizer load...")
            continue
        if any(len(c["params"]) != len(s["params"]) for c, s in zip(cur["param_groups"], opt_sd["param_groups"])):
            logger.info(f"optimizer {idx}: params count mismatch, skipping optimizer load...")
            continue
        # shapes: compare saved tensors with the parameters they belong to
        id_to_param = {}
        for g_cur, g_obj in zip(cur["param_groups"], opt.param_groups):
            id_to_param.update(dict(zip(g_cur["params"], g_obj["params"])))
        for pid, st in opt_sd["state"].items():
            p = id_to_param.get(pid)
            for k, v in st.items():
                if p is not None and torch.is_tensor(v) and k in ("m", "v", "momentum_buffer"):
                    assert v.shape == p.shape, f"optimizer {idx} state {k} of param {pid}: {v.shape=} != {p.shape=}"
        opt.load_state_dict(opt_sd)
        for p, st in opt.state.items():
            for k, v in list(st.items()):
                st[k] = _to_device(v, p.device)
        if hasattr(opt, "_batches"):
            opt.load_state_dict(opt.state_dict())  # rebind stacked storage on the right device
