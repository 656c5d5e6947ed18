"""Average saved checkpoints after the fact (scripts/data_processing/sft/ema_posthoc.py of the reference).

``ema``: walk the last ``--last-n`` ``<iteration>.pt`` files of a run in order with ``ema = d*ema + (1-d)*w`` (d = 0.8);
``avg``: plain mean of two checkpoints.  The result is written as ``<iteration>_ema.pt`` with the usual layout,
``optimizer: None`` and ``rng_state: None``."""

from __future__ import annotations

import re
from argparse import ArgumentParser
from pathlib import Path

import torch

from sample_efficient_gpt_b200.training.checkpoint import atomic_torch_save


def list_checkpoints(run_dir: Path) -> list[Path]:
    files = [p for p in run_dir.glob("*.pt") if re.fullmatch(r"\d+\.pt", p.name)]
    return sorted(files, key=lambda p: int(p.stem))


def ema_of(paths: list[Path], decay: float = 0.8) -> dict:
    first = torch.load(paths[0], map_location="cpu", weights_only=False)
    ema = {k: v.clone().float() if torch.is_floating_point(v) else v.clone() for k, v in first["model"].items()}
    last = first
    for p in paths[1:]:
        last = torch.load(p, map_location="cpu", weights_only=False)
        for k, v in last["model"].items():
            if torch.is_floating_point(v):
                ema[k].mul_(decay).add_(v.float(), alpha=1.0 - decay)
    if "lm_head.weight" in ema and "embedding.weight" in ema:
        ema["lm_head.weight"] = ema["embedding.weight"]
    return {"config": last["config"], "model": ema, "optimizer": None, "iteration": last["iteration"], "run_id": last.get("run_id"),
            "rng_state": None}


def average_of(a: Path, b: Path) -> dict:
    ca, cb = (torch.load(p, map_location="cpu", weights_only=False) for p in (a, b))
    model = {k: (v.float() + cb["model"][k].float()) / 2 if torch.is_floating_point(v) else v for k, v in ca["model"].items()}
    return {"config": cb["config"], "model": model, "optimizer": None, "iteration": cb["iteration"], "run_id": cb.get("run_id"), "rng_state": None}


def main():
    p = ArgumentParser()
    p.add_argument("--run-dir", type=Path, required=True)
    p.add_argument("--mode", default="ema", choices=["ema", "avg"])
    p.add_argument("--decay", type=float, default=0.8)
    p.add_argument("--last-n", type=int, default=6)
    a = p.parse_args()
    ckpts = list_checkpoints(a.run_dir)
    assert ckpts, f"no <iteration>.pt files in {a.run_dir}"
    out = ema_of(ckpts[-a.last_n :], a.decay) if a.mode == "ema" else average_of(ckpts[-2], ckpts[-1])
    dst = a.run_dir / f"{out['iteration']}_ema.pt"
    atomic_torch_save(out, dst)
    print(dst)


if __name__ == "__main__":
    main()
