"""Command-line entry point.

Same flags as the reference (train.py:29-48): ``--config <python module | yaml>``, ``--config-key``,
``--override '{"a.b": v}'``, ``--train-path``, ``--validation-path``, ``--load-from``, ``--world-size``.
Launch with ``torchrun --nproc-per-node N -m sample_efficient_gpt_b200.train ... --world-size N``.
The process-group backend is NCCL on GPUs and gloo on CPU (``--backend`` overrides).
"""

from __future__ import annotations

import argparse
import ast
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist

from sample_efficient_gpt_b200.training.trainer import Trainer
from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, dataclass_to_nested_dict, load_cfg, wandb_run_name
from sample_efficient_gpt_b200.utils.logger import logger


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Train a sample-efficient GPT on B200")
    p.add_argument("--config", type=str, default="gpt_small_faster", help="python config module or YAML file")
    p.add_argument("--config-key", type=str, default=None, help="experiment key inside a YAML file")
    p.add_argument("--override", type=str, default="", help='JSON of dotted-key overrides, e.g. {"optim.lr": 1e-3}')
    p.add_argument("--train-path", type=str, default=None)
    p.add_argument("--validation-path", type=str, default=None)
    p.add_argument("--load-from", type=str, default=None)
    p.add_argument("--world-size", type=int, default=1)
    p.add_argument("--backend", type=str, default=None, help="nccl | gloo (default: nccl on GPU, gloo on CPU)")
    p.add_argument("--wandb", action="store_true", help="log to Weights & Biases on the main rank")
    return p.parse_args(argv)


def wandb_main_rank(world_size: int, rank: int) -> bool:
    """Rank that owns the wandb run (train.py:99-105 of the reference: rank 2 of 4, rank 0 of 8, none otherwise);
    here single-process runs log too."""
    if world_size == 4:
        return rank == 2
    if world_size in (1, 8):
        return rank == 0
    return False


def resolve(cfg, args):
    """Apply CLI/JSON overrides and derive the run name; returns (cfg, run_name)."""
    override = json.loads(args.override) if args.override else {}
    if isinstance(override.get("optim.seesaw_steps"), str):
        override["optim.seesaw_steps"] = tuple(ast.literal_eval(override["optim.seesaw_steps"]))
    cli = {"data.train_path": args.train_path, "data.validation_path": args.validation_path, "trainer.load_from": args.load_from}
    override.update({k: v for k, v in cli.items() if v is not None})
    if override.get("trainer.run_name"):
        cfg.trainer.run_name = override["trainer.run_name"]
        run_name = wandb_run_name(cfg)
    else:
        run_name = wandb_run_name(cfg)[:47]
        suffix = "_".join(f"{k.split('.')[-1][:4]}={str(v)[:4]}" for k, v in override.items())
        if suffix:
            run_name = f"{run_name}_{suffix}"
    cfg = apply_overrides(cfg, override)
    if not cfg.data.train_path or not cfg.data.validation_path:
        raise ValueError("Both train and validation paths must be provided via config or CLI overrides.")
    cfg = apply_overrides(cfg, {"optim.cosine_steps": cfg.trainer.max_steps})
    cfg.trainer.save_dir = Path(cfg.trainer.save_dir) / run_name
    return cfg, run_name


def train(rank: int, cfg, args):
    cfg, run_name = resolve(cfg, args)
    logger.info(f"Training run: {run_name}")
    world = dist.get_world_size() if dist.is_initialized() else 1
    run = None
    if args.wandb and wandb_main_rank(world, rank):
        import wandb

        run = wandb.init(project=cfg.project, name=run_name, config=dataclass_to_nested_dict(cfg))
    trainer = Trainer(cfg, load_from=args.load_from, wandb=run)
    trainer.train()
    if run is not None:
        run.finish()


def main(argv=None):
    args = parse_args(argv)
    cfg = load_cfg(args.config, args.config_key)
    cfg.optim.lr = float(cfg.optim.lr)
    if cfg.optim.muon_lr is not None:
        cfg.optim.muon_lr = float(cfg.optim.muon_lr)
    if args.world_size > 1:
        use_cuda = torch.cuda.is_available() and cfg.trainer.device.startswith("cuda")
        backend = args.backend or ("nccl" if use_cuda else "gloo")
        if use_cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend)
        try:
            train(dist.get_rank(), cfg, args)
        finally:
            dist.destroy_process_group()
    else:
        train(0, cfg, args)


if __name__ == "__main__":
    main()
