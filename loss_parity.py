"""Loss-curve parity: the same IMU-1 430M training run on this package and on the unmodified reference.

    python loss_parity.py --impl ours --steps 600 --out parity_ours.json
    python loss_parity.py --impl reference --steps 600 --out parity_ref.json
    python loss_parity.py --compare parity_ours.json parity_ref.json
    torchrun --nproc-per-node 2 ... loss_parity.py --impl ours --gpus 2 --steps 600 --out parity_ours_2gpu.json

With ``--gpus N`` (N = 2 here: one micro-batch of 8 per GPU) the run goes through everything a multi-GPU job uses - bucketed
gradient reduction over the NVLink kernels, sharded NorMuon with the all-gather in the GEMM epilogue - on the *same* 16
sequences per optimizer step as the single-GPU run: every rank draws the single-GPU run's two micro-batches and keeps its
own, and the schedule position advances by two per step as it does there.  Rank r's loss is micro-step r of the step.

Both arms: stage ``stable`` of ``configs/imu1_base.yaml`` (their own copy), random init from the same seed, the same
synthetic Zipf(s=1.1) token shards read by their own loaders from the same data seed, 16 sequences of 2048 tokens per
optimizer step as two accumulated micro-batches of 8 (what the reference can hold on one GPU), no zero-LR phase and a
100-step warm-up so that the comparison covers real learning.  The training loss of every micro-step is recorded.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
from pathlib import Path

import torch

import bench

OVERRIDES = {"optim.zero_lr_steps": 0, "optim.warmup_steps": 100, "trainer.gradient_accumulation_steps": 2, "trainer.log_every": 10**9,
             "trainer.load_from": None, "data.batch_size": 8, "data.context_length": bench.SEQ}


def run_distributed(steps: int, n_gpus: int) -> list[float] | None:
    import torch.distributed as dist

    from sample_efficient_gpt_b200.training.data import MemoryMappedDataset
    from sample_efficient_gpt_b200.training.trainer import Trainer
    from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, load_cfg

    world, rank, local = bench.dist_setup(n_gpus)
    assert world == 2, "two micro-batches of 8 per optimizer step: one per GPU"
    tmp = [tempfile.mkdtemp(prefix="segpt_parity_dist_") if rank == 0 else None]
    dist.broadcast_object_list(tmp, src=0)
    tmp = Path(tmp[0])
    if rank == 0:
        bench.make_dataset(tmp)
    dist.barrier()
    paths = {"data.train_path": str(tmp / "train"), "data.validation_path": str(tmp / "val.npy"), "trainer.save_dir": str(tmp / "ckpt")}
    cfg = load_cfg(str(bench.ROOT / "sample_efficient_gpt_b200/configs/imu1_base.yaml"), "stable")
    cfg = apply_overrides(cfg, {**OVERRIDES, **paths, "data.tokenizer_path": "", "trainer.device": f"cuda:{local}", "trainer.dtype": "bfloat16",
                                "trainer.ema_every": 0, "trainer.gradient_accumulation_steps": 1, "data.batch_size": 8 * world,
                                "optim.shard_muon": True, "trainer.comm_backend": os.environ.get("SEGPT_COMM_BACKEND", "auto")})
    cfg.optim.lr, cfg.optim.muon_lr = float(cfg.optim.lr), float(cfg.optim.muon_lr)
    trainer = Trainer(cfg)
    assert trainer.ddp is not None
    source = MemoryMappedDataset(cfg.data.train_path, cfg.data.context_length, trainer.device, cfg.data.seed)  # the single-GPU stream
    losses = []
    for step in range(steps):
        micro = [source._get_batch_internal(8) for _ in range(world)]
        x, y = micro[rank]
        trainer.iteration = 2 * step + 1  # where the single-GPU run stands when it takes this optimizer step
        log = trainer.train_step(x.to(trainer.device), y.to(trainer.device))
        both = [torch.zeros((), device=trainer.device) for _ in range(world)]
        dist.all_gather(both, log["train_loss"].detach().float().reshape(()))
        losses.extend(both)
    trainer.check_kernel_status()
    out = [float(v) for v in torch.stack(losses).cpu()]
    dist.destroy_process_group()
    return out if rank == 0 else None


def run(impl: str, steps: int) -> list[float]:
    tmp = Path(tempfile.mkdtemp(prefix=f"segpt_parity_{impl}_"))
    bench.make_dataset(tmp)
    paths = {"data.train_path": str(tmp / "train"), "data.validation_path": str(tmp / "val.npy"), "trainer.save_dir": str(tmp / "ckpt")}
    if impl == "ours":
        from sample_efficient_gpt_b200.training.trainer import Trainer
        from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, load_cfg

        cfg = load_cfg(str(bench.ROOT / "sample_efficient_gpt_b200/configs/imu1_base.yaml"), "stable")
        cfg = apply_overrides(cfg, {**OVERRIDES, **paths, "data.tokenizer_path": "", "trainer.device": "cuda:0", "trainer.dtype": "bfloat16",
                                    "trainer.ema_every": 0})
        cfg.optim.lr, cfg.optim.muon_lr = float(cfg.optim.lr), float(cfg.optim.muon_lr)
        trainer = Trainer(cfg)
        fetch = trainer.fetch_batch
    else:
        sys.path.insert(0, str(bench.ROOT / "baseline" / "_ref"))
        os.environ.setdefault("WANDB_MODE", "disabled")
        os.environ.setdefault("NO_VAL", "1")
        os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
        from sample_efficient_gpt.training.trainer import Trainer
        from sample_efficient_gpt.utils.config_tools import apply_overrides, load_config_from_yaml

        bench.make_tokenizer(tmp / "tok")
        cfg = load_config_from_yaml(bench.ROOT / "baseline/_ref/sample_efficient_gpt/configs/imu1_base.yaml", "stable")
        cfg = apply_overrides(cfg, {**OVERRIDES, **paths, "data.tokenizer_path": str(tmp / "tok"), "optim.lr": float(cfg.optim.lr),
                                    "optim.muon_lr": float(cfg.optim.muon_lr)})
        trainer = Trainer(cfg, compile=True)

        def fetch():
            x, y = trainer.train_dataset.get_batch(cfg.data.batch_size)
            return x.to(cfg.trainer.device), y.to(cfg.trainer.device)

    losses = []
    for _ in range(2 * steps):
        x, y = fetch()
        log = trainer.train_step(x, y)
        trainer.iteration += 1
        losses.append(log["train_loss"].detach() if torch.is_tensor(log["train_loss"]) else torch.tensor(float(log["train_loss"])))
    return [float(v) for v in torch.stack([l.float().cpu() for l in losses])]


def compare(a_path: str, b_path: str) -> dict:
    a, b = json.load(open(a_path)), json.load(open(b_path))
    la, lb = torch.tensor(a["losses"]), torch.tensor(b["losses"])
    n = min(len(la), len(lb))
    la, lb = la[:n], lb[:n]
    diff = (la - lb).abs()
    win = 50
    smooth = lambda t: t.unfold(0, win, win).mean(-1)
    out = {"micro_steps": n, "first_loss": [float(la[0]), float(lb[0])], "final_window_mean": [float(la[-win:].mean()), float(lb[-win:].mean())],
           "max_abs_diff": float(diff.max()), "mean_abs_diff": float(diff.mean()),
           "max_abs_diff_of_50_step_means": float((smooth(la) - smooth(lb)).abs().max()) if n >= win else None,
           "windows": [[round(float(x), 4), round(float(y), 4)] for x, y in zip(smooth(la), smooth(lb))] if n >= win else []}
    print(json.dumps(out))
    return out


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--steps", type=int, default=600, help="optimizer steps (two micro-steps each)")
    p.add_argument("--out", default=None)
    p.add_argument("--compare", nargs=2, default=None)
    p.add_argument("--gpus", type=int, default=1, help="2: the multi-GPU path on the single-GPU run's data (launch under torchrun)")
    a = p.parse_args()
    if a.compare:
        compare(*a.compare)
        return
    if a.gpus > 1:
        assert a.impl == "ours"
        losses = run_distributed(a.steps, a.gpus)
        if losses is None:
            return
    else:
        losses = run(a.impl, a.steps)
    if a.out:
        Path(a.out).parent.mkdir(parents=True, exist_ok=True)
        json.dump({"impl": a.impl, "steps": a.steps, "losses": losses}, open(a.out, "w"))
    print(json.dumps({"impl": a.impl, "first": losses[0], "last": sum(losses[-20:]) / 20}))


if __name__ == "__main__":
    main()
