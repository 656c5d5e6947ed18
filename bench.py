"""Headline benchmark: training tokens/s of IMU-1 430M (seq 2048, 16 sequences per GPU, bf16).

``python bench.py --gpus N --steps K --warmup W [--impl ours|reference]``; for N > 1 launch it with
``python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py ...``.
Rank 0 prints ONE JSON line.  Every timed step is a full training step: forward, backward, gradient
reduction, NorMuon + AdamW update (gradient accumulation 1), weight EMA every 10 steps.

Two measurements per run:
  * ``value``: K steps timed on the device with CUDA events (barrier + synchronize on both sides, max over
    ranks) with the batches already resident on the GPU (a different batch every step);
  * ``e2e``: K steps through the public API (``Trainer.fetch_batch`` + ``Trainer.train_step``): every step
    copies its int32 inputs/targets from pinned host memory and reads the loss back to the host.
Data are synthetic Zipf(s=1.1) token ids, weights are random-init.  ``--impl reference`` runs the unmodified
reference package from ``baseline/_ref`` through its own ``Trainer`` on the same config and data.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent
VOCAB, SEQ, MICRO_BATCH = 49152, 2048, 16
METRIC = "training tokens/sec (IMU-1 430M, seq 2048, micro-batch 16/GPU, bf16)"
MODEL_DESC = "IMU-1 430M (30 layers, d 1152, 18q/6kv heads x 64, SwiGLU 3072, vocab 49152)"
# Further configurations of this package's own arm (``--model``); the headline (and the reference arm) is ``imu1``.
MODELS = {
    "imu1": None,
    "moe": dict(yaml="imu1_moe.yaml", key=None, seq=2048, micro_batch=8, overrides={"trainer.dist_mode": "ddp_ep"},
                metric="training tokens/sec (IMU-1 MoE 16 experts top-2, seq 2048, micro-batch 8/GPU, bf16)",
                desc="IMU-1 attention stack, every FFN a 16-expert top-2 SwiGLU MoE (expert width 768, capacity 1.25, aux 0.01)"),
    "dense_1p5b": dict(yaml="dense_1p5b.yaml", key=None, seq=4096, micro_batch=4, overrides={},
                       metric="training tokens/sec (dense 1.5B, seq 4096, micro-batch 4/GPU, bf16, activation recompute)",
                       desc="dense 1.5B (24 layers, d 2048, 16q/4kv heads x 128, SwiGLU 5632, vocab 49152)"),
}


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    p.add_argument("--config-key", type=str, default="bench")
    p.add_argument("--no-e2e", action="store_true", help="skip the end-to-end phase")
    p.add_argument("--no-check", action="store_true", help="multi-GPU runs: skip the comparison of the NVLink kernels with torch.distributed collectives before timing")
    p.add_argument("--model", type=str, default="imu1", choices=sorted(MODELS), help="imu1 is the headline configuration")
    return p.parse_args()


# ----------------------------------------------------------------------------- helpers
def zipf_tokens(n: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    ranks = np.arange(1, VOCAB + 1, dtype=np.float64)
    cdf = np.cumsum(ranks**-1.1)
    cdf /= cdf[-1]
    return np.searchsorted(cdf, rng.random(n)).astype(np.uint16)


def make_dataset(root: Path, n_tokens: int = 8_000_000) -> tuple[Path, Path]:
    """Train directory with two .npy shards and a single-file validation set of Zipf ids."""
    train = root / "train"
    train.mkdir(parents=True, exist_ok=True)
    toks = zipf_tokens(n_tokens, 0)
    half = n_tokens // 2
    np.save(train / "shard_000.npy", toks[:half])
    np.save(train / "shard_001.npy", toks[half:])
    val = root / "val.npy"
    np.save(val, zipf_tokens(300_000, 1))
    return train, val


class ClockSampler:
    """Samples SM clock and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if n_gpus > 1 and world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} needs a torchrun launch with {n_gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def barrier_sync(world: int):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms: float, world: int) -> float:
    if world == 1:
        return ms
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


HOST_ENQUEUE_MS: list[float] = []


def timed_loop(step_fn, n_steps: int, world: int) -> float:
    """Milliseconds for n_steps calls of step_fn(i), device-timed, max over ranks."""
    barrier_sync(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    t0 = time.perf_counter()
    for i in range(n_steps):
        step_fn(i)
    e1.record()
    HOST_ENQUEUE_MS.append((time.perf_counter() - t0) * 1e3 / max(n_steps, 1))  # host time to enqueue one step
    barrier_sync(world)
    return max_over_ranks(e0.elapsed_time(e1), world)


def emit(args, world, rank, ms_dev, ms_e2e, launches, clocks, impl, extra_cfg, h2d, d2h):
    if rank != 0:
        return
    global_batch = MICRO_BATCH * world
    tokens = global_batch * SEQ * args.steps
    value = tokens / (ms_dev / 1e3)
    e2e_val = tokens / (ms_e2e / 1e3) if ms_e2e else None
    line = {
        "metric": extra_cfg.pop("_metric", METRIC),
        "value": value,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_dev / args.steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic Zipf(s=1.1) token ids, random-init weights",
        "impl": impl,
        "config": {
            "model": extra_cfg.pop("_desc", MODEL_DESC),
            "global_batch": global_batch,
            "seq_len": SEQ,
            "parallelism": f"dp{world}",
            "grad_accum": 1,
            "optimizer": "NorMuonCWD + AdamW, every step",
            "l2_policy": "per-step working set (activations > 40 GB) far exceeds the 126 MB L2; a new batch every step",
            **extra_cfg,
        },
        "clocks": clocks,
        "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": (ms_e2e / args.steps) if ms_e2e else None},
        "gpu_launches": launches,
        "host_enqueue_ms_per_step": round(HOST_ENQUEUE_MS[0], 2) if HOST_ENQUEUE_MS else None,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- our implementation
def run_ours(args):
    global SEQ, MICRO_BATCH
    world, rank, local = dist_setup(args.gpus)
    from sample_efficient_gpt_b200 import ops
    from sample_efficient_gpt_b200.training.trainer import Trainer
    from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, load_cfg

    if ops.ext() is None:
        raise SystemExit(f"CUDA extension is not built: {ops.ext_error()!r}")
    tmp = Path(tempfile.mkdtemp(prefix="segpt_bench_"))
    if rank == 0:
        make_dataset(tmp)
    if world > 1:
        obj = [str(tmp)]
        dist.broadcast_object_list(obj, src=0)
        tmp = Path(obj[0])
    spec = MODELS[args.model]
    extra = {}
    if spec is None:
        cfg = load_cfg(str(ROOT / "sample_efficient_gpt_b200/configs/imu1_base.yaml"), args.config_key)
    else:
        SEQ, MICRO_BATCH = spec["seq"], spec["micro_batch"]
        cfg = load_cfg(str(ROOT / "sample_efficient_gpt_b200/configs" / spec["yaml"]), spec["key"])
        cfg = apply_overrides(cfg, {"trainer.ema_every": 10, **(spec["overrides"] if world > 1 else {})})
        extra = {"_metric": spec["metric"], "_desc": spec["desc"]}
    cfg = apply_overrides(cfg, {
        "data.train_path": str(tmp / "train"), "data.validation_path": str(tmp / "val.npy"), "data.tokenizer_path": "",
        "data.batch_size": MICRO_BATCH * world, "data.context_length": SEQ,
        "trainer.save_dir": str(tmp / "ckpt"), "trainer.device": f"cuda:{local}", "trainer.dtype": "bfloat16",
        "trainer.gradient_accumulation_steps": 1, "trainer.load_from": None, "trainer.log_every": 10**9,
        "optim.shard_muon": world > 1, "trainer.comm_backend": os.environ.get("SEGPT_COMM_BACKEND", "auto"),
    })
    cfg.optim.lr, cfg.optim.muon_lr = float(cfg.optim.lr), float(cfg.optim.muon_lr)
    trainer = Trainer(cfg)
    comm = "symm-p2p" if (trainer.ddp is not None and trainer.ddp.comm is not None) else ("nccl" if world > 1 else "none")

    # device-resident batches for the device-timed phase (a different one each step)
    n_dev = args.warmup + args.steps
    g = torch.Generator().manual_seed(1234 + rank)
    pool = torch.from_numpy(zipf_tokens(4_000_000, 99 + rank).astype(np.int32))
    starts = torch.randint(0, pool.numel() - SEQ - 1, (n_dev, MICRO_BATCH), generator=g)
    idx = starts[..., None] + torch.arange(SEQ + 1)
    windows = pool[idx].cuda()  # [n_dev, MB, SEQ+1]

    def dev_step(i, base=0):
        w = windows[base + i]
        trainer.train_step(w[:, :-1], w[:, 1:])
        trainer.iteration += 1

    for i in range(args.warmup):
        dev_step(i)
    comm_check = None
    if trainer.ddp is not None and trainer.ddp.comm is not None and not args.no_check:
        from sample_efficient_gpt_b200.parallel.comm_check import run_all

        torch.cuda.synchronize()
        comm_check = run_all(trainer.ddp.comm, with_experts=args.model == "moe")  # raises on every rank when a comparison fails
    sampler = ClockSampler(local)
    sampler.start()
    l0 = ops.launch_count
    ms_dev = timed_loop(lambda i: dev_step(i, args.warmup), args.steps, world)
    launches = ops.launch_count - l0
    clocks = sampler.stop()

    ms_e2e, h2d, d2h = None, 0, 0
    if not args.no_e2e:
        sink = []

        def e2e_step(_i):
            x, y = trainer.fetch_batch()  # pinned host -> device
            log = trainer.train_step(x, y)
            trainer.iteration += 1
            sink.append(float(log["train_loss"]))  # device -> host read of the step's loss

        for i in range(max(1, min(args.warmup, 2))):
            e2e_step(i)
        ms_e2e = timed_loop(e2e_step, args.steps, world)
        h2d = 2 * MICRO_BATCH * SEQ * 4
        d2h = 4
    if trainer.ddp is not None and trainer.ddp.comm is not None:
        trainer.ddp.comm.check()  # raises if a bounded wait on a peer gave up during the run
    emit(args, world, rank, ms_dev, ms_e2e, launches, clocks, "ours",
         {"comm": comm, "sharded_muon": bool(cfg.optim.shard_muon), "ema_every": cfg.trainer.ema_every,
          "block_gemm": os.environ.get("SEGPT_BLOCK_GEMM", "native"), "attention": os.environ.get("SEGPT_ATTN_IMPL", "native"),
          **({"comm_check": comm_check} if comm_check else {}), **extra}, h2d, d2h)
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------- the reference
def make_tokenizer(path: Path):
    """A local 49152-entry word-level tokenizer: the reference trainer only calls decode() on it."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    vocab = {f"t{i}": i for i in range(VOCAB)}
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="t0"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="t0").save_pretrained(str(path))


def run_reference(args):
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "sample_efficient_gpt").exists():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed (offline pip install of the reference package into baseline/_ref)"}))
        return
    sys.path.insert(0, str(ref_root))
    os.environ.setdefault("WANDB_MODE", "disabled")
    os.environ.setdefault("NO_VAL", "1")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    world, rank, local = dist_setup(args.gpus)
    try:
        from sample_efficient_gpt.training.trainer import Trainer
        from sample_efficient_gpt.utils.config_tools import apply_overrides, load_config_from_yaml
    except Exception as e:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"[:300]}))
        return
    tmp = Path(tempfile.mkdtemp(prefix="segpt_ref_"))
    if rank == 0:
        make_dataset(tmp)
        make_tokenizer(tmp / "tok")
    if world > 1:
        obj = [str(tmp)]
        dist.broadcast_object_list(obj, src=0)
        tmp = Path(obj[0])
    yaml_path = ref_root / "sample_efficient_gpt" / "configs" / "imu1_base.yaml"
    cfg = load_config_from_yaml(yaml_path, "stable")
    # The reference keeps about 176 GB of activations at 16 x 2048 tokens per GPU and runs out of memory on a
    # 180 GB B200, so its arm runs the same 16 sequences per GPU and optimizer step as two accumulated
    # micro-batches of 8 (SEGPT_REF_MICRO_BATCH=16 tries the single micro-batch).
    ref_mb = int(os.environ.get("SEGPT_REF_MICRO_BATCH", "8"))
    ga = MICRO_BATCH // ref_mb
    cfg = apply_overrides(cfg, {
        "data.train_path": str(tmp / "train"), "data.validation_path": str(tmp / "val.npy"),
        "data.tokenizer_path": str(tmp / "tok"), "data.batch_size": ref_mb * world, "data.context_length": SEQ,
        "trainer.save_dir": str(tmp / "ckpt"), "trainer.load_from": None, "trainer.gradient_accumulation_steps": ga,
        "trainer.log_every": 10**9, "optim.lr": float(cfg.optim.lr), "optim.muon_lr": float(cfg.optim.muon_lr),
        "optim.zero_lr_steps": 0,
    })
    trainer = Trainer(cfg, compile=True)
    bs = cfg.data.batch_size
    sink = []

    def step(_i, read_loss=False):
        """One optimizer step = ``ga`` reference iterations (its train loop body, training/trainer.py:623-628)."""
        for _ in range(ga):
            inputs, targets = trainer.train_dataset.get_batch(bs)
            inputs, targets = inputs.to(cfg.trainer.device), targets.to(cfg.trainer.device)
            log = trainer.train_step(inputs, targets)
            trainer.iteration += 1
        if read_loss:
            sink.append(float(log["train_loss"]))

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(local)
    sampler.start()
    ms_dev = timed_loop(step, args.steps, world)
    clocks = sampler.stop()
    ms_e2e = None
    if not args.no_e2e:
        ms_e2e = timed_loop(lambda i: step(i, True), args.steps, world)
    emit(args, world, rank, ms_dev, ms_e2e, 0, clocks, "reference",
         {"comm": "nccl" if world > 1 else "none", "compile": True, "micro_batch": ref_mb, "grad_accum": ga,
          "note": "reference Trainer.train_step; 16 sequences per GPU and optimizer step as grad_accum micro-batches "
                  "(a single 16 x 2048 micro-batch exceeds 180 GB in the reference); batches come from its own loader "
                  "(host->device every iteration) in both phases"},
         2 * MICRO_BATCH * SEQ * 4, 4)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if not torch.cuda.is_available():
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device"}))
            return
        raise SystemExit("bench.py needs a CUDA device")
    if args.impl == "reference":
        try:
            run_reference(args)
        except Exception as e:  # the reference arm must not take the harness down
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:400]}))
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
