"""Two gloo ranks on CPU: bucketing plumbing, gradient equality with a single process, sharded NorMuon."""

import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run_workers(mode: str, nproc: int, port: int, timeout: int = 240, env_extra=None):
    env = dict(os.environ)
    env.update(env_extra or {})
    env["OMP_NUM_THREADS"] = "2"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(ROOT / "tests" / "dist_worker.py"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert r.returncode == 0 and f"WORKER-OK {mode}" in r.stdout, (r.stdout[-3000:], r.stderr[-3000:])


def test_two_rank_gloo_ddp_and_sharded_muon():
    run_workers("ddp_cpu", 2, 29631)


def test_two_rank_expert_parallel_engine():
    run_workers("moe_ep_cpu", 2, 29633)


def test_two_rank_expert_parallel_checkpoint_and_clipping():
    run_workers("moe_ckpt_cpu", 2, 29635)


def test_bucket_assignment_rule():
    import torch

    from sample_efficient_gpt_b200.parallel.ddp import assign_buckets

    named = [(f"p{i}", torch.empty(n)) for i, n in enumerate([10, 300, 200, 50, 600, 10])]
    b = assign_buckets(named, 1024)  # bytes; walk in reverse, new bucket when the next tensor would overflow
    assert b == [["p5"], ["p4"], ["p3", "p2"], ["p1"], ["p0"]]
