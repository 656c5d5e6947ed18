"""Gradient-bucket all-reduce bandwidth sweep: this package's NVLink kernels against NCCL.

    torchrun --nproc-per-node 8 -m sample_efficient_gpt_b200.parallel.comm_bench --min-mb 1 --max-mb 512 --out sweep.json
    torchrun --nproc-per-node 8 -m sample_efficient_gpt_b200.parallel.comm_bench --nccl-table      # scripts/nccl_test.py

Per bucket size (MB of fp32 gradients) it times, device-side with CUDA events and as the max over ranks:
  * ``nccl_bf16``   - the reference's path (training/distributed/ddp_bucket.py:91-127): cast fp32 -> bf16, ``all_reduce``,
                      cast back and copy into the gradient views;
  * ``nccl_fp32``   - a plain fp32 ``all_reduce`` (what scripts/nccl_test.py:24-118 measures);
  * ``p2p``         - one kernel per bucket: pack to bf16, reduce-scatter and all-gather over peer loads/stores, unpack;
  * ``multimem``    - the same with NVLS ``multimem`` reductions/stores (when the allocation has a multicast mapping).
Reported: milliseconds, algorithm bandwidth (fp32 bucket bytes / time) and bus bandwidth (bf16 wire bytes x 2(n-1)/n /
time, fp32 bytes for ``nccl_fp32``).  ``--nccl-table`` prints the reference script's three tables (whole / 5 / 50 buckets).
Between timed repetitions a buffer larger than L2 is overwritten.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

L2_FLUSH_BYTES = 256 << 20


def _time_ms(fn, reps: int, warmup: int, flush) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    t = torch.tensor([total / reps], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def sweep(sizes_mb: list[int], reps: int, warmup: int, backends: list[str], blocks: int = 128) -> list[dict]:
    from sample_efficient_gpt_b200.parallel.symm import SymmComm

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    align = 8 * world
    ranges, at = [], 0
    for mb in sizes_mb:
        n = (mb * (1 << 20) // 4 + align - 1) // align * align
        ranges.append((at, at + n))
        at += n
    flat = torch.randn(at, device=dev) * 0.01
    comms = {}
    for name in backends:
        if name in ("p2p", "multimem"):
            try:
                c = SymmComm.create(dev, use_multimem=(name == "multimem"), blocks=blocks)
                c.register_buckets(flat, ranges)
                comms[name] = c
            except RuntimeError as e:
                if rank == 0:
                    print(f"# {name} unavailable: {e}")
    rows = []
    for bi, (mb, (s, e)) in enumerate(zip(sizes_mb, ranges)):
        view = flat[s:e]
        nbytes = (e - s) * 4
        row = {"mb": mb, "world": world, "blocks": blocks}

        def nccl_bf16():
            wire = view.to(torch.bfloat16)
            dist.all_reduce(wire)
            view.copy_(wire)

        def nccl_fp32():
            dist.all_reduce(view)

        fns = {"nccl_bf16": nccl_bf16, "nccl_fp32": nccl_fp32}
        for name, c in comms.items():
            def ours(c=c):
                c.all_reduce_bucket(bi)
                c.wait_all()
            fns[name] = ours
        for name in backends:
            if name not in fns:
                continue
            flat.mul_(0.0).add_(0.01)  # keep magnitudes bounded across repetitions
            ms = _time_ms(fns[name], reps, warmup, flush)
            wire_bytes = nbytes if name == "nccl_fp32" else nbytes // 2
            row[name] = {"ms": ms, "alg_gbs": nbytes / ms / 1e6, "bus_gbs": wire_bytes * 2 * (world - 1) / world / ms / 1e6}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    for c in comms.values():
        c.check()
    return rows


def nccl_table(reps: int = 10, warmup: int = 5) -> list[dict]:
    """Whole buffer / 5 buckets / 50 buckets, 1-1000 MB fp32, MB/s as the mean over ranks."""
    rank, world = dist.get_rank(), dist.get_world_size()
    out = []
    for n_buckets in (1, 5, 50):
        for mb in (1, 10, 100, 1000):
            data = torch.randn(262_144 * mb // n_buckets, device="cuda")
            for _ in range(warmup * n_buckets):
                dist.all_reduce(data)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps * n_buckets):
                dist.all_reduce(data)
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b)], device="cuda")
            dist.all_reduce(t)
            mean_ms = float(t) / world
            out.append({"buckets": n_buckets, "mb": mb, "mb_per_s": mb * reps / (mean_ms / 1e3)})
            data.mul_(0)
    if rank == 0:
        for n_buckets in (1, 5, 50):
            print(f"backend=nccl world_size={world} buckets={n_buckets}")
            print(f"{'MB':>6} {'MB / s':>14}")
            for r in out:
                if r["buckets"] == n_buckets:
                    print(f"{r['mb']:>6} {r['mb_per_s']:>14.1f}")
    return out


def emulate_one_gpu(world: int, mb: int, blocks: int, reps: int) -> dict:
    """The bucket kernel as rank 0 of ``world`` with every rank's wire buffer and flag array on this GPU and all flags set
    in advance, so that no barrier waits: the kernel's own instruction and memory behaviour (what a profiler may look at
    in a single process), without NVLink.  Not a bandwidth number."""
    from sample_efficient_gpt_b200 import ops

    ext = ops.ext()
    n = mb * 1024 * 1024 // 4 // (8 * world) * (8 * world)
    grads = torch.randn(n, device="cuda")
    wires = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    flags = [torch.full((ext.COMM_MAX_BLOCKS * ext.COMM_MAX_RANKS,), 2**30, dtype=torch.int32, device="cuda") for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sq = torch.zeros(1, device="cuda")
    run = lambda: ext.comm_allreduce_bucket(grads, [w.data_ptr() for w in wires], [f.data_ptr() for f in flags], 0, 0, 0, 1, blocks,  # noqa: E731
                                            status, sq, 2_000_000, n)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    out = {"mode": "one GPU plays rank 0, peers' buffers local", "world": world, "mb": mb, "blocks": blocks, "ms": e0.elapsed_time(e1) / reps,
           "status": int(status.item())}
    print(json.dumps(out), flush=True)
    return out


def gemm_allgather(rows: int, cols: int, total: int, reps: int, warmup: int) -> dict:
    """The last GEMM of a sharded Newton-Schulz chain: each rank computes ``a X + B X`` for its share of ``total`` matrices
    ([rows, rows] x [rows, cols]) and the epilogue stores every tile into all ranks' buffers (``extra_dst`` = the peers'
    copies), followed by the device barrier (the reference leaves its matrix ownership commented out,
    training/optimizers/normuon_cwd.py:60-62, and every rank orthogonalises every matrix).  Timed against the same GEMM with a local output only, and against that GEMM
    followed by ``all_gather_into_tensor``; roofline = max(FLOPs at the measured cuBLAS rate, bytes that leave this GPU
    over NVLink at 770 GB/s)."""
    from sample_efficient_gpt_b200.ops import gemm as G
    from sample_efficient_gpt_b200.parallel.symm import SymmComm

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    comm = SymmComm.create(dev)
    per = (total + world - 1) // world
    buf = comm.symm_zeros((world * per, rows, cols), torch.bfloat16)
    mine = buf[rank * per : (rank + 1) * per]
    local = torch.empty_like(mine)
    gathered = torch.empty_like(buf)
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    Bm = (torch.randn(per, rows, rows, device=dev, generator=g) * 0.03).to(torch.bfloat16)
    X = (torch.randn(per, rows, cols, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    peers = comm.peer_addresses(mine)

    def fused():
        G.gemm(Bm, X, c=X, out=mine, b_mn=True, alpha=1.0, beta=0.7, extra_dst=peers)
        comm.barrier()

    def local_only():
        G.gemm(Bm, X, c=X, out=local, b_mn=True, alpha=1.0, beta=0.7)

    def gemm_then_nccl():
        G.gemm(Bm, X, c=X, out=local, b_mn=True, alpha=1.0, beta=0.7)
        dist.all_gather_into_tensor(gathered.view(-1), local.view(-1))

    out = {"world": world, "matrices_per_rank": per, "shape": [rows, cols]}
    for name, fn in (("gemm_local_only", local_only), ("gemm_epilogue_allgather", fused), ("gemm_then_nccl_allgather", gemm_then_nccl)):
        out[name + "_ms"] = _time_ms(fn, reps, warmup, flush)
    torch.cuda.synchronize()
    comm.check()
    assert G.status() == 0
    flops = per * 2.0 * rows * rows * cols
    link_bytes = (world - 1) * per * rows * cols * 2
    out["flops_ms_at_1390_tflops"] = flops / 1389.6e12 * 1e3
    out["link_ms_at_770_gbs"] = link_bytes / 770e9 * 1e3
    out["roofline_ms"] = max(out["flops_ms_at_1390_tflops"], out["link_ms_at_770_gbs"])
    out["fused_over_roofline"] = out["gemm_epilogue_allgather_ms"] / out["roofline_ms"] if out["roofline_ms"] > 0 else None
    if rank == 0:
        print(json.dumps(out), flush=True)
    return out


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--emulate-ranks", type=int, default=0, help="single process, one GPU: run the bucket kernel as rank 0 of N with local stand-ins for the peers (profiling)")
    p.add_argument("--mb", type=int, default=32, help="--emulate-ranks: bucket size")
    p.add_argument("--min-mb", type=int, default=1)
    p.add_argument("--max-mb", type=int, default=512)
    p.add_argument("--reps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--backends", default="nccl_bf16,nccl_fp32,p2p,multimem")
    p.add_argument("--blocks", type=int, default=128, help="CTAs of the NVLink kernels (training uses 32 to leave SMs to the backward pass)")
    p.add_argument("--nccl-table", action="store_true")
    p.add_argument("--gemm-allgather", action="store_true", help="time the GEMM whose epilogue stores its tiles into every rank's buffer (sharded Newton-Schulz)")
    p.add_argument("--rows", type=int, default=1152)
    p.add_argument("--cols", type=int, default=3072)
    p.add_argument("--matrices", type=int, default=30)
    p.add_argument("--out", default=None)
    a = p.parse_args(argv)
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if a.emulate_ranks > 1:
        emulate_one_gpu(a.emulate_ranks, a.mb, a.blocks, a.reps)
        return
    dist.init_process_group("nccl")
    try:
        if a.gemm_allgather:
            rows = [gemm_allgather(a.rows, a.cols, a.matrices, a.reps, a.warmup)]
        elif a.nccl_table:
            rows = nccl_table()
        else:
            sizes, mb = [], a.min_mb
            while mb <= a.max_mb:
                sizes.append(mb)
                mb *= 2
            rows = sweep(sizes, a.reps, a.warmup, a.backends.split(","), a.blocks)
        if a.out and dist.get_rank() == 0:
            os.makedirs(os.path.dirname(a.out) or ".", exist_ok=True)
            with open(a.out, "w") as f:
                json.dump(rows, f, indent=1)
    finally:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
