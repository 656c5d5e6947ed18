"""Correctness checks of the NVLink kernels against torch.distributed collectives on a live communicator.

Run by ``bench.py`` before timing (its JSON line then carries ``"comm_check": "ok"``) and by the multi-GPU tests at whatever
world size the box offers.  Every check is collective: all ranks call it, all ranks get the same verdict (failures are
all-reduced before anything is raised, so that no rank leaves while others still wait for it in a kernel).

  * ``check_bucket_allreduce``: the registered gradient buckets are filled with per-rank random values and reduced by the
    bucket kernel; the result must equal the fp32 NCCL/gloo sum of the bf16-rounded inputs to within one bf16 unit in the
    last place, and must be bit-identical on all ranks.
  * ``check_gemm_allgather``: the GEMM epilogue that stores its tiles into every rank's buffer (the all-gather of the
    sharded Newton-Schulz result) against ``all_gather_into_tensor`` of the locally computed products.
  * ``check_expert_exchange``: dispatch + routed grouped GEMM + combine over peer memory against ``all_to_all_single``.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor


def _agree(ok: bool, what: str, device) -> None:
    flag = torch.tensor([0.0 if ok else 1.0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    torch.cuda.synchronize(device)
    if float(flag.item()) > 0:
        raise AssertionError(f"comm check failed on at least one rank: {what}" + ("" if ok else " (this rank)"))


def check_bucket_allreduce(comm, rounds: int = 2) -> None:
    flat, world, rank = comm.flat_grads, comm.world, comm.rank
    assert flat is not None and comm.bucket_ranges, "no gradient buckets are registered with this communicator"
    saved = flat.clone()
    ok, detail = True, ""
    for it in range(rounds):
        g = torch.Generator(device=flat.device).manual_seed(4242 + 97 * it + rank)
        flat.copy_(torch.randn(flat.numel(), device=flat.device, generator=g) * (1.0 + it))
        want = flat.to(torch.bfloat16).float()
        dist.all_reduce(want, group=comm.group)
        comm.take_grad_sq()
        for bi in range(len(comm.bucket_ranges)):
            comm.all_reduce_bucket(bi)
        comm.wait_all()
        torch.cuda.synchronize(flat.device)
        comm.check()
        lo, hi = comm.bucket_ranges[0][0], comm.bucket_ranges[-1][1]
        got, ref = flat[lo:hi], want[lo:hi]
        # the kernel sums the bf16-rounded terms in fp32 in rank order and rounds the sum to bf16: one unit in the last
        # place of bf16 (2^-8 relative for round-to-nearest, doubled for the different summation order) bounds the difference
        tol = ref.abs() * 2.0**-7 + 1e-6
        bad = (got - ref).abs() > tol
        if bool(bad.any()):
            ok, detail = False, f"all-reduce differs from the fp32 sum of bf16 inputs at {int(bad.sum())} of {bad.numel()} elements"
        sq = float(comm.take_grad_sq().item())
        sq_ref = float((got.double() ** 2).sum().item())
        if abs(sq - sq_ref) > 1e-3 * max(sq_ref, 1e-6):
            ok, detail = False, f"sum of squares from inside the kernel {sq} vs {sq_ref}"
        mine = got.contiguous()
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine, group=comm.group)
        if not all(torch.equal(e, mine) for e in everyone):
            ok, detail = False, "ranks ended with different reduced values"
    flat.copy_(saved)
    _agree(ok, "bucket all-reduce: " + detail, flat.device)


def check_gemm_allgather(comm, rows: int = 384, cols: int = 640, per_rank: int = 3) -> None:
    from sample_efficient_gpt_b200.ops import gemm as G

    world, rank, dev = comm.world, comm.rank, comm.device
    buf = comm.symm_zeros((world * per_rank, rows, cols), torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(777 + rank)
    Bm = (torch.randn(per_rank, rows, rows, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    X = (torch.randn(per_rank, rows, cols, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    mine = buf[rank * per_rank : (rank + 1) * per_rank]
    torch.cuda.synchronize(dev)
    dist.barrier(comm.group)
    # Y = 0.7 X + B X, stored into this rank's rows of every rank's buffer from the GEMM's epilogue
    G.gemm(Bm, X, c=X, out=mine, b_mn=True, alpha=1.0, beta=0.7, extra_dst=comm.peer_addresses(mine))
    comm.barrier()
    torch.cuda.synchronize(dev)
    comm.check()
    local = (0.7 * X.float() + torch.bmm(Bm.float(), X.float())).to(torch.bfloat16)
    ref = torch.empty_like(buf)
    dist.all_gather_into_tensor(ref.view(-1), local.contiguous().view(-1), group=comm.group)
    err = (buf.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item()
    ok = G.status() == 0 and err <= 2e-2 * scale
    _agree(ok, f"GEMM epilogue all-gather: max difference {err} at scale {scale}, status {G.status()}", dev)


def check_expert_exchange(comm, n_experts: int | None = None, tokens: int = 1500, d: int = 256, top_k: int = 2) -> None:
    from sample_efficient_gpt_b200.ops import gemm as G
    from sample_efficient_gpt_b200.ops import moe as M

    world, rank, dev = comm.world, comm.rank, comm.device
    E = n_experts or 2 * world
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(tokens, d, generator=g).to(dev).bfloat16()
    wr = (torch.randn(E, d, generator=torch.Generator().manual_seed(7)) * 0.2).to(dev)
    cap = M.capacity(tokens, top_k, E, 0.9)
    probs, idx, w, slot, totals = M.route(x, wr, top_k, cap)
    ref = M.TorchExchange(E, comm.group)
    eye = torch.eye(d, device=dev, dtype=torch.bfloat16).expand(E // world, d, d).contiguous()
    ok, detail = True, ""
    for overlap in (False, True):
        peer = M.PeerExchange(E, comm, overlap=overlap)
        peer.begin_step()
        got, arrival = peer.dispatch("t", x, idx, slot, totals, w, cap)
        want, _ = ref.dispatch("t", x, idx, slot, totals, w, cap)
        out_t, route = peer.expert_output("y", tuple(want.shape), torch.bfloat16, dev)
        yb = G.gemm(got, eye, out=out_t, wait=arrival, route=route)
        gv = torch.randn(tokens, d, generator=g).to(dev).bfloat16()
        out, dots = peer.collect("y", yb, idx, slot, w, cap, torch.float32, dot_key="y", dot_buf=yb, g=gv)
        rout, rdots = ref.collect("y", want, idx, slot, w, cap, torch.float32, dot_buf=want, g=gv)
        torch.cuda.synchronize(dev)
        if G.status() != 0 or not torch.allclose(out, rout, atol=2e-2, rtol=2e-2) or not torch.allclose(dots, rdots, atol=0.5, rtol=3e-2):
            ok, detail = False, f"overlap={overlap}: status {G.status()}, max difference {float((out - rout).abs().max())}"
    comm.check()
    _agree(ok, "expert-parallel exchange: " + detail, dev)


def run_all(comm, with_experts: bool = False) -> str:
    """All checks that apply; returns "ok" (raises on every rank otherwise)."""
    if comm.flat_grads is not None and comm.bucket_ranges:
        check_bucket_allreduce(comm)
    check_gemm_allgather(comm)
    if with_experts:
        check_expert_exchange(comm)
    return "ok"
