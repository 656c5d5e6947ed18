"""Worker for the multi-process tests; launched by torchrun from test_ddp_gloo.py / test_gpu_multi.py.

Modes: ``ddp_cpu`` (gloo ranks on CPU), ``comm_gpu`` and ``train_gpu`` (one rank per GPU, NCCL bootstrap).
Prints ``WORKER-OK <mode>`` from rank 0 on success; any assertion makes the launcher exit non-zero.
"""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from sample_efficient_gpt_b200.models import Transformer  # noqa: E402
from sample_efficient_gpt_b200.optim import NorMuonCWD  # noqa: E402
from sample_efficient_gpt_b200.parallel.ddp import DDP, assign_buckets  # noqa: E402
from sample_efficient_gpt_b200.training.engine import FusedEngine  # noqa: E402
from sample_efficient_gpt_b200.training.loss import efficient_cross_entropy  # noqa: E402


def tiny_model(device):
    torch.manual_seed(7)
    m = Transformer(2, 512, 64, 4, 128, attn_qknorm=True, attn_val_residual=True, attn_gating="per-head", layernorm_scaling=True,
                    n_kv_heads=2, weight_tying=True)
    return m.to(device)


def ddp_cpu(rank, world):
    m = tiny_model("cpu")
    if rank != 0:  # DDP must overwrite this with rank 0's weights
        with torch.no_grad():
            for p in m.parameters():
                p.add_(1.0)
    ddp = DDP(m, bucket_size_mb=0.05)
    assert len(ddp.bucket_names) > 3
    names = [n for b in ddp.bucket_names for n in b]
    assert names == [n for n, _ in reversed(list(m.named_parameters()))]
    ref = tiny_model("cpu")
    for a, b in zip(m.parameters(), ref.parameters()):
        assert torch.equal(a, b), "broadcast from rank 0 failed"
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 512, (4, 16), generator=g)
    tg = torch.randint(0, 512, (4, 16), generator=g)
    # reference: full batch on one process
    logits, _ = ref(ids)
    loss, _, _ = efficient_cross_entropy(logits, tg)
    loss.backward()
    # autograd path: each rank takes half the batch, loss pre-scaled by local/global
    sl = slice(rank * 2, rank * 2 + 2)
    logits, _ = ddp(ids[sl])
    loss, _, _ = efficient_cross_entropy(logits, tg[sl])
    (loss * 0.5).backward()
    ddp.finish_gradient_synchronization()
    for (n, a), b in zip(m.named_parameters(), ref.parameters()):
        assert torch.allclose(a.grad, b.grad, rtol=0.05, atol=2e-3 * float(b.grad.abs().max()) + 1e-6), f"autograd path {n}"
    # engine path with explicit grads_ready notifications and no_sync accumulation
    ddp.zero_grad()
    eng = FusedEngine(m, torch.float32)
    eng.grad_ready = ddp.grads_ready
    with ddp.no_sync():
        eng.forward_backward(ids[sl], tg[sl], 0.25, first_micro_step=True)
    eng.forward_backward(ids[sl], tg[sl], 0.25, first_micro_step=False)
    ddp.finish_gradient_synchronization()
    for (n, a), b in zip(m.named_parameters(), ref.parameters()):
        assert torch.allclose(a.grad, b.grad, rtol=0.05, atol=2e-3 * float(b.grad.abs().max()) + 1e-6), f"engine path {n}"
    # sharded NorMuon == unsharded NorMuon on identical gradients
    ps_a = [torch.nn.Parameter(p.detach().clone()) for p in ref.parameters() if p.ndim == 2 and p.shape[0] != 512]
    ps_b = [torch.nn.Parameter(p.detach().clone()) for p in ps_a]
    oa = NorMuonCWD(ps_a, lr=0.02, momentum=0.9, weight_decay=0.1, shard=True)
    ob = NorMuonCWD(ps_b, lr=0.02, momentum=0.9, weight_decay=0.1, shard=False)
    assert oa.is_distributed and not ob.is_distributed
    for step in range(3):
        gg = torch.Generator().manual_seed(100 + step)
        for p, q in zip(ps_a, ps_b):
            gr = torch.randn(p.shape, generator=gg)
            p.grad, q.grad = gr.clone(), gr.clone()
        ra, rb = oa.step(), ob.step()
        assert abs(float(ra) - float(rb)) < 1e-5
    for p, q in zip(ps_a, ps_b):
        assert torch.allclose(p, q, atol=1e-6), "sharded Muon diverged from the unsharded step"
    oa.consolidate_state()
    sa, sb = oa.state_dict(), ob.state_dict()
    for k in sb["state"]:
        assert torch.allclose(sa["state"][k]["momentum_buffer"], sb["state"][k]["momentum_buffer"], atol=1e-6)


def comm_gpu(rank, world):
    from sample_efficient_gpt_b200.parallel.symm import SymmComm

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    for use_mm in ([False, True] if os.environ.get("SEGPT_TEST_MULTIMEM", "0") == "1" else [False]):
        comm = SymmComm.create(dev, use_multimem=use_mm, blocks=8)
        align = comm.bucket_alignment()
        sizes = [align * 3, align * 1000, align * 17 + 0, 4 * 1024 * 1024 // align * align]
        ranges, off = [], 0
        for s in sizes:
            ranges.append((off, off + s))
            off += s
        flat = torch.zeros(off, device=dev)
        comm.register_buckets(flat, ranges)
        for it in range(3):
            torch.manual_seed(1000 * it + rank)
            flat.copy_(torch.randn(off, device=dev))
            want = flat.to(torch.bfloat16).float()
            dist.all_reduce(want)
            for bi in range(len(ranges)):
                comm.all_reduce_bucket(bi)
            comm.wait_all()
            torch.cuda.synchronize()
            comm.check()
            bad = (flat - want).abs() > want.abs() * 2.0**-7 + 1e-6  # one unit in the last place of the bf16 result
            assert not bool(bad.any()), f"all-reduce differs from the fp32 sum of the bf16 inputs at {int(bad.sum())} elements (multimem={use_mm})"
            gathered = [torch.empty_like(flat) for _ in range(world)]
            dist.all_gather(gathered, flat)
            for g in gathered:
                assert torch.equal(g, flat), "ranks ended with different reduced values"
        rows = 5
        buf = comm.symm_zeros((world * rows, 48, 64), torch.bfloat16)
        for it in range(2):
            buf.zero_()
            buf[rank * rows : (rank + 1) * rows] = float(rank + 1 + it)
            torch.cuda.synchronize()
            dist.barrier()
            comm.all_gather_inplace(buf, rows)
            torch.cuda.synchronize()
            comm.check()
            for r in range(world):
                assert torch.all(buf[r * rows : (r + 1) * rows] == float(r + 1 + it)), "all-gather mismatch"
        # the same comparisons that bench.py runs on its live communicator, plus the expert-parallel exchange
        from sample_efficient_gpt_b200.parallel import comm_check

        comm_check.check_bucket_allreduce(comm)
        comm_check.check_gemm_allgather(comm)
        comm_check.check_expert_exchange(comm)


def train_gpu(rank, world):
    """Two optimizer steps of a small model: NVLink-kernel communicator vs torch.distributed collectives."""
    import numpy as np

    from sample_efficient_gpt_b200.training.trainer import Trainer
    from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, load_cfg

    local = int(os.environ.get("LOCAL_RANK", "0"))
    results = {}
    for backend in ("nccl", "p2p"):
        cfg = load_cfg("tiny_cpu.yaml")
        cfg = apply_overrides(cfg, {"trainer.device": f"cuda:{local}", "trainer.dtype": "bfloat16", "trainer.comm_backend": backend,
                                    "model.vocab_size": 4096, "data.batch_size": 4 * world, "optim.shard_muon": True,
                                    "trainer.save_dir": "/tmp/segpt_multi", "trainer.bucket_size_mb": 1.0})
        tr = Trainer(cfg)
        assert (tr.ddp.comm is not None) == (backend == "p2p")
        g = torch.Generator().manual_seed(5 + rank)
        for _ in range(3):
            w = torch.randint(0, 4096, (4, 257), generator=g).cuda()
            tr.train_step(w[:, :-1], w[:, 1:])
            tr.iteration += 1
        torch.cuda.synchronize()
        if tr.ddp.comm is not None:
            tr.ddp.comm.check()
        results[backend] = [p.detach().clone() for p in tr.model.parameters()]
        flat = torch.cat([p.flatten() for p in results[backend]])
        other = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(other, flat)
        for o in other:
            assert torch.equal(o, flat), f"{backend}: ranks diverged"
    for a, b in zip(results["nccl"], results["p2p"]):
        assert torch.allclose(a, b, atol=3e-2, rtol=0.1), (a - b).abs().max()


def moe_ep_cpu(rank, world):
    """Expert parallelism through the engine on gloo ranks: each rank holds half of the experts and half of the batch;
    gradients must equal those of one process holding everything (no drops, no load-balance term: both depend on
    how the batch is split)."""
    moe = dict(n_experts=4, top_k=2, d_ff=64, capacity_factor=4.0, aux_loss_weight=0.0)
    kw = dict(attn_qknorm=True, attn_val_residual=True, attn_gating="per-head", layernorm_scaling=True, n_kv_heads=2, weight_tying=True)
    torch.manual_seed(11)
    full = Transformer(2, 256, 64, 4, 128, moe=dict(moe), **kw)
    torch.manual_seed(11)
    part = Transformer(2, 256, 64, 4, 128, moe=dict(moe, ep_group=dist.group.WORLD), **kw)
    assert len(part.blocks[0].ffn.experts.up) == 2
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 256, (4, 12), generator=g)
    tg = torch.randint(0, 256, (4, 12), generator=g)
    logits, _ = full(ids)
    loss, _, _ = efficient_cross_entropy(logits, tg)
    loss.backward()
    from sample_efficient_gpt_b200.ops.moe import TorchExchange

    eng = FusedEngine(part, torch.float32, moe_exchange=TorchExchange(4, dist.group.WORLD))
    sl = slice(rank * 2, rank * 2 + 2)
    out = eng.forward_backward(ids[sl], tg[sl], 0.5)
    want = dict(full.named_parameters())
    for n, p in part.named_parameters():
        if ".experts." in n:
            kind, e = n.rsplit(".", 2)[-2:]
            ref_p = want[n.rsplit(".", 1)[0] + f".{int(e) + rank * 2}"]
            assert torch.equal(p, ref_p), f"expert init differs: {n}"
            got = p.grad
        else:
            ref_p = want[n]
            got = p.grad.clone()
            dist.all_reduce(got)
        assert torch.allclose(got, ref_p.grad, rtol=2e-3, atol=1e-6 + 1e-4 * float(ref_p.grad.abs().max())), n
    # a step with drops and the load-balance term: runs, stays finite, expert state dict names global ids
    moe2 = dict(n_experts=4, top_k=2, d_ff=64, capacity_factor=0.7, aux_loss_weight=0.05, ep_group=dist.group.WORLD)
    torch.manual_seed(3)
    m2 = Transformer(2, 256, 64, 4, 128, moe=moe2, **kw)
    e2 = FusedEngine(m2, torch.float32, moe_exchange=TorchExchange(4, dist.group.WORLD))
    o2 = e2.forward_backward(ids[sl], tg[sl], 0.5)
    assert torch.isfinite(o2.loss) and float(o2.aux_loss) > 0
    assert all(torch.isfinite(p.grad).all() for p in m2.parameters())
    keys = [k for k in m2.state_dict() if ".experts.up." in k and k.startswith("blocks.0.")]
    assert sorted(int(k.rsplit(".", 1)[1]) for k in keys) == [rank * 2, rank * 2 + 1]


def moe_gpu(rank, world):
    """Expert-parallel exchange over peer memory against all_to_all_single, then a few optimizer steps of an MoE model with
    dist_mode=ddp_ep on both communication backends."""
    from sample_efficient_gpt_b200.ops import moe as M
    from sample_efficient_gpt_b200.parallel.symm import SymmComm
    from sample_efficient_gpt_b200.training.trainer import Trainer
    from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, load_cfg

    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    comm = SymmComm.create(dev)
    E, k, T, d = 4 * world, 2, 1500, 256
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T, d, generator=g).to(dev).bfloat16()
    wr = (torch.randn(E, d, generator=torch.Generator().manual_seed(7)) * 0.2).to(dev)
    cap = M.capacity(T, k, E, 0.9)
    probs, idx, w, slot, totals = M.route(x, wr, k, cap)
    from sample_efficient_gpt_b200.ops import gemm as G

    ref = M.TorchExchange(E, dist.group.WORLD)
    eye = torch.eye(d, device=dev, dtype=torch.bfloat16).expand(E // world, d, d).contiguous()
    for overlap in (False, True):
        peer = M.PeerExchange(E, comm, overlap=overlap)
        assert peer.overlap == overlap
        for scaled in (None, w):
            peer.begin_step()
            got, arrival = peer.dispatch("t", x, idx, slot, totals, scaled, cap)
            want, _ = ref.dispatch("t", x, idx, slot, totals, scaled, cap)
            assert (arrival is not None) == overlap
            # "experts" = identity: the grouped GEMM consumes the dispatched rows (waiting per source region on the arrival
            # flags in the overlapped mode) and produces the rows that the combine returns
            out_t, route = peer.expert_output("y", tuple(want.shape), torch.bfloat16, dev)
            yb = G.gemm(got, eye, out=out_t, wait=arrival, route=route)
            gv = torch.randn(T, d, generator=g).to(dev).bfloat16()
            out, dots = peer.collect("y", yb, idx, slot, scaled, cap, torch.float32, dot_key="y", dot_buf=yb, g=gv)
            rout, rdots = ref.collect("y", want, idx, slot, scaled, cap, torch.float32, dot_buf=want, g=gv)
            torch.cuda.synchronize()
            assert G.status() == 0
            assert torch.allclose(out, rout, atol=2e-2, rtol=2e-2), f"combine mismatch (overlap={overlap})"
            assert torch.allclose(dots, rdots, atol=0.5, rtol=3e-2), f"dots mismatch (overlap={overlap})"
    comm.check()

    results = {}
    for backend in ("nccl", "p2p"):
        cfg = load_cfg("tiny_cpu.yaml")
        cfg = apply_overrides(cfg, {"trainer.device": f"cuda:{local}", "trainer.dtype": "bfloat16", "trainer.comm_backend": backend,
                                    "trainer.dist_mode": "ddp_ep", "model.vocab_size": 4096, "data.batch_size": 4 * world,
                                    "model.n_experts": 2 * world, "model.moe_top_k": 2, "model.moe_d_ff": 128,
                                    "model.moe_capacity_factor": 1.25, "model.moe_aux_loss_weight": 0.01,
                                    "optim.shard_muon": True, "trainer.save_dir": "/tmp/segpt_moe", "trainer.bucket_size_mb": 1.0})
        tr = Trainer(cfg)
        assert tr.engine is not None and tr.engine.moe is not None
        assert isinstance(tr.engine.moe.ex, M.PeerExchange if backend == "p2p" else M.TorchExchange)
        gg = torch.Generator().manual_seed(5 + rank)
        for _ in range(3):
            wds = torch.randint(0, 4096, (4, 257), generator=gg).cuda()
            log = tr.train_step(wds[:, :-1], wds[:, 1:])
            tr.iteration += 1
        torch.cuda.synchronize()
        assert torch.isfinite(log["train_loss"]) and float(log["moe_aux_loss"]) > 0
        if tr.ddp.comm is not None:
            tr.ddp.comm.check()
        results[backend] = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
        shared = torch.cat([p.flatten() for n, p in results[backend].items() if ".experts." not in n])
        other = [torch.empty_like(shared) for _ in range(world)]
        dist.all_gather(other, shared)
        for o in other:
            assert torch.equal(o, shared), f"{backend}: replicated parameters diverged"
    for n in results["nccl"]:
        a, b = results["nccl"][n], results["p2p"][n]
        assert torch.allclose(a, b, atol=3e-2, rtol=0.1), (n, float((a - b).abs().max()))


def moe_ckpt_cpu(rank, world):
    """Expert-parallel trainer on gloo ranks: a checkpoint holds every rank's experts and their optimizer state in the layout
    of a single process; it reloads under expert parallelism (each rank finds its own experts and state) and in one
    process; with clipping on, replicated parameters stay bit-identical across ranks."""
    import tempfile

    from sample_efficient_gpt_b200.training.trainer import Trainer
    from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, load_cfg

    tmp = [tempfile.mkdtemp(prefix="segpt_epckpt_") if rank == 0 else None]
    dist.broadcast_object_list(tmp, src=0)
    over = {"trainer.device": "cpu", "trainer.dtype": "float32", "trainer.dist_mode": "ddp_ep", "model.vocab_size": 512,
            "data.batch_size": 2 * world, "data.context_length": 32, "model.n_experts": 2 * world, "model.moe_top_k": 2,
            "model.moe_d_ff": 64, "model.moe_capacity_factor": 2.0, "model.moe_aux_loss_weight": 0.01, "trainer.save_dir": tmp[0],
            "trainer.clip_fix": True, "trainer.max_grad_norm": 0.05, "trainer.ema_every": 1, "data.train_path": "", "data.validation_path": ""}
    cfg = apply_overrides(load_cfg("tiny_cpu.yaml"), over)
    tr = Trainer(cfg)
    assert len(tr.optimizers) == 3 and tr.ep_group is not None
    g = torch.Generator().manual_seed(5 + rank)
    for _ in range(3):
        w = torch.randint(0, 512, (2, 33), generator=g)
        log = tr.train_step(w[:, :-1], w[:, 1:])
        tr.iteration += 1
    assert float(log["grad_norm"]) > 0.05, "the test wants clipping to be active"
    norms = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(norms, log["grad_norm"].reshape(1).float())
    assert all(torch.equal(n, norms[0]) for n in norms), "every rank must see the same global gradient norm"
    shared = torch.cat([p.detach().flatten() for n, p in tr.model.named_parameters() if ".experts." not in n])
    other = [torch.empty_like(shared) for _ in range(world)]
    dist.all_gather(other, shared)
    assert all(torch.equal(o, shared) for o in other), "replicated parameters diverged under clipping"
    tr.save_state()
    dist.barrier()
    path = Path(tmp[0]) / f"{tr.iteration}.pt"
    ck = torch.load(path, map_location="cpu", weights_only=False)
    E = 2 * world
    for kind in ("up", "down"):
        keys = sorted(int(k.rsplit(".", 1)[1]) for k in ck["model"] if k.startswith(f"blocks.0.ffn.experts.{kind}."))
        assert keys == list(range(E)), f"file holds experts {keys}"
    ema = torch.load(Path(tmp[0]) / f"{tr.iteration}_ema.pt", map_location="cpu", weights_only=False)["model"]
    assert sum(k.startswith("blocks.0.ffn.experts.up.") for k in ema) == E
    assert len(ck["optimizer"]) == 2
    # this rank's experts and their momentum are in the file under their global ids
    mine = {n: p for n, p in tr.model.named_parameters() if ".experts." in n}
    for n, p in mine.items():
        head, e = n.rsplit(".", 1)
        assert torch.equal(ck["model"][f"{head}.{int(e) + rank * 2}"], p.detach()), n
    # reload under expert parallelism: parameters and optimizer state come back exactly
    tr2 = Trainer(cfg, load_from=str(path))
    assert tr2.iteration == tr.iteration
    for (n, a), (_, b) in zip(tr.model.named_parameters(), tr2.model.named_parameters()):
        assert torch.equal(a, b), f"parameter {n} after reload"
    for oa, ob in zip(tr.optimizers, tr2.optimizers):
        for ga, gb in zip(oa.param_groups, ob.param_groups):
            for pa, pb in zip(ga["params"], gb["params"]):
                for k, v in oa.state[pa].items():
                    if torch.is_tensor(v):
                        assert torch.equal(v, ob.state[pb][k]), f"optimizer state {k} after reload"
    # one more step from both: identical results
    w = torch.randint(0, 512, (2, 33), generator=torch.Generator().manual_seed(77 + rank))
    la, lb = tr.train_step(w[:, :-1], w[:, 1:]), tr2.train_step(w[:, :-1], w[:, 1:])
    assert torch.allclose(la["train_loss"], lb["train_loss"]), (float(la["train_loss"]), float(lb["train_loss"]))
    for (n, a), (_, b) in zip(tr.model.named_parameters(), tr2.model.named_parameters()):
        assert torch.allclose(a, b, atol=1e-6), f"{n} differs by {float((a - b).abs().max())} one step after the reload"
    dist.barrier()
    if rank == 0:  # the same file in a process that holds all experts (what a single-GPU user or a converter sees)
        from sample_efficient_gpt_b200.models import build_model
        from sample_efficient_gpt_b200.utils.config_tools import load_config

        full = build_model(load_config(ck["config"]).model, device="cpu", dtype=torch.float32)
        missing = full.load_state_dict(ck["model"], strict=True)
        assert not missing.missing_keys and not missing.unexpected_keys
        n_mats = sum(1 for n, p in full.named_parameters() if p.ndim >= 2 and not any(k in n for k in ("embedding", "lm_head", ".router.")))
        assert sum(len(g["params"]) for g in ck["optimizer"][1]["param_groups"]) == n_mats
        from sample_efficient_gpt_b200.optim import NorMuonCWD

        opt = NorMuonCWD([p for n, p in full.named_parameters() if p.ndim >= 2 and not any(k in n for k in ("embedding", "lm_head", ".router."))])
        opt.load_state_dict(ck["optimizer"][1])  # group structure and shapes match a freshly built optimizer
        for grp in opt.param_groups:
            for p in grp["params"]:
                assert opt.state[p]["momentum_buffer"].shape == p.shape


def main():
    mode = sys.argv[1]
    cuda = mode.endswith("_gpu")
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    try:
        {"ddp_cpu": ddp_cpu, "moe_ep_cpu": moe_ep_cpu, "comm_gpu": comm_gpu, "train_gpu": train_gpu, "moe_gpu": moe_gpu,
         "moe_ckpt_cpu": moe_ckpt_cpu}[mode](rank, world)
        dist.barrier()
        if rank == 0:
            print(f"WORKER-OK {mode}", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
