"""MoE kernels (csrc/moe.cu) against the PyTorch statements of ops/moe.py, and the bf16 engine on a GPU against the fp32
engine on the CPU."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(T=1000, d=256, E=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, d, generator=g).cuda().bfloat16()
    wr = (torch.randn(E, d, generator=g) * 0.2).cuda()
    return x, wr


@pytest.mark.parametrize("T,E,k,cf", [(1000, 16, 2, 1.25), (257, 8, 1, 0.5), (4096, 32, 4, 1.0)])
def test_route_and_slots_match_reference(T, E, k, cf):
    from sample_efficient_gpt_b200 import ops
    from sample_efficient_gpt_b200.ops import moe as M

    x, wr = _inputs(T, 256, E)
    cap = M.capacity(T, k, E, cf)
    probs, idx, w, slot, totals = M.route(x, wr, k, cap)
    assert ops.has_kernel("moe_route") and idx.dtype == torch.int32
    ref_probs = (x.float() @ wr.t()).softmax(-1)
    assert torch.allclose(probs, ref_probs, atol=2e-6, rtol=1e-4)
    rw, ridx = ref_probs.topk(k, -1)
    gap_ok = (rw[:, -1] - ref_probs.scatter(1, ridx, -1.0).max(-1).values) > 1e-5 if k < E else torch.ones(T, dtype=torch.bool, device="cuda")
    assert gap_ok.float().mean() > 0.99
    assert torch.equal(idx[gap_ok].long(), ridx[gap_ok])
    assert torch.allclose(w[gap_ok], (rw / rw.sum(-1, keepdim=True))[gap_ok], atol=1e-5)
    # slots: recompute from the kernel's own idx with the reference statement
    flat = idx.long().reshape(-1)
    onehot = torch.nn.functional.one_hot(flat, E)
    pos = (onehot.cumsum(0) - 1).gather(1, flat[:, None]).squeeze(1).reshape(idx.shape)
    assert torch.equal(totals.long(), onehot.sum(0))
    assert torch.equal(slot.long(), torch.where(pos < cap, pos, torch.full_like(pos, -1)))
    if cf < 1:
        assert (slot < 0).any()


@pytest.mark.parametrize("scaled", [False, True])
def test_push_pull_match_reference_single_rank(scaled):
    from sample_efficient_gpt_b200.ops import moe as M

    T, d, E, k = 777, 384, 8, 2
    x, wr = _inputs(T, d, E, seed=1)
    cap = M.capacity(T, k, E, 0.8)
    probs, idx, w, slot, totals = M.route(x, wr, k, cap)
    peer, ref = M.PeerExchange(E, None, "cuda"), M.TorchExchange(E, None)
    ww = w if scaled else None
    peer._buffer("b", cap, d).fill_(7.0)  # stale content: tails must come back as zeros
    got, _ = peer.dispatch("b", x, idx, slot, totals, ww, cap)
    want, _ = ref.dispatch("b", x, idx, slot, totals, ww, cap)
    assert got.shape == want.shape == (E, cap, d)
    assert torch.allclose(got.float(), want.float(), atol=1e-2 if scaled else 0, rtol=1e-2 if scaled else 0)
    y = torch.randn_like(want)
    y2 = torch.randn_like(want)
    g = torch.randn(T, d, device="cuda").bfloat16()
    peer._bufs["y"], peer._bufs["y2"] = y.view(E, 1, cap, d).clone(), y2.view(E, 1, cap, d).clone()
    out, dots = peer.collect("y", peer._bufs["y"].view(E, cap, d), idx, slot, ww, cap, torch.float32, dot_buf=peer._bufs["y2"].view(E, cap, d), g=g)
    rout, rdots = ref.collect("y", y, idx, slot, ww, cap, torch.float32, dot_buf=y2, g=g)
    assert torch.allclose(out, rout, atol=1e-4, rtol=1e-4) and torch.allclose(dots, rdots, atol=2e-3, rtol=1e-3)
    out_lp, none = peer.collect("y", peer._bufs["y"].view(E, cap, d), idx, slot, ww, cap, torch.bfloat16)
    assert none is None and torch.allclose(out_lp.float(), rout, atol=3e-2, rtol=2e-2)


def test_route_bwd_matches_reference():
    from sample_efficient_gpt_b200 import ops
    from sample_efficient_gpt_b200.ops import moe as M

    T, E, k = 999, 16, 2
    probs = torch.randn(T, E, device="cuda").softmax(-1)
    idx = probs.topk(k, -1).indices.int()
    dw = torch.randn(T, k, device="cuda")
    aux = torch.rand(E, device="cuda")
    got = M.route_bwd(probs, idx, dw, aux)
    ops._DISABLED.add("moe")
    try:
        want = M.route_bwd(probs, idx, dw, aux)
    finally:
        ops._DISABLED.discard("moe")
    assert torch.allclose(got, want, atol=1e-6, rtol=1e-4)


def test_engine_moe_bf16_gpu_against_fp32_cpu():
    from sample_efficient_gpt_b200.models import Transformer
    from sample_efficient_gpt_b200.ops import moe as M
    from sample_efficient_gpt_b200.training.engine import FusedEngine

    def build():
        torch.manual_seed(0)
        moe = dict(n_experts=8, top_k=2, d_ff=128, capacity_factor=1.25, aux_loss_weight=0.01)
        return Transformer(2, 512, 256, 4, 512, attn_qknorm=True, attn_val_residual=True, attn_gating="per-head", layernorm_scaling=True,
                           n_kv_heads=2, weight_tying=True, moe=moe)

    ids = torch.randint(0, 512, (4, 256))
    tg = torch.randint(0, 512, (4, 256))
    cpu = build()
    ref = FusedEngine(cpu, torch.float32).forward_backward(ids, tg, 1.0)
    gpu = build().cuda()
    eng = FusedEngine(gpu, torch.bfloat16)
    assert isinstance(eng.moe.ex, M.PeerExchange)
    out = eng.forward_backward(ids.cuda(), tg.cuda(), 1.0)
    torch.cuda.synchronize()
    assert float(out.loss) == pytest.approx(float(ref.loss), rel=2e-2)
    assert float(out.aux_loss) == pytest.approx(float(ref.aux_loss), rel=5e-2)
    worst = {}
    for (n, p), q in zip(gpu.named_parameters(), cpu.parameters()):
        g, r = p.grad.float().cpu(), q.grad
        assert torch.isfinite(g).all(), n
        cos = torch.nn.functional.cosine_similarity(g.flatten(), r.flatten(), dim=0)
        worst[n] = float(cos)
        if r.norm() > 1e-6 and p.ndim >= 2:
            assert cos > 0.95, (n, float(cos))  # bf16 activations + a few tokens routed differently
