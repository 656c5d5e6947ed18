"""Fused CUDA paths of the optimizers against the batched PyTorch statement of the same update."""

import pytest
import torch

from sample_efficient_gpt_b200 import ops
from sample_efficient_gpt_b200.optim import AdamW, Muon, NorMuon, NorMuonCWD

pytestmark = pytest.mark.gpu
SHAPES = [(256, 128), (256, 128), (256, 128), (128, 384), (128, 384), (18, 256), (18, 256), (192, 192)]


def _run(cls, fused: bool, steps=3, with_shadows=True):
    torch.manual_seed(0)
    ps = [torch.nn.Parameter((torch.randn(s) * 0.1).cuda()) for s in SHAPES]
    opt = cls(ps, lr=0.02, momentum=0.9, weight_decay=0.1)
    if with_shadows:
        for p in ps:
            opt.lowp_shadows[p] = p.detach().to(torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(1)
    if not fused:
        ops._DISABLED.add("muon_fused")
    try:
        ratios = []
        for _ in range(steps):
            for p in ps:
                p.grad = torch.randn(p.shape, device="cuda", generator=g)
            ratios.append(float(opt.step()))
    finally:
        ops._DISABLED.discard("muon_fused")
    return ps, opt, ratios


@pytest.mark.parametrize("cls", [NorMuonCWD, NorMuon, Muon])
def test_fused_muon_step_matches_unfused(cls):
    assert ops.has_kernel("muon_tail") and ops.has_kernel("gemm")
    before = ops.launch_count
    pf, of, rf = _run(cls, True)
    assert ops.launch_count > before
    pu, ou, ru = _run(cls, False)
    torch.manual_seed(0)
    init = [(torch.randn(s) * 0.1).cuda() for s in SHAPES]
    for a, b, p0 in zip(pf, pu, init):
        da, db = (a.detach() - p0).flatten(), (b.detach() - p0).flatten()
        cos = torch.nn.functional.cosine_similarity(da, db, dim=0)
        assert cos > 0.995, f"{tuple(a.shape)}: update cosine {cos}"
        assert (da.norm() / db.norm() - 1).abs() < 0.02
        sh = of.lowp_shadows[a]
        assert torch.equal(sh, a.detach().to(torch.bfloat16))
    for x, y in zip(rf, ru):
        assert x == pytest.approx(y, rel=2e-2)
    for a, b in zip(pf, pu):
        sa, sb = of.state[a], ou.state[b]
        assert torch.allclose(sa["momentum_buffer"], sb["momentum_buffer"], atol=1e-6)
        if "second_momentum_buffer" in sa:
            assert torch.allclose(sa["second_momentum_buffer"], sb["second_momentum_buffer"], rtol=0.05, atol=1e-8)


def test_fused_adamw_matches_foreach_path():
    torch.manual_seed(2)
    shapes = [(1000,), (64, 300), (1,)]
    a = [torch.nn.Parameter(torch.randn(s).cuda()) for s in shapes]
    b = [torch.nn.Parameter(p.detach().clone()) for p in a]
    oa = AdamW(a, lr=1e-2, betas=(0.9, 0.99), weight_decay=0.1)
    ob = AdamW(b, lr=1e-2, betas=(0.9, 0.99), weight_decay=0.1)
    for _ in range(3):
        gs = [torch.randn(s).cuda() for s in shapes]
        for p, q, g in zip(a, b, gs):
            p.grad, q.grad = g.clone(), g.clone()
        oa.step()
        ops._DISABLED.add("adamw")
        try:
            ob.step()
        finally:
            ops._DISABLED.discard("adamw")
    for p, q in zip(a, b):
        assert torch.allclose(p, q, atol=1e-6)
        assert oa.state[p]["t"] == 4
