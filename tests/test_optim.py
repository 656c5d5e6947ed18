import pytest
import torch

from sample_efficient_gpt_b200.optim import AdamW, Muon, NorMuon, NorMuonCWD, SGD, clip_grad_norm_, newton_schulz
from sample_efficient_gpt_b200.optim.newton_schulz import POLAR_EXPRESS_COEFFS


def test_adamw_golden():
    # values produced by the reference AdamW (training/optimizer.py:33-112)
    p = torch.nn.Parameter(torch.tensor([1.0, -2.0, 3.0]))
    opt = AdamW([p], lr=6e-3, betas=(0.95, 0.99), weight_decay=0.0)
    p.grad = torch.tensor([0.1, -0.2, 0.3])
    opt.step()
    assert torch.allclose(p.data, torch.tensor([0.994, -1.994, 2.994]), atol=1e-6)
    st = opt.state[p]
    assert st["t"] == 2 and torch.allclose(st["m"], torch.tensor([0.005, -0.01, 0.015]), atol=1e-8)
    assert torch.allclose(st["v"], torch.tensor([1e-4, 4e-4, 9e-4]), atol=1e-9)
    p.grad = torch.tensor([0.1, 0.2, -0.3])
    opt.step()
    assert torch.allclose(p.data, torch.tensor([0.98800004, -1.99415386, 2.99415374]), atol=2e-6)


def test_adamw_zeroes_nan_grads_and_sgd():
    p = torch.nn.Parameter(torch.ones(3))
    opt = AdamW([p], lr=1e-2, weight_decay=0.0)
    p.grad = torch.tensor([float("nan"), 1.0, 1.0])
    opt.step()
    assert torch.isfinite(p).all() and p[0] == 1.0
    q = torch.nn.Parameter(torch.ones(2))
    s = SGD([q], lr=1.0)
    q.grad = torch.ones(2)
    s.step(); s.step()
    assert torch.allclose(q.data, torch.ones(2) - 1 - 1 / 2**0.5)


def _ns_oracle(G):
    X = G.to(torch.bfloat16)
    tr = G.size(-2) > G.size(-1)
    if tr:
        X = X.mT
    X = X / (X.norm() + 1e-7)
    for a, b, c in POLAR_EXPRESS_COEFFS:
        A = (X.float() @ X.float().mT).to(torch.bfloat16)
        B = (b * A.float() + c * (A.float() @ A.float())).to(torch.bfloat16)
        X = (a * X.float() + B.float() @ X.float()).to(torch.bfloat16)
    return X.mT if tr else X


def test_newton_schulz_matches_oracle_and_orthogonalises():
    torch.manual_seed(0)
    for shape in [(48, 96), (96, 48), (64, 64)]:
        G = torch.randn(shape)
        X = newton_schulz(G)
        assert X.shape == G.shape and X.dtype == torch.bfloat16
        assert torch.allclose(X.float(), _ns_oracle(G).float(), atol=2e-2)
        s = torch.linalg.svdvals(X.float())
        assert s.max() < 1.3 and s.min() > 0.5
    Gb = torch.randn(3, 32, 64)
    Xb = newton_schulz(Gb)
    for i in range(3):
        assert torch.allclose(Xb[i].float(), newton_schulz(Gb[i]).float(), atol=2e-2)


def _normuon_cwd_naive(ps, grads, state, lr, wd, mu, beta2=0.95):
    """Per-matrix restatement of training/optimizers/normuon_cwd.py:13-31,67-113."""
    sq = 0.0
    for p, g in zip(ps, grads):
        st = state.setdefault(id(p), {})
        if not st:
            st["m"] = torch.zeros_like(g)
            st["s"] = torch.zeros_like(g[..., 0:1]) if p.size(-2) >= p.size(-1) else torch.zeros_like(g[0:1, ...])
        st["m"].lerp_(g, 1 - mu)
        gg = g.lerp(st["m"], mu)
        v = newton_schulz(gg.bfloat16()).float()
        vn = v.norm()
        vm = (v * v).mean(-1, keepdim=True) if p.size(-2) >= p.size(-1) else (v * v).mean(-2, keepdim=True)
        st["s"].lerp_(vm, 1 - beta2)
        v = v * torch.rsqrt(st["s"].clamp_min(1e-10))
        v = v * (vn / v.norm().clamp_min(1e-10))
        mask = torch.eq(torch.signbit(v), torch.signbit(p)).float()
        p.sub_(lr * wd * p * mask)
        p.sub_(lr * max(1, p.size(0) / p.size(1)) ** 0.5 * v)
        sq += float(vn) ** 2
    return sq**0.5 / len(ps)


def test_normuon_cwd_matches_naive_loop():
    torch.manual_seed(1)
    shapes = [(32, 16), (32, 16), (16, 48), (24, 24), (16, 48)]
    ps = [torch.nn.Parameter(torch.randn(s) * 0.1) for s in shapes]
    ref_ps = [p.detach().clone() for p in ps]
    opt = NorMuonCWD(ps, lr=0.02, momentum=0.9, weight_decay=0.1)
    assert sorted(len(g["params"]) for g in opt.param_groups) == [1, 2, 2]
    state = {}
    for _ in range(3):
        grads = [torch.randn_like(p) for p in ps]
        for p, g in zip(ps, grads):
            p.grad = g.clone()
        ratio = opt.step()
        with torch.no_grad():
            want = _normuon_cwd_naive(ref_ps, grads, state, 0.02, 0.1, 0.9)
        assert float(ratio) == pytest.approx(want, rel=1e-3)
        for p, r in zip(ps, ref_ps):
            assert torch.allclose(p.data, r, atol=2e-4), (p.data - r).abs().max()
    st = opt.state[ps[0]]
    assert st["momentum_buffer"].shape == (32, 16) and st["second_momentum_buffer"].shape == (32, 1)
    assert opt.state[ps[2]]["second_momentum_buffer"].shape == (1, 48)


def test_muon_family_state_dict_roundtrip():
    torch.manual_seed(2)
    ps = [torch.nn.Parameter(torch.randn(8, 16)) for _ in range(3)]
    opt = NorMuonCWD(ps, lr=0.01)
    for p in ps:
        p.grad = torch.randn_like(p)
    opt.step()
    sd = opt.state_dict()
    assert all(v["momentum_buffer"]._base is None for v in sd["state"].values())  # clones, not views of the stack
    ps2 = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    opt2 = NorMuonCWD(ps2, lr=0.01)
    opt2.load_state_dict(sd)
    for p, q in zip(ps, ps2):
        p.grad = torch.ones_like(p)
        q.grad = torch.ones_like(q)
    opt.step(); opt2.step()
    for p, q in zip(ps, ps2):
        assert torch.allclose(p, q, atol=1e-6)


def test_plain_muon_and_normuon_decay_rules():
    torch.manual_seed(3)
    w = torch.randn(8, 8)
    for cls, decays in ((Muon, True), (NorMuon, False)):
        p = torch.nn.Parameter(w.clone())
        opt = cls([p], lr=0.1, weight_decay=0.5, momentum=0.9)
        p.grad = torch.zeros_like(p)  # zero gradient -> zero update, only decay can move p
        opt.step()
        moved = not torch.allclose(p.data, w)
        assert moved == decays


def test_clip_grad_norm_generator_quirk():
    ps = [torch.nn.Parameter(torch.ones(4)) for _ in range(2)]
    for p in ps:
        p.grad = torch.full((4,), 3.0)
    n = clip_grad_norm_((p for p in ps), 1.0)  # a generator is exhausted by the norm pass: nothing is scaled
    assert float(n) == pytest.approx((9 * 8) ** 0.5) and float(ps[0].grad[0]) == 3.0
    n = clip_grad_norm_(ps, 1.0)
    tot = sum(float(p.grad.square().sum()) for p in ps) ** 0.5
    assert tot == pytest.approx(1.0, rel=1e-4)
