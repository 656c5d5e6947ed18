"""CUDA kernels against the plain PyTorch fp32 statement of the same op (ops/reference.py)."""

import pytest
import torch

from sample_efficient_gpt_b200 import ops
from sample_efficient_gpt_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ext():
    e = ops.ext()
    assert e is not None, f"extension not built: {ops.ext_error()!r}"
    return e


def close(a, b, atol, rtol=0.0, name=""):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    bound = atol + rtol * b.abs().max().item()
    assert err <= bound, f"{name}: max err {err} > {bound}"


@pytest.mark.parametrize("d", [256, 1152, 2048, 200])
@pytest.mark.parametrize("bf16", [True, False])
def test_add_rmsnorm(d, bf16):
    torch.manual_seed(0)
    T = 515
    lp = torch.bfloat16 if bf16 else torch.float32
    res = torch.randn(T, d, device=DEV)
    delta = torch.randn(T, d, device=DEV).to(lp)
    gain = torch.rand(d, device=DEV) + 0.5
    for dl in (delta, None):
        x, y, rstd, kurt = _ext().add_rmsnorm_fwd(res, dl, gain, 0.5, 1e-5, bf16, True)
        xr, yr, rr, kr = ref.add_rmsnorm_fwd(res, dl, gain, 0.5, 1e-5, torch.float32, True)
        close(x, xr, 1e-6, name="x")
        close(y, yr, 2e-2 if bf16 else 1e-5, name="y")
        close(rstd, rr, 1e-5, name="rstd")
        close(kurt, kr, 0, 1e-4, name="kurt")
        dy = torch.randn(T, d, device=DEV).to(lp)
        dres_in = torch.randn(T, d, device=DEV)
        for di in (dres_in, None):
            dres, dres_lp, dgain = _ext().add_rmsnorm_bwd(dy, di, xr, gain, rr, 0.5, bf16)
            dr, _, dgr = ref.add_rmsnorm_bwd(dy, di, xr, gain, rr, 0.5, torch.float32)
            close(dres, dr, 1e-4, name="dres")
            close(dres_lp, dr, 3e-2 if bf16 else 1e-4, name="dres_lp")
            close(dgain, dgr, 1e-3, 1e-4, name="dgain")


@pytest.mark.parametrize("bf16", [True, False])
def test_swiglu_and_gate(bf16):
    torch.manual_seed(1)
    lp = torch.bfloat16 if bf16 else torch.float32
    tol = 3e-2 if bf16 else 1e-5
    u = torch.randn(333, 2 * 768, device=DEV).to(lp)
    df = torch.randn(333, 768, device=DEV).to(lp)
    close(_ext().swiglu_fwd(u), ref.swiglu_fwd(u.float()), tol, name="swiglu")
    close(_ext().swiglu_bwd(df, u), ref.swiglu_bwd(df.float(), u.float()), tol, name="dswiglu")
    for hd, H in ((64, 18), (128, 4), (32, 5)):
        o = torch.randn(257, H, hd, device=DEV).to(lp)
        z = torch.randn(257, H, device=DEV).to(lp)
        dg = torch.randn(257, H * hd, device=DEV).to(lp)
        close(_ext().gate_fwd(o, z), ref.gate_fwd(o.float(), z.float()), tol, name="gate")
        do, dz = _ext().gate_bwd(dg, o, z)
        dor, dzr = ref.gate_bwd(dg.float(), o.float(), z.float())
        close(do, dor, tol, name="do")
        close(dz, dzr, 0.25 if bf16 else 1e-4, name="dz")
        # gate logits and their gradient as columns of wider tensors (the fused qkv+gate projection's layout)
        wide = torch.randn(257, H + 40, device=DEV).to(lp)
        zs = wide[:, 8 : 8 + H]
        dwide = torch.full((257, H + 40), 7.0, device=DEV).to(lp)
        close(_ext().gate_fwd(o, zs), ref.gate_fwd(o.float(), zs.float()), tol, name="gate strided")
        do2, dz2 = _ext().gate_bwd(dg, o, zs, dwide[:, 16 : 16 + H])
        dor2, dzr2 = ref.gate_bwd(dg.float(), o.float(), zs.float())
        close(do2, dor2, tol, name="do strided")
        close(dwide[:, 16 : 16 + H], dzr2, 0.25 if bf16 else 1e-4, name="dz strided")
        assert dz2.data_ptr() == dwide[:, 16 : 16 + H].data_ptr()
        assert bool((dwide[:, :16] == 7.0).all()) and bool((dwide[:, 16 + H :] == 7.0).all()), "columns around dz must stay untouched"


@pytest.mark.parametrize("hd,H,Hkv", [(64, 18, 6), (128, 4, 2), (32, 4, 4)])
@pytest.mark.parametrize("bf16", [True, False])
@pytest.mark.parametrize("qknorm", [True, False])
def test_qkv_post(hd, H, Hkv, bf16, qknorm):
    torch.manual_seed(2)
    B, S = 2, 67
    lp = torch.bfloat16 if bf16 else torch.float32
    tol = 4e-2 if bf16 else 1e-4
    from sample_efficient_gpt_b200.models.rope import rope_tables

    cos, sin = rope_tables(128, 10000.0, hd, DEV)
    qkv = torch.randn(B * S, (H + 2 * Hkv) * hd, device=DEV).to(lp)
    v1 = torch.randn(B, S, Hkv, hd, device=DEV).to(lp)
    sc = [torch.tensor([v], device=DEV) for v in (1.3, 0.8, 0.5, 1.1)]
    args = (cos, sin, *sc, B, S, H, Hkv, hd, qknorm)
    for v1_ in (v1, None):
        q, k, v = _ext().qkv_post_fwd(qkv, v1_, *args)
        qr, kr, vr = ref.qkv_post_fwd(qkv.float(), None if v1_ is None else v1_.float(), *args)
        close(q, qr, tol, name="q"); close(k, kr, tol, name="k"); close(v, vr, tol, name="v")
        dq, dk = torch.randn_like(q), torch.randn_like(k)
        for dv in (torch.randn_like(v), torch.randn(v.shape, device=DEV)):
            out = _ext().qkv_post_bwd(dq, dk, dv, qkv, v1_, *args)
            outr = ref.qkv_post_bwd(dq.float(), dk.float(), dv.float(), qkv.float(), None if v1_ is None else v1_.float(), *args)
            close(out[0], outr[0], tol * 2, name="dqkv")
            if v1_ is None:
                assert out[1] is None
            else:
                close(out[1], outr[1], tol, name="dv1")
            for i, nm in zip(range(2, 6), ("dqgain", "da1", "da2", "dvscale")):
                close(out[i], outr[i], 0.5 if bf16 else 1e-2, 2e-3, name=nm)
            if v1_ is not None:  # the running sum over blocks is updated in place
                run = torch.randn(B, S, Hkv, hd, device=DEV)
                before = run.clone()
                out2 = _ext().qkv_post_bwd(dq, dk, dv, qkv, v1_, *args, None, run)
                assert out2[1].data_ptr() == run.data_ptr()
                close(run, before + outr[1], tol, name="dv1 accumulated")


@pytest.mark.parametrize("B,S,extra", [(3, 72, 0), (4, 640, 0), (2, 328, 24), (1, 8, 0)])
@pytest.mark.parametrize("qknorm", [True, False])
def test_qkv_post_shared_memory_variant(B, S, extra, qknorm):
    """bf16, head_dim 64, S a multiple of 8: token rows are staged through shared memory with bulk copies (several tiles
    per CTA, a ragged last tile, and qkv / dqkv as the leading columns of a wider projection output)."""
    from sample_efficient_gpt_b200.models.rope import rope_tables
    from sample_efficient_gpt_b200.ops import gemm as G

    torch.manual_seed(4)
    H, Hkv, hd = 18, 6, 64
    n = (H + 2 * Hkv) * hd
    cos, sin = rope_tables(1024, 10000.0, hd, DEV)
    wide = torch.randn(B * S, n + extra, device=DEV).to(torch.bfloat16)
    qkv = wide[:, :n]
    v1 = torch.randn(B, S, Hkv, hd, device=DEV).to(torch.bfloat16)
    sc = [torch.tensor([v], device=DEV) for v in (1.3, 0.8, 0.5, 1.1)]
    args = (cos, sin, *sc, B, S, H, Hkv, hd, qknorm)
    for v1_ in (v1, None):
        q, k, v = _ext().qkv_post_fwd(qkv, v1_, *args)
        torch.cuda.synchronize()
        assert G.status() == 0
        qr, kr, vr = ref.qkv_post_fwd(qkv.float(), None if v1_ is None else v1_.float(), *args)
        close(q, qr, 4e-2, name="q"); close(k, kr, 4e-2, name="k"); close(v, vr, 4e-2, name="v")
        dq, dk, dv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
        dwide = torch.full((B * S, n + extra), 7.0, device=DEV).to(torch.bfloat16)
        out = _ext().qkv_post_bwd(dq, dk, dv, qkv, v1_, *args, dwide[:, :n])
        torch.cuda.synchronize()
        assert G.status() == 0
        outr = ref.qkv_post_bwd(dq.float(), dk.float(), dv.float(), qkv.float(), None if v1_ is None else v1_.float(), *args)
        close(out[0], outr[0], 8e-2, name="dqkv")
        if extra:
            assert bool((dwide[:, n:] == 7.0).all()), "columns beside dqkv must stay untouched"
        for i, nm in zip(range(2, 6), ("dqgain", "da1", "da2", "dvscale")):
            close(out[i], outr[i], 0.5, 2e-3, name=nm)
        if v1_ is not None:
            close(out[1], outr[1], 4e-2, name="dv1")
            run = torch.randn(B, S, Hkv, hd, device=DEV)
            before = run.clone()
            out2 = _ext().qkv_post_bwd(dq, dk, dv, qkv, v1_, *args, None, run)
            assert out2[1].data_ptr() == run.data_ptr()
            close(run, before + outr[1], 4e-2, name="dv1 accumulated")


def test_ce_chunk():
    torch.manual_seed(3)
    rows, V = 300, 49152
    logits = (torch.randn(rows, V, device=DEV) * 3).to(torch.bfloat16)
    tg = torch.randint(0, V, (rows,), device=DEV)
    tg[5] = -100
    loss = torch.empty(rows, device=DEV); z = torch.empty(rows, device=DEV); lse = torch.empty(rows, device=DEV)
    lr, zr, lser = ref.softmax_ce_fwd(logits.float() * 0.5, tg, 1e-6, -100)
    gr = ref.softmax_ce_bwd(logits.float() * 0.5, tg, lser, torch.full((rows,), 0.01, device=DEV), 1e-6, -100) * 0.5
    work = logits.clone()
    _ext().ce_chunk_fwd_bwd(work, tg, loss, z, lse, 1e-6, -100, 0.01, 0.5, True)
    close(loss, lr, 1e-3, name="loss"); close(z, zr, 1e-6, name="z"); close(lse, lser, 1e-3, name="lse")
    close(work, gr, 1e-4, 1e-2, name="dlogits")
    assert float(work[5].abs().max()) == 0.0 and float(loss[5]) == 0.0
    for Vs in (4096, 1000 * 8, 65536):
        lg = torch.randn(7, Vs, device=DEV).to(torch.bfloat16)
        t2 = torch.randint(0, Vs, (7,), device=DEV)
        l2 = torch.empty(7, device=DEV); z2 = torch.empty(7, device=DEV); s2 = torch.empty(7, device=DEV)
        _ext().ce_chunk_fwd_bwd(lg.clone(), t2, l2, z2, s2, 1e-6, -100, 1.0, 1.0, False)
        close(l2, ref.softmax_ce_fwd(lg.float(), t2, 1e-6, -100)[0], 1e-3, name=f"loss V={Vs}")


def test_fused_linear_ce_matches_reference():
    torch.manual_seed(4)
    T, d, V = 1000, 256, 4096
    h = torch.randn(T, d, device=DEV).to(torch.bfloat16)
    w = (torch.randn(V, d, device=DEV) / d**0.5).to(torch.bfloat16)
    tg = torch.randint(0, V, (T,), device=DEV)
    from sample_efficient_gpt_b200.ops.cross_entropy import linear_ce_fwd_bwd

    loss, z, dh, dw = linear_ce_fwd_bwd(h, w, tg, 1e-6, -100, 1.0 / T, 1.0, chunk=384)
    lr, zr, dhr, dwr = ref.linear_ce_fwd_bwd(h.float(), w.float(), tg, 1e-6, -100, 1.0 / T, 1.0, chunk=512)
    close(loss, lr, 2e-2, name="loss"); close(dh, dhr, 1e-5, 3e-2, name="dh"); close(dw, dwr, 1e-5, 3e-2, name="dW")


def test_multi_tensor_adamw_ema_cast():
    torch.manual_seed(5)
    shapes = [(1000,), (3, 70000), (1,), (257, 129)]
    ps = [torch.randn(s, device=DEV) for s in shapes]
    gs = [torch.randn(s, device=DEV) for s in shapes]
    gs[0][3] = float("nan")
    ms = [torch.randn(s, device=DEV) * 0.1 for s in shapes]
    vs = [torch.rand(s, device=DEV) * 0.1 for s in shapes]
    sh = [torch.empty(s, device=DEV, dtype=torch.bfloat16) if i % 2 == 0 else torch.empty(0, device=DEV) for i, s in enumerate(shapes)]
    rp, rm, rv = [p.clone() for p in ps], [m.clone() for m in ms], [v.clone() for v in vs]
    lr, wd, b1, b2, eps, ss = 1e-2, 0.1, 0.9, 0.99, 1e-8, 0.0123
    _ext().adamw(ps, gs, ms, vs, sh, lr, wd, b1, b2, eps, ss)
    for i in range(len(ps)):
        g = torch.nan_to_num(gs[i], nan=0.0)
        rp[i].mul_(1 - lr * wd); rm[i].mul_(b1).add_(g, alpha=1 - b1); rv[i].mul_(b2).addcmul_(g, g, value=1 - b2)
        rp[i].addcdiv_(rm[i], rv[i].sqrt() + eps, value=-ss)
        close(ps[i], rp[i], 1e-5, name="p"); close(ms[i], rm[i], 1e-6, name="m"); close(vs[i], rv[i], 1e-6, name="v")
        if sh[i].numel():
            close(sh[i], rp[i], 2e-2, name="shadow")
    ema = [torch.randn(s, device=DEV) for s in shapes]
    want = [0.8 * e + 0.2 * p for e, p in zip(ema, ps)]
    _ext().ema(ema, ps, 0.8)
    for e, w in zip(ema, want):
        close(e, w, 1e-6, name="ema")
    dst = [torch.empty(s, device=DEV, dtype=torch.bfloat16) for s in shapes]
    _ext().cast_bf16(dst, ps)
    for d_, p in zip(dst, ps):
        assert torch.equal(d_, p.to(torch.bfloat16))


@pytest.mark.parametrize("B,S,H,Hkv", [(1, 128, 1, 1), (2, 256, 4, 2), (1, 512, 6, 2), (2, 1024, 3, 1), (2, 200, 4, 2), (1, 77, 2, 1), (3, 129, 2, 2), (1, 2048, 3, 1), (1, 1300, 2, 2)])
def test_native_attention_forward(B, S, H, Hkv):
    from sample_efficient_gpt_b200.ops import gemm as G

    assert ops.has_kernel("fa_fwd")
    torch.manual_seed(7)
    q = torch.randn(B, S, H, 64, device=DEV).to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, 64, device=DEV).to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, 64, device=DEV).to(torch.bfloat16)
    o, lse = _ext().fa_fwd(q, k, v, True)
    torch.cuda.synchronize()
    assert G.status() == 0, "a bounded wait inside the attention kernel gave up"
    o_ref, lse_ref = ref.attention_fwd(q.float(), k.float(), v.float(), True, 0)
    close(o, o_ref, 2e-2, 2e-2, name="O")
    close(lse, lse_ref, 2e-2, name="LSE")


@pytest.mark.parametrize("B,S,H,Hkv", [(1, 128, 1, 1), (2, 256, 4, 2), (1, 512, 6, 2), (2, 1024, 3, 1), (1, 2048, 3, 1), (2, 200, 4, 2), (1, 77, 2, 1),
                                       (1, 1300, 2, 2)])
def test_native_attention_backward(B, S, H, Hkv):
    """dq/dk/dv of the tcgen05 backward kernel against autograd of the fp32 statement of the same attention."""
    from sample_efficient_gpt_b200.ops import gemm as G

    assert ops.has_kernel("fa_bwd")
    torch.manual_seed(11)
    q = torch.randn(B, S, H, 64, device=DEV).to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, 64, device=DEV).to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, 64, device=DEV).to(torch.bfloat16)
    do = torch.randn(B, S, H, 64, device=DEV).to(torch.bfloat16)
    o, lse = _ext().fa_fwd(q, k, v, True)
    dq, dk, dv = _ext().fa_bwd(do, q, k, v, o, lse, True)
    torch.cuda.synchronize()
    assert G.status() == 0, "a bounded wait inside the attention kernel gave up"
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    rep = H // Hkv
    kk, vv = kf.repeat_interleave(rep, dim=2), vf.repeat_interleave(rep, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", qf, kk) / 8.0
    s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=DEV), 1), float("-inf"))
    o_ref = torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1), vv)
    o_ref.backward(do.float())
    close(dq, qf.grad, 3e-2, 3e-2, name="dQ")
    close(dk, kf.grad, 3e-2, 3e-2, name="dK")
    close(dv, vf.grad, 3e-2, 3e-2, name="dV")
    for got, want, nm in ((dq, qf.grad, "dQ"), (dk, kf.grad, "dK"), (dv, vf.grad, "dV")):  # relative L2: bf16 rounding level
        rel = float((got.float() - want).norm() / want.norm())
        assert rel < 1.5e-2, f"{nm}: relative L2 error {rel}"


def test_native_attention_stage_timers():
    """The optional stage timers report the walk length of the profiled CTA and leave the results unchanged."""
    torch.manual_seed(5)
    B, S, H, Hkv = 1, 512, 2, 1
    q = torch.randn(B, S, H, 64, device=DEV).to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, 64, device=DEV).to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, 64, device=DEV).to(torch.bfloat16)
    do = torch.randn(B, S, H, 64, device=DEV).to(torch.bfloat16)
    pf = torch.zeros(16, dtype=torch.int64, device=DEV)
    pb = torch.zeros(16, dtype=torch.int64, device=DEV)
    o, lse = _ext().fa_fwd(q, k, v, True)
    o2, lse2 = _ext().fa_fwd(q, k, v, True, pf)
    g = _ext().fa_bwd(do, q, k, v, o, lse, True)
    g2 = _ext().fa_bwd(do, q, k, v, o, lse, True, pb)
    torch.cuda.synchronize()
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    assert torch.equal(g[1], g2[1]) and torch.equal(g[2], g2[2])  # dQ sums in an order that may differ from run to run
    # the forward's profiled CTA holds the last two query tiles and reports the walk of the first of them
    assert pf[15].item() == S // 128 - 1 and pb[15].item() == (H // Hkv) * (S // 128)
    assert pf[:8].sum().item() > 0 and pb[:8].sum().item() > 0
