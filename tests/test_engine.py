"""The hand-scheduled forward/backward (training/engine.py) against autograd of the module path, on CPU."""

import pytest
import torch

from sample_efficient_gpt_b200.models import Transformer
from sample_efficient_gpt_b200.ops import reference as ref
from sample_efficient_gpt_b200.training.engine import FusedEngine, engine_supports
from sample_efficient_gpt_b200.training.loss import efficient_cross_entropy, fused_linear_cross_entropy


def _model(**kw):
    torch.manual_seed(0)
    base = dict(attn_qknorm=True, attn_val_residual=True, attn_gating="per-head", layernorm_scaling=True, n_kv_heads=2, weight_tying=True)
    base.update(kw)
    m = Transformer(3, 300, 128, 4, 192, **base)
    with torch.no_grad():
        for b in m.blocks:
            if hasattr(b.attn, "sdpa_qknorm"):
                b.attn.sdpa_qknorm.gain.fill_(1.3)
            if b.attn.value_residual:
                b.attn.alpha1.fill_(0.8); b.attn.alpha2.fill_(0.5); b.attn.scale.fill_(1.1)
            b.ln1.gain.add_(torch.randn_like(b.ln1.gain) * 0.1)
    return m


@pytest.mark.parametrize("kw", [dict(), dict(num_grad_checkpoint_layers=2), dict(attn_gating=False, attn_qknorm=False),
                                dict(attn_val_residual=False, n_kv_heads=4), dict(mup_base_width=64)])
def test_engine_gradients_match_autograd(kw):
    m = _model(**kw)
    ids = torch.randint(0, 300, (2, 33))
    tg = torch.randint(0, 300, (2, 33))
    tg[0, 3] = -100
    logits, kurt = m(ids)
    loss, z, _ = efficient_cross_entropy(logits, tg)
    (loss * 0.7).backward()
    want = {n: p.grad.clone() for n, p in m.named_parameters()}
    for p in m.parameters():
        p.grad = None
    eng = FusedEngine(m, torch.float32)
    out = eng.forward_backward(ids, tg, 0.7)
    assert float(out.loss) == pytest.approx(float(loss), rel=1e-5) and float(out.z_loss) == pytest.approx(float(z), rel=1e-4)
    assert torch.allclose(out.kurtosis, kurt, rtol=1e-4)
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, want[n], rtol=2e-3, atol=1e-6 + 1e-4 * float(want[n].abs().max())), n
    eng.forward_backward(ids, tg, 0.7, first_micro_step=False)  # accumulation doubles every gradient
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, 2 * want[n], rtol=2e-3, atol=1e-6 + 2e-4 * float(want[n].abs().max())), n
    ev = eng.forward_loss(ids, tg)
    assert float(ev.loss) == pytest.approx(float(loss), rel=1e-5)
    # the gradients are views of one flat buffer: the global norm is a single reduction over it
    from sample_efficient_gpt_b200.optim.clip import grad_norm

    flat_norm = eng.flat_grad_norm()
    assert flat_norm is not None and float(flat_norm) == pytest.approx(float(grad_norm([p.grad for p in m.parameters()])), rel=2e-4)
    next(m.parameters()).grad = torch.zeros_like(next(m.parameters()))  # a gradient that left the buffer: no shortcut
    assert eng.flat_grad_norm() is None


def test_engine_fused_gate_projection_matches_autograd():
    """qkv and gate projections as one GEMM (gate rows appended to the qkv weight, strided qkv view, [dqkv | dz] gradient)."""
    m = _model()
    ids = torch.randint(0, 300, (2, 33))
    tg = torch.randint(0, 300, (2, 33))
    logits, _ = m(ids)
    loss, _, _ = efficient_cross_entropy(logits, tg)
    loss.backward()
    want = {n: p.grad.clone() for n, p in m.named_parameters()}
    for p in m.parameters():
        p.grad = None
    eng = FusedEngine(m, torch.float32, fuse_gate=True)
    assert len(eng.qkvz_w) == 3 and eng.qkvz_w[0].size(0) % 8 == 0
    out = eng.forward_backward(ids, tg, 1.0)
    assert float(out.loss) == pytest.approx(float(loss), rel=1e-5)
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, want[n], rtol=2e-3, atol=1e-6 + 1e-4 * float(want[n].abs().max())), n
    eng.forward_backward(ids, tg, 1.0, first_micro_step=False)
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, 2 * want[n], rtol=2e-3, atol=1e-6 + 2e-4 * float(want[n].abs().max())), n


def test_engine_rejects_unsupported_models():
    m = _model(attn_gating="elementwise")
    assert not engine_supports(m)
    with pytest.raises(ValueError):
        FusedEngine(m)


def test_loss_definitions_and_fused_linear_ce():
    torch.manual_seed(1)
    h = torch.randn(40, 32, requires_grad=True)
    w = torch.randn(100, 32, requires_grad=True)
    tg = torch.randint(0, 100, (40,))
    tg[7] = -100
    logits = h @ w.t()
    loss, z, bpb = efficient_cross_entropy(logits, tg, per_token_byte_lengths=torch.ones(100) * 2)
    lse = torch.logsumexp(logits, -1)
    per = lse - logits.gather(1, tg.clamp_min(0)[:, None]).squeeze(1) + 1e-6 * lse**2
    per = torch.where(tg == -100, torch.zeros_like(per), per)
    assert torch.allclose(loss, per.mean(), atol=1e-6)  # ignored tokens count in the mean with a zero loss
    assert float(bpb) == pytest.approx(float(per.sum() * 2 / 80 * 1.44269), rel=1e-4)
    gh, gw = torch.autograd.grad(loss, (h, w))
    loss2, z2, _ = fused_linear_cross_entropy(h, w, tg)
    gh2, gw2 = torch.autograd.grad(loss2, (h, w))
    assert torch.allclose(loss, loss2, atol=1e-6) and torch.allclose(z, z2, atol=1e-8)
    assert torch.allclose(gh, gh2, atol=1e-6) and torch.allclose(gw, gw2, atol=1e-6)
    assert not z.requires_grad  # the z-loss value carries no gradient of its own


def test_reference_op_backward_formulas_against_autograd():
    torch.manual_seed(2)
    T, d = 12, 16
    x = torch.randn(T, d, requires_grad=True); g = torch.rand(d, requires_grad=True) + 0.5
    _, y, rstd, _ = ref.add_rmsnorm_fwd(x, None, g, 0.7, 1e-5, torch.float32, False)
    dy = torch.randn(T, d)
    gx, gg = torch.autograd.grad((y * dy).sum(), (x, g))
    dres, _, dgain = ref.add_rmsnorm_bwd(dy, None, x.detach(), g.detach(), rstd.detach(), 0.7, torch.float32)
    assert torch.allclose(dres, gx, atol=1e-5) and torch.allclose(dgain, gg, atol=1e-5)
    u = torch.randn(T, 2 * d, requires_grad=True)
    f = ref.swiglu_fwd(u)
    df = torch.randn(T, d)
    assert torch.allclose(ref.swiglu_bwd(df, u.detach()), torch.autograd.grad((f * df).sum(), u)[0], atol=1e-5)
    q = torch.randn(2, 9, 4, 8, requires_grad=True); k = torch.randn(2, 9, 2, 8, requires_grad=True); v = torch.randn(2, 9, 2, 8, requires_grad=True)
    o, lse = ref.attention_fwd(q, k, v)
    do = torch.randn_like(o)
    want = torch.autograd.grad((o * do).sum(), (q, k, v))
    got = ref.attention_bwd(do, q.detach(), k.detach(), v.detach(), o.detach(), lse.detach())
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=1e-5)


def test_feed_forward_ops_fall_back_to_their_statements_on_cpu():
    """``ops.up_swiglu`` / ``ops.down_dgrad_swiglu`` (one fused launch each on CUDA) are GEMM + SwiGLU statements elsewhere."""
    from sample_efficient_gpt_b200 import ops

    torch.manual_seed(0)
    T, d, F = 37, 24, 16
    x, w_up, w_down = torch.randn(T, d), torch.randn(2 * F, d) * 0.2, torch.randn(d, F) * 0.2
    u, f = ops.up_swiglu(x, w_up)
    assert torch.allclose(u, x @ w_up.T, atol=1e-5)
    assert torch.allclose(f, torch.nn.functional.silu(u[:, :F]) * u[:, F:], atol=1e-5)
    dy = torch.randn(T, d)
    du = ops.down_dgrad_swiglu(dy, w_down, u)
    ur = u.clone().requires_grad_(True)
    (torch.nn.functional.silu(ur[:, :F]) * ur[:, F:]).backward(dy @ w_down)
    assert torch.allclose(du, ur.grad, atol=1e-5)
