import math

import pytest
import torch

from sample_efficient_gpt_b200.models import Transformer
from sample_efficient_gpt_b200.models.moe import MoEFeedForward, route


def test_routing_capacity_and_weights():
    torch.manual_seed(0)
    probs = torch.rand(10, 4).softmax(-1)
    idx, w, pos, keep = route(probs, 2, capacity=3)
    assert torch.allclose(w.sum(-1), torch.ones(10))
    seen = {e: 0 for e in range(4)}
    for t in range(10):
        for c in range(2):
            e = int(idx[t, c])
            assert int(pos[t, c]) == seen[e] and bool(keep[t, c]) == (seen[e] < 3)
            seen[e] += 1
    assert torch.equal(idx, probs.topk(2, -1).indices)


def test_moe_matches_per_token_loop_and_aux_loss():
    torch.manual_seed(1)
    m = MoEFeedForward(32, n_experts=4, top_k=2, d_ff=64, capacity_factor=8.0, aux_loss_weight=0.01)  # nothing dropped
    x = torch.randn(2, 5, 32)
    y = m(x)
    xt = x.reshape(-1, 32)
    probs = (xt @ m.router.linear.weight.t()).softmax(-1)
    want = torch.zeros_like(xt)
    for t in range(xt.size(0)):
        wv, ev = probs[t].topk(2)
        wv = wv / wv.sum()
        for wgt, e in zip(wv, ev):
            u = m.experts.up[int(e)] @ xt[t]
            g, v = u.chunk(2)
            want[t] += wgt * (m.experts.down[int(e)] @ (torch.nn.functional.silu(g) * v))
    assert torch.allclose(y.reshape(-1, 32), want, atol=1e-5)
    frac = torch.nn.functional.one_hot(probs.topk(2).indices.reshape(-1), 4).float().mean(0)
    assert torch.allclose(m.last_aux_loss, 0.01 * 4 * (frac * probs.mean(0)).sum(), atol=1e-7)
    assert float(m.last_drop_fraction) == 0.0
    y.sum().backward()
    assert all(p.grad is not None for p in m.parameters())


def test_token_dropping_at_low_capacity():
    torch.manual_seed(2)
    m = MoEFeedForward(16, n_experts=4, top_k=2, d_ff=64, capacity_factor=0.5)
    x = torch.randn(1, 16, 16)
    assert m.capacity(16) == math.ceil(0.5 * 16 * 2 / 4) == 4
    m(x)
    assert float(m.last_drop_fraction) > 0.0


def test_moe_transformer_trains_and_names():
    torch.manual_seed(3)
    moe = dict(n_experts=4, top_k=2, d_ff=64, capacity_factor=1.25, aux_loss_weight=0.01)
    t = Transformer(2, 64, 32, 2, 64, attn_qknorm=True, attn_val_residual=True, attn_gating="per-head", moe=moe)
    keys = set(t.state_dict())
    assert {"blocks.0.ffn.router.linear.weight", "blocks.0.ffn.experts.up.0", "blocks.1.ffn.experts.down.3"} <= keys
    ids = torch.randint(0, 64, (2, 8))
    logits, _ = t(ids)
    loss = logits.square().mean() + t.aux_loss()
    loss.backward()
    assert t.blocks[0].ffn.router.linear.weight.grad.abs().sum() > 0


def _moe_model(seed=0, **kw):
    from sample_efficient_gpt_b200.models import Transformer

    torch.manual_seed(seed)
    moe = dict(n_experts=4, top_k=2, d_ff=64, capacity_factor=kw.pop("capacity_factor", 1.25), aux_loss_weight=0.05)
    return Transformer(2, 200, 64, 4, 128, attn_qknorm=True, attn_val_residual=True, attn_gating="per-head", layernorm_scaling=True,
                       n_kv_heads=2, weight_tying=True, moe=moe, **kw)


def test_engine_moe_with_recompute_matches_autograd():
    """First block recomputed in the backward sweep (activation checkpointing): routing is recomputed identically and the
    load-balance terms are recorded once."""
    from sample_efficient_gpt_b200.training.engine import FusedEngine
    from sample_efficient_gpt_b200.training.loss import efficient_cross_entropy

    m = _moe_model(num_grad_checkpoint_layers=1)
    ids = torch.randint(0, 200, (2, 24))
    tg = torch.randint(0, 200, (2, 24))
    logits, _ = m(ids)
    loss, _, _ = efficient_cross_entropy(logits, tg)
    aux = m.aux_loss()
    (loss + aux).backward()
    want = {n: p.grad.clone() for n, p in m.named_parameters()}
    for p in m.parameters():
        p.grad = None
    eng = FusedEngine(m, torch.float32)
    out = eng.forward_backward(ids, tg, 1.0)
    assert float(out.aux_loss) == pytest.approx(float(aux), rel=1e-5) and len(eng.moe.aux_terms) == 2
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, want[n], rtol=2e-3, atol=1e-6 + 1e-4 * float(want[n].abs().max())), n


@pytest.mark.parametrize("cf", [1.25, 0.6])
def test_engine_moe_matches_autograd(cf):
    """Hand-scheduled MoE forward/backward (routing, dispatch, grouped GEMMs, combine, router backward incl. the
    load-balance term and dropped assignments) against autograd of the module path."""
    from sample_efficient_gpt_b200.training.engine import FusedEngine, engine_supports
    from sample_efficient_gpt_b200.training.loss import efficient_cross_entropy

    m = _moe_model(capacity_factor=cf)
    assert engine_supports(m)
    ids = torch.randint(0, 200, (2, 24))
    tg = torch.randint(0, 200, (2, 24))
    logits, _ = m(ids)
    loss, _, _ = efficient_cross_entropy(logits, tg)
    aux = m.aux_loss()
    ((loss + aux) * 0.5).backward()
    want = {n: p.grad.clone() for n, p in m.named_parameters()}
    if cf < 1:
        assert float(m.blocks[0].ffn.last_drop_fraction) > 0  # the small capacity really drops assignments
    for p in m.parameters():
        p.grad = None
    eng = FusedEngine(m, torch.float32)
    out = eng.forward_backward(ids, tg, 0.5)
    assert float(out.loss) == pytest.approx(float(loss), rel=1e-5) and float(out.aux_loss) == pytest.approx(float(aux), rel=1e-5)
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, want[n], rtol=2e-3, atol=1e-6 + 1e-4 * float(want[n].abs().max())), n
    eng.forward_backward(ids, tg, 0.5, first_micro_step=False)
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, 2 * want[n], rtol=2e-3, atol=1e-6 + 2e-4 * float(want[n].abs().max())), n
    assert float(eng.forward_loss(ids, tg).loss) == pytest.approx(float(loss), rel=1e-5)


def test_route_bwd_statement_matches_autograd():
    from sample_efficient_gpt_b200.ops import moe as M

    torch.manual_seed(3)
    logits = torch.randn(17, 6, requires_grad=True)
    probs = logits.softmax(-1)
    w, idx = probs.topk(2, -1)
    wn = w / w.sum(-1, keepdim=True)
    dw = torch.randn(17, 2)
    aux = torch.rand(6)
    ((wn * dw).sum() + (probs * aux).sum()).backward()
    got = M.route_bwd(probs.detach(), idx.int(), dw, aux)
    assert torch.allclose(got, logits.grad, atol=1e-6)
