import math

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
