"""Hand-scheduled forward/backward of the mixture-of-experts feed-forward block, used by ``FusedEngine`` in place of
the dense SwiGLU when a block has experts.  Specification: models/moe.py (the reference has no MoE).

Per block, forward:
    route (softmax router, top-k, slots)  ->  dispatch (permute + all-to-all into the owners' buffers)
    ->  grouped up GEMM  ->  SwiGLU  ->  grouped down GEMM  ->  combine (all-to-all back + un-permute + weighted sum)
backward: the mirrored chain (dispatch of ``w * dout``, the four grouped gradient GEMMs, combine of ``dx`` together with the
dot products that give the routing-weight gradients), then the router backward (renormalisation, load-balance term,
softmax) and the two small router GEMMs.

"Grouped" = one batched GEMM over this rank's experts: buffers have the fixed shape ``[E_local, world * cap, d]``, expert
weights are kept stacked (``[E_local, 2 f, d]`` and ``[E_local, d, f]``; the per-expert parameters' bf16 shadows and fp32
gradients are views into the stacks), so on a GPU every expert GEMM of a block is a single launch of the tcgen05 GEMM.
Expert weights receive gradients from every rank's tokens through the exchange and therefore take no part in the
data-parallel gradient reduction.
"""

from __future__ import annotations

import torch
from torch import Tensor

from sample_efficient_gpt_b200 import ops
from sample_efficient_gpt_b200.ops import moe as M


def _bmm(a: Tensor, b: Tensor, a_mn: bool, b_mn: bool, out: Tensor | None = None, out_f32: bool = False, accumulate: bool = False,
         wait=None, route=None):
    """Batched ``op(a) @ op(b)``: a is [.., M, K] (or [.., K, M] with a_mn), b is [.., N, K] (or [.., K, N] with b_mn).
    ``wait``: per-source-region arrival flags of ``a`` (see ``ops.gemm.gemm``); only the tcgen05 GEMM can honour them."""
    from sample_efficient_gpt_b200.ops import gemm as G

    if a.dtype == torch.bfloat16 and G.usable(a, b, out) and ops.kernel_enabled("moe_gemm"):
        return G.gemm(a, b, c=out if accumulate else None, out=out, out_f32=out_f32, a_mn=a_mn, b_mn=b_mn, beta=1.0 if accumulate else 0.0,
                      wait=wait, route=route)
    assert wait is None and route is None, "arrival flags and routed outputs need the tcgen05 GEMM"
    A = a.transpose(-1, -2) if a_mn else a
    B = b if b_mn else b.transpose(-1, -2)
    if out_f32 and a.is_cuda and a.dtype != torch.float32:
        res = torch.bmm(A, B, out_dtype=torch.float32)
    else:
        res = torch.bmm(A.float(), B.float()) if out_f32 else torch.bmm(A, B)
    if out is None:
        return res
    if accumulate:
        out.add_(res)
    else:
        out.copy_(res)
    return out


class MoEEngine:
    def __init__(self, engine, exchange=None):
        self.eng = engine
        model = engine.model
        self.blocks = [i for i, b in enumerate(model.blocks) if b.is_moe]
        ffn0 = model.blocks[self.blocks[0]].ffn
        self.E, self.k, self.f = ffn0.n_experts, ffn0.top_k, ffn0.d_ff
        dev = ffn0.router.linear.weight.device
        if exchange is None:
            exchange = M.PeerExchange(self.E, None, dev) if dev.type == "cuda" and engine.lp == torch.bfloat16 and ops.has_kernel("moe_push") \
                else M.TorchExchange(self.E, None)
        self.ex = exchange
        assert self.ex.e_local == ffn0.n_local, "exchange and model disagree about the experts per rank"
        self.up_w, self.down_w, self.up_g, self.down_g = {}, {}, {}, {}
        lp = engine.lp
        for i in self.blocks:
            ex = model.blocks[i].ffn.experts
            ups, downs = list(ex.up), list(ex.down)
            self.up_w[i] = torch.stack([p.detach().to(lp) for p in ups])
            self.down_w[i] = torch.stack([p.detach().to(lp) for p in downs])
            self.up_g[i] = torch.zeros((len(ups), *ups[0].shape), dtype=torch.float32, device=dev)
            self.down_g[i] = torch.zeros((len(downs), *downs[0].shape), dtype=torch.float32, device=dev)
            for e, (pu, pd) in enumerate(zip(ups, downs)):
                engine.shadows[pu], engine.shadows[pd] = self.up_w[i][e], self.down_w[i][e]
        # Gradients: views into the stacks, unless somebody (data parallelism with replicated experts) already placed
        # the parameters' gradients elsewhere - then the stacks are scratch and are copied out after each block.
        first_expert = model.blocks[self.blocks[0]].ffn.experts.up[0]
        self.grads_in_stacks = first_expert.grad is None
        if self.grads_in_stacks:
            for i in self.blocks:
                ex = model.blocks[i].ffn.experts
                for e, (pu, pd) in enumerate(zip(ex.up, ex.down)):
                    pu.grad, pd.grad = self.up_g[i][e], self.down_g[i][e]
        self.aux_terms: list[Tensor] = []
        self.drop_fractions: list[Tensor] = []

    def refresh(self):
        """Re-cast the stacked weights from the fp32 masters (after a checkpoint load)."""
        for i in self.blocks:
            ex = self.eng.model.blocks[i].ffn.experts
            for e, (pu, pd) in enumerate(zip(ex.up, ex.down)):
                self.up_w[i][e].copy_(pu.detach())
                self.down_w[i][e].copy_(pd.detach())

    def begin_step(self):
        self.aux_terms.clear()
        self.drop_fractions.clear()
        self.ex.begin_step()

    def aux_loss(self) -> Tensor | None:
        return torch.stack(self.aux_terms).sum() if self.aux_terms else None

    # ------------------------------------------------------------------------------------------------ forward
    def forward(self, i: int, n2: Tensor, train: bool = True, record: bool = True):
        ffn = self.eng.model.blocks[i].ffn
        T, d = n2.shape
        cap = ffn.capacity(T)
        probs, idx, w, slot, totals = M.route(n2, ffn.router.linear.weight, self.k, cap)
        frac = totals.float() / float(T * self.k)
        if record:  # not when a checkpointed block is recomputed in the backward sweep
            self.aux_terms.append(ffn.aux_loss_weight * self.E * (frac * probs.mean(0)).sum())
            self.drop_fractions.append((slot < 0).float().mean())
        xb, arrival = self.ex.dispatch(("x", i), n2, idx, slot, totals, None, cap)  # [E_local, world * cap, d]
        u = _bmm(xb, self.up_w[i], False, False, wait=arrival)
        a = ops.swiglu_fwd(u.view(-1, u.size(-1))).view(u.size(0), u.size(1), self.f)
        out, route = self.ex.expert_output(("y", i), (xb.size(0), xb.size(1), d), n2.dtype, n2.device)
        yb = _bmm(a, self.down_w[i], False, False, out=out, route=route)  # routed: lands in the source ranks' buffers
        m, _ = self.ex.collect(("y", i), yb, idx, slot, w, cap, n2.dtype)
        saved = (probs, idx, w, slot, totals, frac, cap, xb, u, a, yb) if train else None
        return m, saved

    # ------------------------------------------------------------------------------------------------ backward
    def backward(self, i: int, dm: Tensor, n2: Tensor, saved, loss_coef: float, first: bool) -> Tensor:
        """dm [T, d] (activation dtype): gradient of the block's FFN output.  Returns d(n2) in the activation dtype and
        accumulates the gradients of the router and of this rank's experts."""
        ffn = self.eng.model.blocks[i].ffn
        probs, idx, w, slot, totals, frac, cap, xb, u, a, yb = saved
        T, d = n2.shape
        dyb, arrival = self.ex.dispatch("dy", dm, idx, slot, totals, w, cap)  # rows already scaled by the routing weights
        da = _bmm(dyb, self.down_w[i], False, True, wait=arrival)  # [E_local, R, f]; the later GEMMs follow it on the stream
        acc = (not first) and self.grads_in_stacks
        _bmm(dyb, a, True, True, out=self.down_g[i], out_f32=True, accumulate=acc)
        du = ops.swiglu_bwd(da.view(-1, self.f), u.view(-1, u.size(-1))).view_as(u)
        out, route = self.ex.expert_output("dx", (xb.size(0), xb.size(1), d), dm.dtype, dm.device)
        dxb = _bmm(du, self.up_w[i], False, True, out=out, route=route)
        _bmm(du, xb, True, True, out=self.up_g[i], out_f32=True, accumulate=acc)
        if not self.grads_in_stacks:
            ex = ffn.experts
            for e, (pu, pd) in enumerate(zip(ex.up, ex.down)):
                if first:
                    pu.grad.copy_(self.up_g[i][e]), pd.grad.copy_(self.down_g[i][e])
                else:
                    pu.grad.add_(self.up_g[i][e]), pd.grad.add_(self.down_g[i][e])
        dn2, dots = self.ex.collect("dx", dxb, idx, slot, None, cap, torch.float32, dot_key=("y", i), dot_buf=yb, g=dm)
        aux_vec = frac * (loss_coef * ffn.aux_loss_weight * self.E / T)
        dlogits = M.route_bwd(probs, idx, dots, aux_vec)  # [T, E] fp32
        wr = ffn.router.linear.weight
        gw = dlogits.t() @ n2.float()
        if first:
            wr.grad.copy_(gw)
        else:
            wr.grad.add_(gw)
        dn2.addmm_(dlogits, wr.detach().float())
        return dn2.to(dm.dtype)
