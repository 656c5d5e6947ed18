"""Mixture-of-experts feed-forward block (no counterpart in the reference, whose FFN is always dense).

Specification:
  * router: bias-free ``Linear(d_model, n_experts)`` on the normed block input, fp32 softmax, top-k experts per token,
    the k weights renormalised to sum to one;
  * capacity: each expert accepts at most ``ceil(capacity_factor * T * k / E)`` assignments per step (T tokens of the
    local batch), taken in token order; later assignments are dropped (their weight contributes nothing);
  * experts: SwiGLU ``down(silu(gate) * up)`` with the packed ``[gate | up]`` projection, expert width ``d_ff``;
  * auxiliary load-balance loss (Switch): ``aux_weight * E * sum_e f_e * P_e`` with f_e the fraction of assignments
    routed to expert e (before dropping) and P_e the mean router probability of e; stored in ``last_aux_loss`` and
    added to the training loss by the trainer.
Parameters: ``router.linear.weight`` [E, d]; ``experts.up.{e}`` [2*d_ff, d]; ``experts.down.{e}`` [d, d_ff] - one matrix
per expert, so NorMuon orthogonalises every expert separately and batches them by shape like any other matrix.

Expert parallelism (``ep_group`` given): the E experts are split evenly across the ranks of the group; a rank keeps
only its own experts' parameters.  Tokens travel to the ranks of their experts and back with two all-to-alls
(``dispatch`` / ``combine``); both are differentiable, so expert weights receive gradients from every rank's tokens
and need no gradient all-reduce.  ``parallel.expert_parallel`` provides the exchange (NCCL/gloo ``all_to_all_single``).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from sample_efficient_gpt_b200.models.core import Linear, mup_trunc_normal_


class Experts(nn.Module):
    """The experts this rank holds: ``n_local`` consecutive ones out of ``n_total``, starting at ``first_global_id``.

    Initial values are drawn for all ``n_total`` experts in order and only the local ones are kept, so that a model built
    from the same seed has the same experts however they are split over ranks.  State-dict keys carry the *global*
    expert id (``up.{g}`` / ``down.{g}``): a file written by one rank names the experts it holds, and loading picks the
    local ones out of whatever a file offers.
    """

    def __init__(self, n_local: int, d_model: int, d_ff: int, first_global_id: int = 0, n_total: int | None = None, device=None,
                 dtype=None):
        super().__init__()
        self.first_global_id = first_global_id
        self.n_total = n_total if n_total is not None else first_global_id + n_local
        self.up = nn.ParameterList()
        self.down = nn.ParameterList()
        for g in range(self.n_total):
            up = mup_trunc_normal_(torch.empty(2 * d_ff, d_model, dtype=dtype), d_model)
            down = mup_trunc_normal_(torch.empty(d_model, d_ff, dtype=dtype), d_ff)
            if first_global_id <= g < first_global_id + n_local:
                self.up.append(nn.Parameter(up.to(device) if device is not None else up))
                self.down.append(nn.Parameter(down.to(device) if device is not None else down))
        self._register_state_dict_hook(self._globalise_keys)
        self._register_load_state_dict_pre_hook(self._localise_keys)

    @staticmethod
    def _globalise_keys(module, state_dict, prefix, local_metadata):
        if module.first_global_id == 0:
            return state_dict
        for kind in ("up", "down"):
            moved = {e: state_dict.pop(f"{prefix}{kind}.{e}") for e in range(len(getattr(module, kind)))}
            for e, t in moved.items():
                state_dict[f"{prefix}{kind}.{module.first_global_id + e}"] = t
        return state_dict

    def _localise_keys(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        n_local = len(self.up)
        for kind in ("up", "down"):
            offered = {int(k[len(prefix) + len(kind) + 1:]): k for k in list(state_dict) if k.startswith(f"{prefix}{kind}.")}
            picked = {g - self.first_global_id: state_dict.pop(k) for g, k in offered.items()
                      if self.first_global_id <= g < self.first_global_id + n_local}
            for k in offered.values():
                state_dict.pop(k, None)  # experts of other ranks
            for e, t in picked.items():
                state_dict[f"{prefix}{kind}.{e}"] = t

    def forward(self, x: Tensor) -> Tensor:
        """x [E_local, C, d] -> [E_local, C, d]."""
        up = torch.stack(list(self.up)).to(x.dtype)
        down = torch.stack(list(self.down)).to(x.dtype)
        u = torch.bmm(x, up.transpose(1, 2))
        g, v = u.chunk(2, dim=-1)
        return torch.bmm(F.silu(g) * v, down.transpose(1, 2))


def route(probs: Tensor, top_k: int, capacity: int):
    """Top-k routing with capacity.  probs [T, E] fp32.

    Returns (expert [T,k] int64, weight [T,k] fp32 renormalised, position [T,k] int64 slot inside the expert's
    buffer, keep [T,k] bool) - assignments are ranked per expert in (token, choice) order."""
    T, E = probs.shape
    w, idx = probs.topk(top_k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    flat = idx.reshape(-1)  # (token, choice) order
    onehot = F.one_hot(flat, E)
    pos = (onehot.cumsum(0) - 1).gather(1, flat[:, None]).squeeze(1).reshape(T, top_k)
    keep = pos < capacity
    return idx, w, pos, keep


class MoEFeedForward(nn.Module):
    def __init__(self, d_model: int, n_experts: int, top_k: int = 2, d_ff: int = 768, capacity_factor: float = 1.25,
                 aux_loss_weight: float = 0.01, ep_group=None, device=None, dtype=None):
        super().__init__()
        self.d_model, self.n_experts, self.top_k = d_model, n_experts, top_k
        self.d_ff = int(d_ff // 64 * 64) if d_ff >= 64 else d_ff
        self.capacity_factor, self.aux_loss_weight = capacity_factor, aux_loss_weight
        self.ep_group = ep_group
        self.ep_world, self.ep_rank = 1, 0
        if ep_group is not None:
            import torch.distributed as dist

            self.ep_world, self.ep_rank = dist.get_world_size(ep_group), dist.get_rank(ep_group)
            assert n_experts % self.ep_world == 0, "experts must divide evenly across the expert-parallel group"
        self.n_local = n_experts // self.ep_world
        self.router = Linear(d_model, n_experts, device=device, dtype=dtype)
        self.experts = Experts(self.n_local, d_model, self.d_ff, self.ep_rank * self.n_local, n_experts, device=device, dtype=dtype)
        self.last_aux_loss: Tensor | None = None
        self.last_drop_fraction: Tensor | None = None

    def capacity(self, n_tokens: int) -> int:
        return max(1, math.ceil(self.capacity_factor * n_tokens * self.top_k / self.n_experts))

    def forward(self, x: Tensor) -> Tensor:
        shape = x.shape
        xt = x.reshape(-1, shape[-1])
        T, E, k = xt.size(0), self.n_experts, self.top_k
        with torch.autocast(xt.device.type, enabled=False):
            logits = F.linear(xt.float(), self.router.linear.weight.float())
            probs = logits.softmax(-1)
        cap = self.capacity(T)
        idx, w, pos, keep = route(probs, k, cap)
        frac = F.one_hot(idx.reshape(-1), E).float().mean(0)  # f_e, assignments before dropping
        self.last_aux_loss = self.aux_loss_weight * E * (frac * probs.mean(0)).sum()
        self.last_drop_fraction = 1.0 - keep.float().mean()
        # dispatch: buffer [E, cap, d]; slot (e, pos) <- token
        slot = (idx * cap + pos).reshape(-1)
        keep_f = keep.reshape(-1)
        tok = torch.arange(T, device=xt.device).repeat_interleave(k)
        buf = xt.new_zeros(E * cap, shape[-1])
        buf = buf.index_copy(0, slot[keep_f], xt[tok[keep_f]])
        buf = buf.view(E, cap, shape[-1])
        if self.ep_world > 1:
            from sample_efficient_gpt_b200.parallel.expert_parallel import combine, dispatch

            local_in = dispatch(buf, self.ep_group)  # [E_local, ep_world * cap, d]
            out_buf = combine(self.experts(local_in), self.ep_group)  # [E, cap, d]
        else:
            out_buf = self.experts(buf)
        # combine: token <- sum_k weight * expert output
        gathered = out_buf.reshape(E * cap, shape[-1])[slot.clamp(max=E * cap - 1)]
        gathered = gathered * (w.reshape(-1) * keep_f.float()).to(gathered.dtype)[:, None]
        out = gathered.view(T, k, shape[-1]).sum(1)
        return out.view(shape)
