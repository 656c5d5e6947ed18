"""Expert-parallel token exchange: differentiable all-to-all dispatch and combine.

``dispatch(buf [E, cap, d])``: every rank sends the slices of ``buf`` that belong to another rank's experts and receives
its own experts' slices from everybody -> ``[E_local, world * cap, d]`` (source-rank major inside an expert).
``combine`` is the inverse exchange.  Each is the other's gradient, so the pair needs no saved tensors.
Baseline implementation on ``torch.distributed.all_to_all_single`` (NCCL on GPUs, gloo on CPU).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor


def _exchange(x: Tensor, group) -> Tensor:
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x.contiguous(), group=group)
    return out


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buf: Tensor, group):
        ctx.group = group
        world = dist.get_world_size(group)
        E, cap, d = buf.shape
        el = E // world
        # rows grouped by destination rank: [world, el, cap, d] is already buf's layout
        recv = _exchange(buf.view(world, el, cap, d), group)  # [src, el, cap, d]
        return recv.permute(1, 0, 2, 3).reshape(el, world * cap, d)

    @staticmethod
    def backward(ctx, g: Tensor):
        return _Combine.apply(g, ctx.group), None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y: Tensor, group):
        ctx.group = group
        world = dist.get_world_size(group)
        el, wc, d = y.shape
        cap = wc // world
        send = y.view(el, world, cap, d).permute(1, 0, 2, 3).contiguous()  # [dst(src of the tokens), el, cap, d]
        recv = _exchange(send, group)  # [owner rank, el, cap, d]
        return recv.reshape(world * el, cap, d)

    @staticmethod
    def backward(ctx, g: Tensor):
        return _Dispatch.apply(g, ctx.group), None


def dispatch(buf: Tensor, group) -> Tensor:
    return _Dispatch.apply(buf, group)


def combine(y: Tensor, group) -> Tensor:
    return _Combine.apply(y, group)
