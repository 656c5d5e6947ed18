"""Causal GQA attention on CUDA tensors: forward returning (O, ctx) and backward from ctx.

Two implementations: this package's tcgen05 flash-attention kernels (``fa_fwd`` / ``fa_bwd`` in the extension; causal,
head_dim 64, any sequence length: the backward extends a ragged sequence with zero rows up to its 128-row tiles) and the library path: PyTorch's fused SDPA (flash / cuDNN backend, native GQA),
differentiated through a private autograd tape so that the caller needs no autograd graph of its own.
``SEGPT_ATTN_IMPL=native|library|auto``: ``auto`` (default) runs the native kernels wherever they apply - in training the
tcgen05 forward + backward pair (inside the training step it is within a few percent of the library pair, which needs
transposed copies of its operands and result), in evaluation and generation the forward - and the library elsewhere
(head_dim other than 64, decoding against a cache);
``native`` raises where ``auto`` would fall back because the kernels are missing; ``library`` forces the library pair.
"""

from __future__ import annotations

import os

import torch
import torch.nn.functional as F
from torch import Tensor

from sample_efficient_gpt_b200 import ops


class _Tape:
    """What the library path keeps for its backward: detached leaves and the taped output."""

    __slots__ = ("q", "k", "v", "out")

    def __init__(self, q, k, v, out):
        self.q, self.k, self.v, self.out = q, k, v, out


def _native_ok(q: Tensor, k: Tensor, v: Tensor, q_start: int, for_backward: bool) -> bool:
    impl = os.environ.get("SEGPT_ATTN_IMPL", "auto")
    if impl == "library" or not ops.has_kernel("fa_fwd"):
        if impl == "native":
            raise RuntimeError("SEGPT_ATTN_IMPL=native but the flash-attention kernels are not built")
        return False
    if for_backward and not ops.has_kernel("fa_bwd"):
        return False  # the library backward needs the library forward's tape
    hd = q.size(-1)
    return (q.dtype == torch.bfloat16 and hd == 64 and q_start == 0 and q.size(1) == k.size(1)
            and q.is_contiguous() and k.is_contiguous() and v.is_contiguous())


def forward(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, q_start: int = 0, for_backward: bool = True):
    """q [B,S,H,hd], k/v [B,S,Hkv,hd] -> (O [B,S,H,hd], ctx).  ``for_backward=False`` (evaluation) lets the native
    forward kernel run even when no native backward is built."""
    if causal and _native_ok(q, k, v, q_start, for_backward):
        ops._count()
        o, lse = ops.ext().fa_fwd(q, k, v, causal)
        return o, lse
    with torch.enable_grad():
        ql, kl, vl = (t.detach().requires_grad_(True) for t in (q, k, v))
        qt, kt, vt = ql.transpose(1, 2), kl.transpose(1, 2), vl.transpose(1, 2)
        if q_start == 0 and q.size(1) == k.size(1):
            o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=causal, enable_gqa=True)
        else:
            qi = q_start + torch.arange(q.size(1), device=q.device)
            kj = torch.arange(k.size(1), device=q.device)
            o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=kj[None, :] <= qi[:, None], enable_gqa=True)
        o = o.transpose(1, 2).contiguous()
    return o.detach(), _Tape(ql, kl, vl, o)


def backward(do: Tensor, q: Tensor, k: Tensor, v: Tensor, o: Tensor, ctx, causal: bool = True, q_start: int = 0):
    if isinstance(ctx, _Tape):
        dq, dk, dv = torch.autograd.grad(ctx.out, (ctx.q, ctx.k, ctx.v), do.reshape(ctx.out.shape))
        return dq, dk, dv
    ops._count(2)
    return ops.ext().fa_bwd(do.contiguous(), q, k, v, o, ctx, causal)
