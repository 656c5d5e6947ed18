"""Model primitives: Linear, Embedding, RMSNorm (with LayerNorm-scaling), SwiGLU, softmax.

State-dict names match the reference (transformer/core.py:11-97): ``Linear`` wraps a bias-free
``nn.Linear`` so its weight is ``<name>.linear.weight``; ``RMSNorm`` has a learnable ``gain`` and a
non-persistent ``position_scale`` buffer holding ``1/sqrt(layer_index)``.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from sample_efficient_gpt_b200.utils.profiling import nvtx_range


def mup_trunc_normal_(w: Tensor, fan_in: int) -> Tensor:
    """Width-aware init: N(0, 1/fan_in) truncated at three standard deviations."""
    sigma = 1.0 / math.sqrt(fan_in)
    return nn.init.trunc_normal_(w, std=sigma, a=-3 * sigma, b=3 * sigma)


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, device=None, dtype=None):
        super().__init__()
        # nn.Linear draws its default init first and is then overwritten: the reference does the same
        # (core.py:18-23), and keeping the RNG draws identical keeps seeds interchangeable.
        self.linear = nn.Linear(in_features, out_features, bias=False, device=device, dtype=dtype)
        mup_trunc_normal_(self.linear.weight, in_features)

    @nvtx_range("linear forward")
    def forward(self, x: Tensor) -> Tensor:
        return self.linear(x)


class Embedding(nn.Module):
    def __init__(self, vocab_size: int, d_model: int, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab_size, d_model, device=device, dtype=dtype))
        mup_trunc_normal_(self.weight, d_model)

    def forward(self, ids: Tensor) -> Tensor:
        return F.embedding(ids, self.weight)


class RMSNorm(nn.Module):
    """y = x * rsqrt(mean(x^2) + eps) * gain * position_scale, computed in fp32."""

    def __init__(self, d_model: int, eps: float = 1e-5, position: int | None = None, device=None, dtype=None):
        super().__init__()
        self.gain = nn.Parameter(torch.ones(d_model, device=device, dtype=dtype))
        self.eps = eps
        scale = 1.0 if position is None else 1.0 / math.sqrt(float(position))
        self.register_buffer("position_scale", torch.tensor(scale, device=device, dtype=torch.float32), persistent=False)

    @nvtx_range("rmsnorm forward")
    def forward(self, x: Tensor) -> Tensor:
        in_dtype = x.dtype
        xf = x.float()
        with torch.autocast(xf.device.type, enabled=False):
            rstd = torch.rsqrt(xf.square().mean(-1, keepdim=True) + self.eps)
            y = xf * rstd * self.gain.float() * self.position_scale
        return y.to(in_dtype)


class SwiGLU(nn.Module):
    """down(silu(gate) * up) with gate and up packed in one projection (gate = first half)."""

    def __init__(self, d_model: int, d_ff: int, device=None, dtype=None):
        super().__init__()
        d_ff = int(d_ff // 64 * 64)
        self.d_ff = d_ff
        self.up = Linear(d_model, 2 * d_ff, device, dtype)
        self.down = Linear(d_ff, d_model, device, dtype)

    @nvtx_range("swiglu forward")
    def forward(self, x: Tensor) -> Tensor:
        gate, up = self.up(x).chunk(2, dim=-1)
        return self.down(F.silu(gate) * up)


def softmax(x: Tensor, dim: int = 0, temperature: float = 1.0) -> Tensor:
    """Max-shifted softmax; a temperature of exactly 0 leaves the logits unscaled (callers then argmax)."""
    o = x - x.max(dim=dim, keepdim=True)[0]
    if temperature != 0.0:
        o = o / temperature
    e = o.exp()
    return e / e.sum(dim=dim, keepdim=True)
