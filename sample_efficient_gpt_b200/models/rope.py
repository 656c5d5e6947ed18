"""Rotary position embedding, split-half convention, fp32 math (transformer/rope.py:13-56)."""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor


def rope_tables(max_seq_len: int, theta: float, head_dim: int, device=None) -> tuple[Tensor, Tensor]:
    """cos / sin of ``p * theta^(-2i/hd)`` for p < max_seq_len, i < hd/2; both ``[max_seq_len, hd/2]`` fp32."""
    i = torch.arange(0, head_dim // 2, device=device)
    inv_freq = theta ** (-2 * i / head_dim)
    ang = torch.outer(torch.arange(max_seq_len, device=device), inv_freq)
    return ang.cos().float(), ang.sin().float()


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """x ``[..., seq, hd]``; cos/sin ``[seq, hd/2]`` (already gathered for the token positions)."""
    xf = x.float()
    half = xf.size(-1) // 2
    x1, x2 = xf[..., :half], xf[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).to(x.dtype)


class RotaryPositionalEmbedding(nn.Module):
    def __init__(self, theta: float, d_k: int, max_seq_len: int, device=None):
        super().__init__()
        cos, sin = rope_tables(max_seq_len, theta, d_k, device)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def forward(self, x: Tensor, token_positions: Tensor | None = None) -> Tensor:
        if token_positions is None:
            cos, sin = self.cos[: x.size(-2)], self.sin[: x.size(-2)]
        else:
            cos, sin = self.cos[token_positions], self.sin[token_positions]
        return apply_rope(x, cos, sin)
