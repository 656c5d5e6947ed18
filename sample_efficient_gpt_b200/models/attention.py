"""Multi-head self-attention with GQA, RoPE, QK RMS-norm, value residual and output gating.

Semantics follow transformer/attention.py:111-267 of the reference:
  * one packed projection ``qkv`` with rows ordered Q | K | V,
  * RoPE (fp32) on Q and K,
  * value residual ``V' = scale * (a1*V + a2*V1) * rsqrt(a1^2 + a2^2 + 1e-8)`` where V1 is the mixed
    value of the first block (its own V for the first block),
  * QK-norm: per token and head RMS normalisation (eps 1e-6) of q and k, q times a learnable scalar,
    then causal softmax attention with scale 1/sqrt(hd),
  * gate ``2*sigmoid(attn_gate(x))`` on the attention output, before the output projection; the gate
    input is the (normed) block input; variants: elementwise, per-head, per-head-hd.
Unlike the reference, K and V stay at KV-head granularity (no repeat to the query heads): the value
mix commutes with the repeat and attention is evaluated per query-head group.

This module is the autograd-capable path (CPU training, evaluation, generation with a KV cache, and
the oracle for the fused CUDA engine, which reads the same parameters).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from sample_efficient_gpt_b200.models.core import Linear
from sample_efficient_gpt_b200.models.rope import RotaryPositionalEmbedding
from sample_efficient_gpt_b200.utils.profiling import nvtx_range

QK_NORM_EPS = 1e-6
VALUE_MIX_EPS = 1e-8


class KVCache:
    """Per-layer cache of rotated keys and un-mixed values, ``[B, Hkv, S, hd]``."""

    def __init__(self):
        self.keys: Tensor | None = None
        self.values: Tensor | None = None

    @property
    def length(self) -> int:
        return 0 if self.keys is None else self.keys.size(2)

    def append(self, k: Tensor, v: Tensor) -> tuple[Tensor, Tensor]:
        if self.keys is None:
            self.keys, self.values = k, v
        else:
            self.keys = torch.cat((self.keys, k), dim=2)
            self.values = torch.cat((self.values, v), dim=2)
        return self.keys, self.values


class SelfDotProductAttnQKNorm(nn.Module):
    """Holds the scalar q gain of the QK-norm (state-dict key ``sdpa_qknorm.gain``)."""

    def __init__(self, head_dim: int):
        super().__init__()
        self.gain = nn.Parameter(torch.tensor([1.0], dtype=torch.float32))

    def normalize(self, q: Tensor, k: Tensor) -> tuple[Tensor, Tensor]:
        with torch.autocast(q.device.type, enabled=False):
            qf, kf = q.float(), k.float()
            qn = (qf * torch.rsqrt(qf.square().mean(-1, keepdim=True) + QK_NORM_EPS)).to(q.dtype)
            kn = (kf * torch.rsqrt(kf.square().mean(-1, keepdim=True) + QK_NORM_EPS)).to(k.dtype)
        return qn * self.gain.to(qn.dtype), kn


def causal_attention(q: Tensor, k: Tensor, v: Tensor, q_start: int = 0) -> Tensor:
    """q ``[B,H,Sq,hd]``, k/v ``[B,Hkv,Sk,hd]``; key j visible to query i iff j <= i + q_start."""
    h, hkv = q.size(1), k.size(1)
    if h != hkv:
        rep = h // hkv
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    v = v.to(q.dtype)
    if q_start == 0 and q.size(2) == k.size(2):
        return F.scaled_dot_product_attention(q, k, v, is_causal=True)
    qi = q_start + torch.arange(q.size(2), device=q.device)
    kj = torch.arange(k.size(2), device=q.device)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=kj[None, :] <= qi[:, None])


class MultiHeadSelfAttention(nn.Module):
    def __init__(
        self,
        d_model: int,
        n_heads: int,
        n_kv_heads: int | None = None,
        theta: float = 10_000,
        max_seq_len: int = 4096,
        qknorm: bool = False,
        value_residual: bool = False,
        gating: bool | str = False,
        head_dim: int | None = None,
        device=None,
        dtype=None,
    ):
        super().__init__()
        self.n_heads = n_heads
        self.n_kv_heads = int(n_kv_heads) if n_kv_heads is not None else n_heads
        if self.n_heads % self.n_kv_heads != 0:
            raise ValueError(f"Invalid GQA: n_heads={n_heads} not divisible by n_kv_heads={self.n_kv_heads}")
        if head_dim is None:
            if d_model % n_heads != 0:
                raise ValueError("d_model must be divisible by n_heads")
            head_dim = d_model // n_heads
        self.head_dim = head_dim
        self.d_model = d_model
        self.rope = RotaryPositionalEmbedding(theta, d_k=head_dim, max_seq_len=max_seq_len, device=device)
        q_out, kv_out = n_heads * head_dim, self.n_kv_heads * head_dim
        self.qkv = Linear(d_model, q_out + 2 * kv_out, device=device, dtype=dtype)
        self.out = Linear(q_out, d_model, device=device, dtype=dtype)
        self.qknorm = qknorm
        if qknorm:
            self.sdpa_qknorm = SelfDotProductAttnQKNorm(head_dim)
        self.value_residual = value_residual
        if value_residual:
            self.alpha1 = nn.Parameter(torch.tensor([1.0], device=device))
            self.alpha2 = nn.Parameter(torch.tensor([0.0], device=device))
            self.scale = nn.Parameter(torch.tensor([1.0], device=device))
        else:
            self.register_buffer("alpha1", torch.tensor([1.0], device=device), persistent=False)
            self.register_buffer("alpha2", torch.tensor([0.0], device=device), persistent=False)
            self.register_buffer("scale", torch.tensor([1.0], device=device), persistent=False)
        self.gating = gating
        if gating:
            if gating == "elementwise":
                self.attn_gate = Linear(d_model, q_out, device=device, dtype=dtype)
            elif gating == "per-head":
                self.attn_gate = Linear(d_model, n_heads, device=device, dtype=dtype)
            elif gating == "per-head-hd":
                self.attn_gate = Linear(head_dim, n_heads, device=device, dtype=dtype)
            else:
                raise ValueError(f"gating={gating!r} is undefined")

    def mix_values(self, v: Tensor, v1: Tensor) -> Tensor:
        c = torch.rsqrt(self.alpha1**2 + self.alpha2**2 + VALUE_MIX_EPS)
        return self.scale * (self.alpha1 * v + self.alpha2 * v1) * c

    @nvtx_range("attention")
    def forward(
        self,
        x: Tensor,
        token_positions: Tensor | None = None,
        v1: Tensor | None = None,
        kv_cache: KVCache | None = None,
    ) -> tuple[Tensor, Tensor]:
        b, s, _ = x.shape
        h, hkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        proj = self.qkv(x)
        q, k, v = proj.split((h * hd, hkv * hd, hkv * hd), dim=-1)
        q = q.view(b, s, h, hd).transpose(1, 2)
        k = k.view(b, s, hkv, hd).transpose(1, 2)
        v = v.view(b, s, hkv, hd).transpose(1, 2)
        if kv_cache is not None:
            q_start = kv_cache.length
            pos = torch.arange(q_start, q_start + s, device=x.device)
        else:
            q_start, pos = 0, token_positions
        with torch.autocast(x.device.type, enabled=False), nvtx_range("RoPE"):
            q = self.rope(q, pos)
            k = self.rope(k, pos)
        if kv_cache is not None:
            k, v = kv_cache.append(k, v)
        v_mixed = self.mix_values(v, v if v1 is None else v1.view_as(v))
        if self.qknorm:
            q, k = self.sdpa_qknorm.normalize(q, k)
        attn = causal_attention(q, k, v_mixed.to(q.dtype) if q.dtype != torch.float32 else v_mixed, q_start)
        attn = attn.transpose(1, 2)  # [b, s, h, hd]
        if not self.gating:
            cat = attn.reshape(b, s, h * hd)
        elif self.gating == "elementwise":
            cat = (2.0 * self.attn_gate(x).sigmoid()) * attn.reshape(b, s, h * hd)
        else:
            gate_in = x if self.gating == "per-head" else x[..., :hd]
            gate = (2.0 * self.attn_gate(gate_in).sigmoid()).unsqueeze(-1)
            cat = (gate * attn).reshape(b, s, h * hd)
        return self.out(cat), v_mixed
