"""Plain PyTorch statements of every fused op (forward and hand-derived backward).

These functions are (a) the CPU implementation of the ops layer, (b) the oracle that the CUDA
kernels are tested against (run them in fp32), and (c) the specification of what each kernel
computes.  Shapes: T = B*S tokens, d model width, H query heads, Hkv KV heads, hd head dim, F ffn
width, V vocabulary.  "lp" is the activation dtype (bf16 on a GPU, fp32 on CPU).

Math sources in the reference: RMSNorm core.py:61-72, RoPE rope.py:36-56, value residual
attention.py:222-228, QK-norm attention.py:51-63, gate attention.py:249-255, SwiGLU core.py:86-89,
cross entropy ops/cross_entropy.py:96-247, block kurtosis transformer.py:58-61.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor

QK_NORM_EPS = 1e-6
VALUE_MIX_EPS = 1e-8


# ----------------------------------------------------------------------------- RMSNorm (+ residual add)
def add_rmsnorm_fwd(res: Tensor, delta: Tensor | None, gain: Tensor, scale: float, eps: float, out_dtype, want_kurt: bool):
    """x = res + delta; y = x * rsqrt(mean(x^2)+eps) * gain * scale.

    Returns (x fp32 [T,d], y out_dtype [T,d], rstd fp32 [T], kurt_sum fp32 scalar | None) where
    kurt_sum = sum_t mean_d(x^4) / max(mean_d(x^2), 1e-8)^2.
    """
    x = res.float() if delta is None else res.float() + delta.float()
    ms = x.square().mean(-1)
    rstd = torch.rsqrt(ms + eps)
    y = (x * rstd[:, None] * (gain.float() * scale)).to(out_dtype)
    kurt = None
    if want_kurt:
        m2 = ms.clamp_min(1e-8)
        kurt = (x.pow(4).mean(-1) / (m2 * m2)).sum()
    return x, y, rstd, kurt


def add_rmsnorm_bwd(dy: Tensor, dres_in: Tensor | None, x: Tensor, gain: Tensor, rstd: Tensor, scale: float, lp_dtype):
    """Returns (dres fp32 [T,d] = dres_in + d(norm)/dx, dres in lp_dtype, dgain fp32 [d])."""
    dyf = dy.float()
    m = dyf * (gain.float() * scale)
    r = rstd[:, None]
    dx = r * m - (r**3) * x * (m * x).mean(-1, keepdim=True)
    dgain = (dyf * x * r).sum(0) * scale
    dres = dx if dres_in is None else dx + dres_in
    return dres, dres.to(lp_dtype), dgain


# ----------------------------------------------------------------------------- qkv post-processing
def _rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """x [B,S,h,hd] fp32, cos/sin [S,hd/2]."""
    half = x.size(-1) // 2
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)


def _rope_t(d: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Transpose (= inverse) rotation applied to a gradient."""
    half = d.size(-1) // 2
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    d1, d2 = d[..., :half], d[..., half:]
    return torch.cat([d1 * c + d2 * s, -d1 * s + d2 * c], dim=-1)


def qkv_post_fwd(qkv, v1, cos, sin, qgain, a1, a2, vscale, B, S, H, Hkv, hd, qknorm: bool):
    """Split packed qkv [T,(H+2Hkv)hd], rotate q/k, RMS-normalise q/k (q times gain), mix v with v1.

    v1 None means "this is the first block": V1 = V.  Returns q^ [B,S,H,hd], k^ [B,S,Hkv,hd],
    v' [B,S,Hkv,hd], all in qkv's dtype.
    """
    lp = qkv.dtype
    q, k, v = qkv.float().split((H * hd, Hkv * hd, Hkv * hd), dim=-1)
    q = _rope(q.reshape(B, S, H, hd), cos[:S], sin[:S])
    k = _rope(k.reshape(B, S, Hkv, hd), cos[:S], sin[:S])
    v = v.reshape(B, S, Hkv, hd)
    if qknorm:
        q = q * torch.rsqrt(q.square().mean(-1, keepdim=True) + QK_NORM_EPS) * qgain.float()
        k = k * torch.rsqrt(k.square().mean(-1, keepdim=True) + QK_NORM_EPS)
    a1f, a2f, sf = a1.float(), a2.float(), vscale.float()
    c = torch.rsqrt(a1f * a1f + a2f * a2f + VALUE_MIX_EPS)
    v1f = v if v1 is None else v1.float().reshape(B, S, Hkv, hd)
    vm = sf * c * (a1f * v + a2f * v1f)
    return q.to(lp), k.to(lp), vm.to(lp)


def qkv_post_bwd(dq, dk, dv, qkv, v1, cos, sin, qgain, a1, a2, vscale, B, S, H, Hkv, hd, qknorm: bool):
    """Gradients of qkv_post_fwd.

    dq/dk/dv: gradients w.r.t. q^, k^, v' (any float dtype; dv may be fp32 because the first block
    adds the accumulated v1 gradients).  Returns (dqkv lp [T,(H+2Hkv)hd], dv1 fp32 [B,S,Hkv,hd] | None,
    dqgain, da1, da2, dvscale as fp32 1-element tensors).
    """
    lp = qkv.dtype
    q, k, v = qkv.float().split((H * hd, Hkv * hd, Hkv * hd), dim=-1)
    q = _rope(q.reshape(B, S, H, hd), cos[:S], sin[:S])
    k = _rope(k.reshape(B, S, Hkv, hd), cos[:S], sin[:S])
    v = v.reshape(B, S, Hkv, hd)
    dq, dk, dv = dq.float(), dk.float(), dv.float()
    dqgain = torch.zeros(1, dtype=torch.float32, device=qkv.device)
    if qknorm:
        g = qgain.float()
        rq = torch.rsqrt(q.square().mean(-1, keepdim=True) + QK_NORM_EPS)
        rk = torch.rsqrt(k.square().mean(-1, keepdim=True) + QK_NORM_EPS)
        dqgain = (dq * q * rq).sum().reshape(1)
        dq = g * rq * dq - g * rq**3 * q * (q * dq).mean(-1, keepdim=True)
        dk = rk * dk - rk**3 * k * (k * dk).mean(-1, keepdim=True)
    dq = _rope_t(dq, cos[:S], sin[:S])
    dk = _rope_t(dk, cos[:S], sin[:S])
    a1f, a2f, sf = a1.float(), a2.float(), vscale.float()
    c = torch.rsqrt(a1f * a1f + a2f * a2f + VALUE_MIX_EPS)
    v1f = v if v1 is None else v1.float().reshape(B, S, Hkv, hd)
    U = a1f * v + a2f * v1f
    s_dvU = (dv * U).sum()
    dvscale = (c * s_dvU).reshape(1)
    da1 = (sf * c * (dv * v).sum() - a1f * c**3 * sf * s_dvU).reshape(1)
    da2 = (sf * c * (dv * v1f).sum() - a2f * c**3 * sf * s_dvU).reshape(1)
    if v1 is None:
        dvv = sf * c * (a1f + a2f) * dv
        dv1 = None
    else:
        dvv = sf * c * a1f * dv
        dv1 = sf * c * a2f * dv
    dqkv = torch.cat([dq.reshape(B * S, H * hd), dk.reshape(B * S, Hkv * hd), dvv.reshape(B * S, Hkv * hd)], dim=-1)
    return dqkv.to(lp), dv1, dqgain, da1, da2, dvscale


# ----------------------------------------------------------------------------- attention
def attention_fwd(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, q_start: int = 0):
    """q [B,Sq,H,hd], k/v [B,Sk,Hkv,hd] -> (O [B,Sq,H,hd] in q.dtype, LSE fp32 [B,H,Sq]).

    Scores scaled by 1/sqrt(hd); query head h reads KV head h // (H/Hkv); key j visible iff j <= i + q_start.
    """
    B, Sq, H, hd = q.shape
    Sk, Hkv = k.size(1), k.size(2)
    rep = H // Hkv
    qf = q.float().permute(0, 2, 1, 3)  # B,H,Sq,hd
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = (qf @ kf.transpose(-1, -2)) / math.sqrt(hd)
    if causal:
        i = torch.arange(Sq, device=q.device)[:, None] + q_start
        j = torch.arange(Sk, device=q.device)[None, :]
        s = s.masked_fill(j > i, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    o = (p @ vf).permute(0, 2, 1, 3)
    return o.to(q.dtype).contiguous(), lse


def attention_bwd(do: Tensor, q: Tensor, k: Tensor, v: Tensor, o: Tensor, lse: Tensor, causal: bool = True, q_start: int = 0):
    """Returns (dq, dk, dv) in the input dtypes; dk/dv are summed over the query heads of each group."""
    B, Sq, H, hd = q.shape
    Sk, Hkv = k.size(1), k.size(2)
    rep = H // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    dof = do.float().permute(0, 2, 1, 3)
    of = o.float().permute(0, 2, 1, 3)
    scale = 1.0 / math.sqrt(hd)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        i = torch.arange(Sq, device=q.device)[:, None] + q_start
        j = torch.arange(Sk, device=q.device)[None, :]
        s = s.masked_fill(j > i, float("-inf"))
    p = torch.exp(s - lse[..., None])
    dvf = p.transpose(-1, -2) @ dof
    dp = dof @ vf.transpose(-1, -2)
    D = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - D)
    dqf = (ds @ kf) * scale
    dkf = (ds.transpose(-1, -2) @ qf) * scale
    dkf = dkf.reshape(B, Hkv, rep, Sk, hd).sum(2)
    dvf = dvf.reshape(B, Hkv, rep, Sk, hd).sum(2)
    return (
        dqf.permute(0, 2, 1, 3).to(q.dtype).contiguous(),
        dkf.permute(0, 2, 1, 3).to(k.dtype).contiguous(),
        dvf.permute(0, 2, 1, 3).to(v.dtype).contiguous(),
    )


# ----------------------------------------------------------------------------- per-head output gate
def gate_fwd(o: Tensor, z: Tensor) -> Tensor:
    """o [T,H,hd], z [T,H] gate logits -> [T,H*hd] = 2*sigmoid(z) * o."""
    g = 2.0 * torch.sigmoid(z.float())
    return (g[..., None] * o.float()).to(o.dtype).reshape(o.size(0), -1)


def gate_bwd(dg: Tensor, o: Tensor, z: Tensor):
    """dg [T,H*hd] -> (do [T,H,hd], dz [T,H])."""
    T, H, hd = o.shape
    sg = torch.sigmoid(z.float())
    dgf = dg.float().reshape(T, H, hd)
    do = (2.0 * sg[..., None] * dgf).to(o.dtype)
    dz = (2.0 * sg * (1.0 - sg) * (dgf * o.float()).sum(-1)).to(z.dtype)
    return do, dz


# ----------------------------------------------------------------------------- SwiGLU
def swiglu_fwd(u: Tensor) -> Tensor:
    """u [T,2F] = [gate | up] -> silu(gate) * up, [T,F]."""
    a, b = u.float().chunk(2, dim=-1)
    return (a * torch.sigmoid(a) * b).to(u.dtype)


def swiglu_bwd(df: Tensor, u: Tensor) -> Tensor:
    a, b = u.float().chunk(2, dim=-1)
    dff = df.float()
    sg = torch.sigmoid(a)
    da = dff * b * (sg + a * sg * (1.0 - sg))
    db = dff * a * sg
    return torch.cat([da, db], dim=-1).to(u.dtype)


# ----------------------------------------------------------------------------- cross entropy
def softmax_ce_fwd(logits: Tensor, targets: Tensor, lse_square_scale: float, ignore_index: int):
    """Per-token (loss, z, lse): loss = lse - x_y + s*lse^2, z = s*lse^2; ignored tokens give 0."""
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    valid = targets != ignore_index
    tgt = lf.gather(-1, targets.clamp_min(0).long()[:, None]).squeeze(-1)
    z = lse_square_scale * lse * lse
    loss = torch.where(valid, lse - tgt + z, torch.zeros_like(lse))
    z = torch.where(valid, z, torch.zeros_like(z))
    return loss, z, lse


def softmax_ce_bwd(logits: Tensor, targets: Tensor, lse: Tensor, grad_tok: Tensor, lse_square_scale: float, ignore_index: int):
    """dlogits = g_i * (softmax * (1 + 2 s lse) - onehot(y)); zero rows for ignored tokens."""
    lf = logits.float()
    p = torch.exp(lf - lse[:, None]) * (1.0 + 2.0 * lse_square_scale * lse)[:, None]
    valid = targets != ignore_index
    p.scatter_add_(1, targets.clamp_min(0).long()[:, None], -torch.ones_like(lse)[:, None])
    p = p * (grad_tok.float() * valid.float())[:, None]
    return p.to(logits.dtype)


def linear_ce_fwd_bwd(
    h: Tensor,
    w: Tensor,
    targets: Tensor,
    lse_square_scale: float,
    ignore_index: int,
    grad_scale: float,
    logit_scale: float = 1.0,
    chunk: int = 4096,
    dw_out: Tensor | None = None,
    need_grad: bool = True,
):
    """Fused head projection + loss, chunked over tokens so the full logits never exist.

    h [T,d] lp, w [V,d] lp.  Returns (loss_tok fp32 [T], z_tok fp32 [T], dh lp [T,d] | None, dW fp32 [V,d] | None)
    with the gradients of ``grad_scale * sum_t loss_t`` (dW is accumulated into ``dw_out`` when given).
    """
    T, d = h.shape
    loss = torch.empty(T, dtype=torch.float32, device=h.device)
    z = torch.empty(T, dtype=torch.float32, device=h.device)
    dh = torch.empty_like(h) if need_grad else None
    dw = None
    if need_grad:
        dw = dw_out if dw_out is not None else torch.zeros(w.shape, dtype=torch.float32, device=h.device)
    for s in range(0, T, chunk):
        e = min(T, s + chunk)
        hc = h[s:e]
        logits = (hc @ w.t()).float() * logit_scale
        l, zz, lse = softmax_ce_fwd(logits, targets[s:e], lse_square_scale, ignore_index)
        loss[s:e], z[s:e] = l, zz
        if need_grad:
            g = torch.full((e - s,), grad_scale * logit_scale, dtype=torch.float32, device=h.device)
            dl = softmax_ce_bwd(logits, targets[s:e], lse, g, lse_square_scale, ignore_index).to(h.dtype)
            dh[s:e] = dl @ w
            dw += (dl.t() @ hc).float()
    return loss, z, dh, dw


# ----------------------------------------------------------------------------- optimizer tails
def normuon_tail(v: Tensor, second: Tensor, beta2: float):
    """Batched neuron-wise normalisation of v [n,r,c] that keeps each matrix' Frobenius norm.

    Updates ``second`` in place; returns (v_normalised fp32, ||v||_F^2 summed over the batch)."""
    v = v.float()
    v_norm = v.norm(dim=(-2, -1), keepdim=True)
    dim = -1 if second.size(-1) == 1 else -2
    second.lerp_(v.square().mean(dim=dim, keepdim=True), 1 - beta2)
    v = v * torch.rsqrt(second.clamp_min(1e-10))
    v = v * (v_norm / v.norm(dim=(-2, -1), keepdim=True).clamp_min(1e-10))
    return v, v_norm.square().sum()
