"""Ops layer: every hot op of the model as an explicit forward / backward pair.

On CUDA tensors an op runs the hand-written sm_100a kernel from the in-tree extension
(``sample_efficient_gpt_b200/_C*.so``, built by ``python -m sample_efficient_gpt_b200.csrc.build``);
on CPU tensors it runs the PyTorch statement in ``ops.reference`` (also the test oracle).
On a machine with a GPU a missing extension is an error, not a silent fallback; set
``SEGPT_ALLOW_TORCH_FALLBACK=1`` to run the PyTorch statements on the GPU anyway (debugging).
Individual kernels can be switched off with ``SEGPT_DISABLE_KERNELS=name1,name2``.
"""

from __future__ import annotations

import importlib
import os

import torch
from torch import Tensor

from sample_efficient_gpt_b200.ops import reference as ref

_EXT = None
_EXT_ERR: Exception | None = None
_DISABLED = {s for s in os.environ.get("SEGPT_DISABLE_KERNELS", "").split(",") if s}
launch_count = 0  # number of kernels of this package launched (bench.py reports it)


def ext():
    """The compiled extension module, or None when it is not built."""
    global _EXT, _EXT_ERR
    if _EXT is None and _EXT_ERR is None:
        try:
            # SEGPT_DEBUG_BOUNDS=1: the build whose kernels check every computed store index (csrc/bounds.cuh)
            name = "_C_dbg" if os.environ.get("SEGPT_DEBUG_BOUNDS", "0") == "1" else "_C"
            _EXT = importlib.import_module(f"sample_efficient_gpt_b200.{name}")
        except Exception as e:  # not built, or built for another torch
            _EXT_ERR = e
    return _EXT


def ext_error() -> Exception | None:
    ext()
    return _EXT_ERR


def has_kernel(name: str) -> bool:
    e = ext()
    return e is not None and name not in _DISABLED and hasattr(e, name)


def kernel_enabled(feature: str) -> bool:
    """Features that choose between this package's kernel and a library call (``SEGPT_DISABLE_KERNELS=ns_gemm``)."""
    return feature not in _DISABLED


def _use_cuda(t: Tensor, name: str) -> bool:
    if not t.is_cuda:
        return False
    if has_kernel(name):
        return True
    if name in _DISABLED or os.environ.get("SEGPT_ALLOW_TORCH_FALLBACK", "0") == "1":
        return False
    raise RuntimeError(
        f"CUDA kernel '{name}' is unavailable ({ext_error()!r}); build the extension with "
        "`python -m sample_efficient_gpt_b200.csrc.build` or set SEGPT_ALLOW_TORCH_FALLBACK=1"
    )


def _count(n: int = 1):
    global launch_count
    launch_count += n


# ----------------------------------------------------------------------------- norm
def add_rmsnorm_fwd(res, delta, gain, scale: float, eps: float, out_dtype, want_kurt: bool = False):
    if _use_cuda(res, "add_rmsnorm_fwd"):
        _count()
        return ext().add_rmsnorm_fwd(res, delta, gain, float(scale), float(eps), out_dtype == torch.bfloat16, want_kurt)
    return ref.add_rmsnorm_fwd(res, delta, gain, scale, eps, out_dtype, want_kurt)


def add_rmsnorm_bwd(dy, dres_in, x, gain, rstd, scale: float, lp_dtype):
    if _use_cuda(x, "add_rmsnorm_bwd"):
        _count(2)
        return ext().add_rmsnorm_bwd(dy, dres_in, x, gain, rstd, float(scale), lp_dtype == torch.bfloat16)
    return ref.add_rmsnorm_bwd(dy, dres_in, x, gain, rstd, scale, lp_dtype)


# ----------------------------------------------------------------------------- qkv post-processing
def qkv_post_fwd(qkv, v1, cos, sin, qgain, a1, a2, vscale, B, S, H, Hkv, hd, qknorm, pos=None):
    """``pos`` (int32 scalar tensor): added to every token's position - decode steps (S == 1) at the cache length."""
    if _use_cuda(qkv, "qkv_post_fwd"):
        _count()
        return ext().qkv_post_fwd(qkv, v1, cos, sin, qgain, a1, a2, vscale, B, S, H, Hkv, hd, qknorm, pos)
    if pos is not None:
        p0 = int(pos)
        cos, sin = cos[p0:], sin[p0:]
    return ref.qkv_post_fwd(qkv, v1, cos, sin, qgain, a1, a2, vscale, B, S, H, Hkv, hd, qknorm)


def qkv_post_bwd(dq, dk, dv, qkv, v1, cos, sin, qgain, a1, a2, vscale, B, S, H, Hkv, hd, qknorm, dqkv_out=None, dv1_acc=None):
    """``qkv`` may be a column slice of a wider projection output; ``dqkv_out`` (same shape and row stride as ``qkv``)
    receives the gradient in place of a fresh buffer.  ``dv1_acc`` (fp32 [B,S,Hkv,hd]): the running sum of the
    value-residual gradients of the later blocks; this block's contribution is added in place and the sum is returned."""
    if _use_cuda(qkv, "qkv_post_bwd"):
        _count(2)
        return ext().qkv_post_bwd(dq, dk, dv, qkv, v1, cos, sin, qgain, a1, a2, vscale, B, S, H, Hkv, hd, qknorm, dqkv_out, dv1_acc)
    out = ref.qkv_post_bwd(dq, dk, dv, qkv, v1, cos, sin, qgain, a1, a2, vscale, B, S, H, Hkv, hd, qknorm)
    if dqkv_out is not None:
        dqkv_out.copy_(out[0])
        out = (dqkv_out, *out[1:])
    if dv1_acc is not None and out[1] is not None:
        out = (out[0], dv1_acc.add_(out[1]), *out[2:])
    return out


# ----------------------------------------------------------------------------- attention
def attention_fwd(q, k, v, causal: bool = True, q_start: int = 0, for_backward: bool = True):
    if q.is_cuda:
        from sample_efficient_gpt_b200.ops import attention as attn_impl

        return attn_impl.forward(q, k, v, causal, q_start, for_backward)
    return ref.attention_fwd(q, k, v, causal, q_start)


def attention_bwd(do, q, k, v, o, lse, causal: bool = True, q_start: int = 0):
    if q.is_cuda:
        from sample_efficient_gpt_b200.ops import attention as attn_impl

        return attn_impl.backward(do, q, k, v, o, lse, causal, q_start)
    return ref.attention_bwd(do, q, k, v, o, lse, causal, q_start)


# ----------------------------------------------------------------------------- gate / swiglu
def gate_fwd(o, z):
    if _use_cuda(o, "gate_fwd"):
        _count()
        return ext().gate_fwd(o, z)
    return ref.gate_fwd(o, z)


def gate_bwd(dg, o, z, dz_out=None):
    """``z`` may be a column slice of a wider tensor; ``dz_out`` ([T, H], likewise) receives the gate-logit gradient."""
    if _use_cuda(o, "gate_bwd"):
        _count()
        return ext().gate_bwd(dg, o, z, dz_out)
    do, dz = ref.gate_bwd(dg, o, z)
    if dz_out is not None:
        dz_out.copy_(dz)
        dz = dz_out
    return do, dz


def swiglu_fwd(u):
    if _use_cuda(u, "swiglu_fwd"):
        _count()
        return ext().swiglu_fwd(u)
    return ref.swiglu_fwd(u)


def swiglu_bwd(df, u):
    if _use_cuda(u, "swiglu_bwd"):
        _count()
        return ext().swiglu_bwd(df, u)
    return ref.swiglu_bwd(df, u)


def up_swiglu(x: Tensor, w: Tensor):
    """(u, f) of a SwiGLU feed-forward's first half: u = x w^T for w = [F gate rows | F up rows], f = silu(u[:, :F]) * u[:, F:]
    (transformer/core.py:86-89 of the reference).  On CUDA one launch of the tcgen05 GEMM whose epilogue stores u and forms
    f from the rounded tile while it is still on chip (``SEGPT_FUSE_SWIGLU=0``: GEMM, then the element-wise kernel;
    both give the same bits)."""
    if (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.size(0) % 256 == 0
            and os.environ.get("SEGPT_FUSE_SWIGLU", "1") != "0" and has_kernel("gemm_swiglu") and _native_gemm(x, w)):
        _count()
        return ext().gemm_swiglu(x, w)
    u = matmul_nt(x, w)
    return u, swiglu_fwd(u)


def down_dgrad_swiglu(dy: Tensor, w_down: Tensor, u: Tensor) -> Tensor:
    """Gradient of u = (gate | up) [M, 2F] of a SwiGLU feed-forward from the gradient dy [M, d] of its output and the down
    projection's weight w_down [d, F]: du = swiglu_bwd(dy @ w_down, u) (what autograd derives for transformer/core.py:86-89 of
    the reference).  On CUDA one launch: the GEMM's epilogue takes df
    (rounded to bf16, as a stored df would be) straight from the accumulator, so df never reaches memory
    (``SEGPT_FUSE_SWIGLU=0``: GEMM, then the element-wise kernel; both give the same bits)."""
    if (dy.is_cuda and dy.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16 and u.dtype == torch.bfloat16 and dy.dim() == 2
            and w_down.size(1) % 256 == 0 and os.environ.get("SEGPT_FUSE_SWIGLU", "1") != "0" and has_kernel("gemm_swiglu_bwd")
            and _native_gemm(dy, w_down) and u.is_contiguous()):
        _count()
        return ext().gemm_swiglu_bwd(dy, w_down, u)
    return swiglu_bwd(matmul_nn(dy, w_down), u)


# ----------------------------------------------------------------------------- GEMMs
_NATIVE_GEMM_MIN_ROWS = int(os.environ.get("SEGPT_NATIVE_GEMM_MIN_ROWS", "128"))


def _native_gemm(*tensors) -> bool:
    """The block projections (and their gradients) run on this package's tcgen05 GEMM (CTA pairs, csrc/gemm_pair.cu);
    ``SEGPT_BLOCK_GEMM=library`` sends them to the library GEMM instead (comparison runs)."""
    if os.environ.get("SEGPT_BLOCK_GEMM", "native") != "native":
        return False
    # Products with a handful of rows (the one-token decode step: rows = batch) are matrix-vector work: a 256 x 256 tile
    # kernel keeps a dozen CTA pairs busy on them, the library's small-row kernels run the decode step 1.6x faster.
    if tensors[0].dim() == 2 and tensors[0].size(0) < _NATIVE_GEMM_MIN_ROWS:
        return False
    from sample_efficient_gpt_b200.ops import gemm as G

    return all(t.dtype == torch.bfloat16 for t in tensors[:2]) and G.usable(*tensors)


def matmul_nt(x: Tensor, w: Tensor, out_dtype=None) -> Tensor:
    """x [M,K] @ w[N,K]^T -> [M,N] on the tcgen05 GEMM; the library GEMM for CPU tensors, fp32 runs and shapes that do
    not meet the TMA alignment rules."""
    if out_dtype in (None, x.dtype) and _native_gemm(x, w):
        from sample_efficient_gpt_b200.ops import gemm as G

        return G.gemm(x, w)
    if x.is_cuda and out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, w.t(), out_dtype=out_dtype)
    y = x @ w.t()
    return y if out_dtype is None else y.to(out_dtype)


def matmul_nn(x: Tensor, w: Tensor) -> Tensor:
    """x [M,N] @ w [N,K] -> [M,K] (data gradient of a linear layer)."""
    if _native_gemm(x, w):
        from sample_efficient_gpt_b200.ops import gemm as G

        return G.gemm(x, w, b_mn=True)
    return x @ w


def wgrad_accumulate(main_grad: Tensor, dy: Tensor, x: Tensor, first: bool):
    """main_grad (fp32 [N,K]) (+)= dy[T,N]^T @ x[T,K] with fp32 accumulation."""
    if _native_gemm(dy, x, main_grad):
        from sample_efficient_gpt_b200.ops import gemm as G

        G.gemm(dy, x, a_mn=True, b_mn=True, c=None if first else main_grad, out=main_grad, out_f32=True, beta=0.0 if first else 1.0)
        return
    if dy.is_cuda and dy.dtype != torch.float32:
        if first:
            torch.mm(dy.t(), x, out_dtype=torch.float32, out=main_grad)
        else:
            torch.addmm(main_grad, dy.t(), x, out_dtype=torch.float32, out=main_grad)
        return
    if first:
        torch.mm(dy.t().float(), x.float(), out=main_grad)
    else:
        main_grad.addmm_(dy.t().float(), x.float())


# ----------------------------------------------------------------------------- cross entropy
def linear_ce_fwd_bwd(h, w, targets, lse_square_scale, ignore_index, grad_scale, logit_scale=1.0, dw_out=None, need_grad=True):
    if h.is_cuda and h.dtype == torch.bfloat16 and has_kernel("ce_chunk_fwd_bwd"):
        from sample_efficient_gpt_b200.ops import cross_entropy as ce_impl

        return ce_impl.linear_ce_fwd_bwd(
            h, w, targets, lse_square_scale, ignore_index, grad_scale, logit_scale, dw_out=dw_out, need_grad=need_grad
        )
    if h.is_cuda and h.dtype == torch.bfloat16:
        _use_cuda(h, "ce_chunk_fwd_bwd")  # raises unless fallback is allowed
    return ref.linear_ce_fwd_bwd(
        h, w, targets, lse_square_scale, ignore_index, grad_scale, logit_scale, dw_out=dw_out, need_grad=need_grad
    )


class _SoftmaxCE(torch.autograd.Function):
    """Per-token (loss, z) from materialised logits; the gradient flows through ``loss`` only."""

    @staticmethod
    def forward(ctx, logits, targets, lse_square_scale, ignore_index):
        loss, z, lse = ref.softmax_ce_fwd(logits, targets, lse_square_scale, ignore_index)
        ctx.save_for_backward(logits, targets, lse)
        ctx.cfg = (lse_square_scale, ignore_index)
        ctx.mark_non_differentiable(z)
        return loss, z

    @staticmethod
    def backward(ctx, grad_loss, _grad_z):
        logits, targets, lse = ctx.saved_tensors
        s, ig = ctx.cfg
        return ref.softmax_ce_bwd(logits, targets, lse, grad_loss, s, ig), None, None, None


def softmax_cross_entropy(logits: Tensor, targets: Tensor, lse_square_scale: float = 1e-6, ignore_index: int = -100):
    return _SoftmaxCE.apply(logits, targets, lse_square_scale, ignore_index)


class _LinearCE(torch.autograd.Function):
    """mean-reduced fused head + loss: gradients are produced in the forward sweep and scaled in backward."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, lse_square_scale, ignore_index, logit_scale):
        need = hidden.requires_grad or weight.requires_grad
        T = hidden.size(0)
        lp = hidden.dtype
        loss_tok, z_tok, dh, dw = linear_ce_fwd_bwd(
            hidden.detach(), weight.detach().to(lp), targets, lse_square_scale, ignore_index, 1.0 / T, logit_scale, need_grad=need
        )
        if need:
            ctx.save_for_backward(dh, dw)
        ctx.wdtype = weight.dtype
        ctx.mark_non_differentiable(z_tok, loss_tok)
        return loss_tok.mean(), z_tok, loss_tok

    @staticmethod
    def backward(ctx, g_mean, _gz, _gl):
        dh, dw = ctx.saved_tensors
        return dh * g_mean.to(dh.dtype), (dw * g_mean).to(ctx.wdtype), None, None, None, None


def linear_cross_entropy(hidden, weight, targets, lse_square_scale=1e-6, ignore_index=-100, logit_scale=1.0):
    """Returns (mean loss [differentiable], per-token z, per-token loss [detached])."""
    return _LinearCE.apply(hidden, weight, targets, lse_square_scale, ignore_index, logit_scale)


# ----------------------------------------------------------------------------- optimizer kernels
def fused_adamw(ps, grads, ms, vs, shadows, lr, wd, beta1, beta2, eps, step_size):
    _count()
    ext().adamw(ps, grads, ms, vs, [s if s is not None else torch.empty(0, device=ps[0].device) for s in shadows],
                float(lr), float(wd), float(beta1), float(beta2), float(eps), float(step_size))


def fused_ema(shadow, srcs, decay):
    _count()
    ext().ema(shadow, srcs, float(decay))


def newton_schulz_cuda(G, epsilon, coeffs):
    from sample_efficient_gpt_b200.ops import newton_schulz as ns_impl

    return ns_impl.newton_schulz(G, epsilon, coeffs)
