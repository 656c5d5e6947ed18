"""CUDA path of the fused head projection + cross-entropy.

The [tokens, vocab] logits are produced chunk by chunk into one reused bf16 buffer, turned into losses and
(in place) into logit gradients by ``ce_chunk_fwd_bwd`` (DRAM sees one read and one write of the chunk), and
immediately consumed by the two gradient GEMMs, so the only full-size tensors are the inputs and outputs.
The three GEMMs of a chunk run on this package's tcgen05 GEMM (``x W^T``, ``dlogits W`` and ``dlogits^T x`` read their
operands in place through K-major / MN-major tensor maps; the weight gradient accumulates in fp32 through the GEMM's
``beta * C`` epilogue); ``SEGPT_DISABLE_KERNELS=ce_gemm`` sends them to the library instead.
Math: transformer/ops/cross_entropy.py:96-247 and fused_linear_cross_entropy.py:13-346 of the reference
(the latter is present but unused there; its live path stores all logits).
"""

from __future__ import annotations

import torch
from torch import Tensor

from sample_efficient_gpt_b200 import ops

_BUF: dict = {}


def _logits_buffer(rows: int, V: int, device) -> Tensor:
    key = (rows, V, str(device))
    buf = _BUF.get(key)
    if buf is None:
        _BUF.clear()
        buf = torch.empty((rows, V), dtype=torch.bfloat16, device=device)
        _BUF[key] = buf
    return buf


def linear_ce_fwd_bwd(h, w, targets, lse_square_scale, ignore_index, grad_scale, logit_scale=1.0, dw_out=None,
                      need_grad=True, chunk: int = 8192):
    assert h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "CUDA fused linear-CE runs in bf16"
    T, d = h.shape
    V = w.size(0)
    dev = h.device
    targets = targets.reshape(-1).to(torch.int64).contiguous()
    loss = torch.empty(T, dtype=torch.float32, device=dev)
    z = torch.empty(T, dtype=torch.float32, device=dev)
    lse = torch.empty(T, dtype=torch.float32, device=dev)
    dh = torch.empty_like(h) if need_grad else None
    dw = None
    if need_grad:
        dw = dw_out if dw_out is not None else torch.zeros((V, d), dtype=torch.float32, device=dev)
    chunk = min(chunk, T)
    buf = _logits_buffer(chunk, V, dev)
    ext = ops.ext()
    from sample_efficient_gpt_b200.ops import gemm as G

    own = ops.kernel_enabled("ce_gemm") and G.usable(h, w, buf) and d % 8 == 0 and (dw is None or G.usable(dw))
    for s in range(0, T, chunk):
        e = min(T, s + chunk)
        lg = buf[: e - s]
        if own:
            G.gemm(h[s:e], w, out=lg)
        else:
            torch.mm(h[s:e], w.t(), out=lg)
        ext.ce_chunk_fwd_bwd(lg, targets[s:e], loss[s:e], z[s:e], lse[s:e], lse_square_scale, ignore_index,
                             grad_scale, logit_scale, need_grad)
        ops._count()
        if need_grad:
            if own:
                G.gemm(lg, w, b_mn=True, out=dh[s:e])
                G.gemm(lg, h[s:e], a_mn=True, b_mn=True, c=dw, out=dw, out_f32=True, beta=1.0)
            else:
                torch.mm(lg, w, out=dh[s:e])
                torch.addmm(dw, lg.t(), h[s:e], out_dtype=torch.float32, out=dw)
    return loss, z, dh, dw
