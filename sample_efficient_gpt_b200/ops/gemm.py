"""Python face of the tcgen05 GEMM (csrc/gemm.cu): ``D = alpha * A op(B) + beta * C`` on bf16 operands.

``mm_nt(x, w)`` = x @ w^T, ``mm_nn(x, w)`` = x @ w, ``mm_tn(a, b)`` = a^T @ b; all read their operands in place
(the kernel takes K-major and MN-major tiles), accept a leading batch dimension and accumulate in fp32.
``usable(t...)`` tells whether the tensors meet the TMA alignment rules (contiguous last dimension, row and
batch strides multiples of 8 elements, 16-byte aligned base); callers fall back to the library GEMM otherwise.
"""

from __future__ import annotations

import os

import torch
from torch import Tensor

from sample_efficient_gpt_b200 import ops


def usable(*tensors: Tensor) -> bool:
    if not ops.has_kernel("gemm"):
        return False
    for t in tensors:
        if t is None:
            continue
        if not (t.is_cuda and t.dim() in (2, 3) and t.stride(-1) == 1 and t.stride(-2) % 8 == 0 and t.data_ptr() % 16 == 0):
            return False
        if t.dim() == 3 and t.stride(0) % 8 != 0:
            return False
    return True


# Which kernel runs: "pair" = one 256 x 256 tile per CTA pair (tcgen05 cta_group::2, TMA-store epilogue, tiles of
# the last wave cut along the contraction), "single" = one CTA per 128-row tile.
DEFAULT_IMPL = 0 if os.environ.get("SEGPT_GEMM_IMPL", "pair") == "single" else 1


def gemm(a, b, c=None, out=None, out_f32=False, a_mn=False, b_mn=False, alpha=1.0, beta=0.0, symmetric=False,
         extra_dst: list[int] | None = None, wait: tuple | None = None, route: tuple | None = None, impl: int | None = None,
         split_k: bool = True, wait_limit: int = 0) -> Tensor:
    """``impl``: 1 pair kernel, 0 single-CTA kernel, None = ``SEGPT_GEMM_IMPL``.  ``split_k`` (pair kernel): tiles of the last, partly filled
    wave may be cut into ranges of the contraction that several pairs compute and one of them sums in a fixed order (a
    per-stream workspace of the extension holds the parts, allocated at the first call on a stream - make that call
    before capturing the stream into a CUDA graph); False: whole tiles only.  ``wait_limit``: cycles a
    wait inside the kernel may stand still before it gives up and sets the status word (0 = default).
    ``extra_dst``: device addresses of up to 7 more buffers with the output's layout (peer memory of other ranks);
    every output tile is stored to all of them from the epilogue.
    ``wait`` = (flags int32 tensor, seq, region_rows): rows ``[r * region_rows, (r+1) * region_rows)`` of ``a`` are being
    written by rank r and are complete once ``flags[r] >= seq``; the kernel's producer waits per tile (bounded).
    ``route`` = (addresses, route_rows, batch_stride, base, ld): the output is not stored locally; rows
    ``[r * route_rows, (r+1) * route_rows)`` of batch entry ``b`` go to buffer ``addresses[r]`` (of rank r) at element offset
    ``base + b * batch_stride + (row - r * route_rows) * ld + column``."""
    ops._count()
    flags, seq, rows = wait if wait is not None else (None, 0, 0)
    rp, rr, rbs, rbase, rld = route if route is not None else ([], 0, 0, 0, 0)
    return ops.ext().gemm(a, b, c, out, out_f32, a_mn, b_mn, float(alpha), float(beta), symmetric, extra_dst or [], flags, int(seq), int(rows),
                          list(rp), int(rr), int(rbs), int(rbase), int(rld), DEFAULT_IMPL if impl is None else int(impl), bool(split_k),
                          int(wait_limit))


def mm_nt(x: Tensor, w: Tensor, **kw) -> Tensor:
    """x [.., M, K] @ w [.., N, K]^T."""
    return gemm(x, w, **kw)


def mm_nn(x: Tensor, w: Tensor, **kw) -> Tensor:
    """x [.., M, K] @ w [.., K, N]."""
    return gemm(x, w, b_mn=True, **kw)


def mm_tn(a: Tensor, b: Tensor, **kw) -> Tensor:
    """a [.., K, M]^T @ b [.., K, N] (weight gradient: dy^T @ x)."""
    return gemm(a, b, a_mn=True, b_mn=True, **kw)


def status(device_index: int | None = None) -> int:
    """0 unless a bounded wait inside a GEMM kernel gave up (synchronises the device)."""
    if device_index is None:
        device_index = torch.cuda.current_device()
    return int(ops.ext().gemm_status(device_index))
