"""Newton-Schulz chain on the tcgen05 GEMM.

Per iteration and for a whole batch of same-shape matrices: the Gram matrix ``A`` computes only the tiles on or above
the diagonal and mirrors them when its contraction is long (>= 2048), and all tiles otherwise; ``B = b A + c A A`` is computed in full, because with the addend fetched by TMA the
plain epilogue is faster than the mirrored one on this short contraction; the update ``a X + B X`` (wide X) or
``a X + X B`` (tall X) reads its operands in place (K-major and MN-major tiles), so tall matrices are never
transposed: for ``R > C`` the chain runs on ``X^T`` implicitly with ``A = X^T X``.  Every product accumulates in fp32
and is rounded to bf16, as in the reference (training/optimizers/muon_triton.py:327-377).  A short side that is not a
multiple of 8 (the 18 x d gate matrices; TMA wants 16-byte rows) is padded with zero rows or columns, which the chain
leaves zero, so the result is the one of the unpadded matrix.
"""

from __future__ import annotations

import torch
from torch import Tensor

import os

from sample_efficient_gpt_b200.ops import gemm as G

_SYM_B = os.environ.get("SEGPT_NS_SYMMETRIC_B", "0") == "1"  # mirrored instead of full computation of b A + c A A
# The Gram matrix is mirrored (upper-triangle tiles only) when its contraction is at least this long: the mirrored epilogue
# is slower than the TMA store and hides only behind a long mainloop (30 matrices, chain of 5: 1152 x 1152 runs 1.95 ms
# mirrored and 1.56 ms in full; 1152 x 3072 2.71 against 2.78 ms; 6144 x 1152 4.06 against 4.71 ms).
_SYM_A_MIN_K = int(os.environ.get("SEGPT_NS_SYMMETRIC_A_MIN_K", "2048"))


def ns_iterations(X: Tensor, Y: Tensor, coeffs, final_extra_dst=None) -> Tensor:
    """Run the chain on normalised bf16 ``X [n, R, C]`` ping-ponging with ``Y`` (same shape); returns the buffer
    that holds the result (``Y`` for an odd number of iterations).

    ``final_extra_dst(buffer) -> list[int]``: peer addresses that mirror the buffer receiving the last iteration's
    output; the last GEMM then stores every tile to those as well (the all-gather of the result happens in its
    epilogue).  Returns ``(result, True)`` instead of ``result`` when that happened."""
    n, R, C = X.shape
    tall = R > C
    r = min(R, C)
    if r % 8 != 0 and max(R, C) % 8 == 0 and X.is_cuda and X.dtype == torch.bfloat16 and G.usable(X.new_empty(8, 8)):
        rp = (r + 7) // 8 * 8
        Xp = X.new_zeros((n, R, rp) if tall else (n, rp, C))
        (Xp[:, :, :r] if tall else Xp[:, :r]).copy_(X)
        res = ns_iterations(Xp, torch.empty_like(Xp), coeffs)
        Y.copy_(res[:, :, :r] if tall else res[:, :r])
        return Y
    if r % 8 == 0 and max(R, C) % 8 == 0 and G.usable(X, Y):
        A = torch.empty((n, r, r), dtype=torch.bfloat16, device=X.device)
        B = torch.empty_like(A)
        last = len(coeffs) - 1
        pushed = False
        for it, (a, b, c) in enumerate(coeffs):
            sym_a = max(R, C) >= _SYM_A_MIN_K
            if tall:
                G.gemm(X, X, out=A, a_mn=True, b_mn=True, symmetric=sym_a)  # X^T X
            else:
                G.gemm(X, X, out=A, symmetric=sym_a)  # X X^T
            G.gemm(A, A, c=A, out=B, alpha=c, beta=b, symmetric=_SYM_B)
            extra = final_extra_dst(Y) if (it == last and final_extra_dst is not None) else None
            pushed = pushed or bool(extra)
            if tall:
                G.gemm(X, B, c=X, out=Y, alpha=1.0, beta=a, extra_dst=extra)  # X B (B symmetric)
            else:
                G.gemm(B, X, c=X, out=Y, b_mn=True, alpha=1.0, beta=a, extra_dst=extra)  # B X
            X, Y = Y, X
        return (X, True) if final_extra_dst is not None and pushed else X
    for a, b, c in coeffs:
        A = (X.mT @ X) if tall else (X @ X.mT)
        B = torch.baddbmm(A, A, A, beta=b, alpha=c)
        if tall:
            torch.baddbmm(X, X, B, beta=a, out=Y)
        else:
            torch.baddbmm(X, B, X, beta=a, out=Y)
        X, Y = Y, X
    return X


def newton_schulz(Gm: Tensor, epsilon: float, coeffs) -> Tensor:
    """Orthogonalise ``Gm`` ([R, C] or [n, R, C], any float dtype): normalise by the Frobenius norm, run the chain."""
    X = Gm.to(torch.bfloat16)
    squeeze = X.dim() == 2
    if squeeze:
        X = X.unsqueeze(0)
    X = (X / (X.norm(dim=(-2, -1), keepdim=True) + epsilon)).contiguous()
    out = ns_iterations(X, torch.empty_like(X), coeffs)
    return out.squeeze(0) if squeeze else out
