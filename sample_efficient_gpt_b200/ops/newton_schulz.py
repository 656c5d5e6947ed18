"""Newton-Schulz chain on the tcgen05 GEMM.

Per iteration and for a whole batch of same-shape matrices: ``A = X X^T`` and ``B = b A + c A A`` compute only the
tiles on or above the diagonal and mirror them (both results are symmetric); ``X = a X + B X`` reads X as an MN-major
operand, so nothing is transposed.  Every product accumulates in fp32 and is rounded to bf16, as in the reference
(training/optimizers/muon_triton.py:327-377).  Shapes the TMA path cannot take (a side that is not a multiple of 8,
e.g. the 18 x d gate matrices) use the library batched GEMM.
"""

from __future__ import annotations

import torch
from torch import Tensor

from sample_efficient_gpt_b200.ops import gemm as G


def newton_schulz(Gm: Tensor, epsilon: float, coeffs) -> Tensor:
    X = Gm.to(torch.bfloat16)
    squeeze = X.dim() == 2
    if squeeze:
        X = X.unsqueeze(0)
    transposed = X.size(-2) > X.size(-1)
    if transposed:
        X = X.mT
    X = (X / (X.norm(dim=(-2, -1), keepdim=True) + epsilon)).contiguous()
    r = X.size(-2)
    if r % 8 == 0 and X.size(-1) % 8 == 0 and G.usable(X):
        A = torch.empty((X.size(0), r, r), dtype=torch.bfloat16, device=X.device)
        B = torch.empty_like(A)
        Y = torch.empty_like(X)
        for a, b, c in coeffs:
            G.gemm(X, X, out=A, symmetric=True)
            G.gemm(A, A, c=A, out=B, alpha=c, beta=b, symmetric=True)
            G.gemm(B, X, c=X, out=Y, b_mn=True, alpha=1.0, beta=a)
            X, Y = Y, X
    else:
        for a, b, c in coeffs:
            A = X @ X.mT
            B = torch.baddbmm(A, A, A, beta=b, alpha=c)
            X = torch.baddbmm(X, B, X, beta=a)
    if transposed:
        X = X.mT
    return X.squeeze(0) if squeeze else X
