"""Newton-Schulz orthogonalisation with the seven "polar express" coefficient triples.

Math (training/optimizers/muon_triton.py:327-377 of the reference): ``X0 = bf16(G)``, transposed when
rows > cols, divided by ``||X0||_F + 1e-7``; per triple (a, b, c): ``A = X X^T``, ``B = b A + c A A``,
``X = a X + B X``; every product accumulates in fp32 and is rounded to bf16.  Works on a single
matrix or on a batch ``[n, rows, cols]`` (one launch per product for the whole batch).

On a GPU the three products run on the sm_100a tcgen05 GEMM of this package when it is built
(``ops.ns_gemm``); this file is the plain PyTorch statement that also serves as the CPU oracle.
"""

from __future__ import annotations

import torch
from torch import Tensor

POLAR_EXPRESS_COEFFS = (
    (7.2086, -15.5131, 9.0178),
    (3.9623, -2.5813, 0.4542),
    (3.9466, -2.5765, 0.4544),
    (3.8991, -2.5671, 0.4566),
    (3.7186, -2.5308, 0.4653),
    (3.1390, -2.3073, 0.4733),
    (2.1715, -1.5246, 0.3885),
)


def _mm(a: Tensor, b: Tensor) -> Tensor:
    """bf16 x bf16 -> bf16 with fp32 accumulation (explicit upcast on CPU, tensor cores on CUDA)."""
    if a.is_cuda:
        return a @ b
    return (a.float() @ b.float()).to(a.dtype)


def newton_schulz(G: Tensor, epsilon: float = 1e-7, coeffs=POLAR_EXPRESS_COEFFS, dtype=torch.bfloat16) -> Tensor:
    if G.is_cuda and dtype == torch.bfloat16:
        from sample_efficient_gpt_b200 import ops

        if ops.has_kernel("gemm") and ops.kernel_enabled("ns_gemm"):
            return ops.newton_schulz_cuda(G, epsilon, coeffs)
    X = G.to(dtype)
    transposed = G.size(-2) > G.size(-1)
    if transposed:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + epsilon)
    X = X.contiguous()
    for a, b, c in coeffs:
        A = _mm(X, X.mT)
        if X.is_cuda:
            B = torch.baddbmm(A, A, A, beta=b, alpha=c) if A.ndim == 3 else torch.addmm(A, A, A, beta=b, alpha=c)
            X = torch.baddbmm(X, B, X, beta=a) if X.ndim == 3 else torch.addmm(X, B, X, beta=a)
        else:
            Af = A.float()
            B = (b * Af + c * (Af @ Af)).to(dtype)
            X = (a * X.float() + B.float() @ X.float()).to(dtype)
    if transposed:
        X = X.mT
    return X
