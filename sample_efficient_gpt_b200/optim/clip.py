"""Global gradient norm and clipping (training/optimizer.py:190-206 of the reference).

``clip_grad_norm_`` scales only when it receives a re-iterable collection.  The reference trainer
hands it a generator, which the norm pass exhausts, so its gradients are never scaled; the trainer
here reproduces that by default (``trainer.clip_fix=false``) and passes a list when the fix is on.
"""

from __future__ import annotations

from collections.abc import Iterable

import torch
from torch import Tensor


def grad_norm(grads: list[Tensor]) -> Tensor:
    """sqrt(sum ||g||^2) with one fused multi-tensor norm."""
    if not grads:
        raise ValueError("grads are empty!")
    norms = torch._foreach_norm(grads)
    return torch.linalg.vector_norm(torch.stack([n.float() for n in norms]))


def clip_grad_norm_(params: Iterable[torch.nn.Parameter], max_grad_norm: float = 1.0, eps: float = 1e-8) -> Tensor:
    grads = [p.grad for p in params if p.grad is not None]
    norm = grad_norm(grads)
    # a second pass over ``params``: empty for a generator, the full list otherwise
    second = [p.grad for p in params if p.grad is not None]
    if second:
        # scale by min(1, max/(norm+eps)) without a host sync
        factor = (max_grad_norm / (norm + eps)).clamp(max=1.0)
        factor = torch.where(norm >= max_grad_norm, factor, torch.ones_like(factor))
        torch._foreach_mul_(second, factor)
    return norm
