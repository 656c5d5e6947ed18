"""AdamW (decoupled decay, bias correction folded into the step size) and a toy SGD.

Update rule and state layout (``t``, ``m``, ``v``; ``t`` starts at 1 and is stored incremented) are
those of training/optimizer.py:13-112 of the reference, so optimizer state in its checkpoints loads.
NaN gradient entries are zeroed.  Differences: the whole parameter list is updated with multi-tensor
calls (one fused CUDA kernel over all tensors when the extension is built, ``torch._foreach`` ops
otherwise) and nothing synchronises the host.
"""

from __future__ import annotations

from typing import Any

import torch
from torch import Tensor

from sample_efficient_gpt_b200.utils.profiling import nvtx_range


class SGD(torch.optim.Optimizer):
    """p -= lr / sqrt(t + 1) * g."""

    def __init__(self, params, lr: float = 1e-3):
        super().__init__(params, dict(lr=lr))

    @torch.no_grad()
    def step(self, closure: Any | None = None):
        loss = None if closure is None else closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                t = st.get("t", 0)
                p.add_(p.grad, alpha=-group["lr"] / (t + 1) ** 0.5)
                st["t"] = t + 1
        return loss


class AdamW(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-4, betas=(0.9, 0.95), weight_decay: float = 1e-6, eps: float = 1e-8):
        super().__init__(params=params, defaults=dict(lr=lr, betas=betas, weight_decay=weight_decay, eps=eps))
        self.lowp_shadows: dict[Tensor, Tensor] = {}  # param -> bf16 copy refreshed by the fused kernel

    @nvtx_range("adamw step")
    @torch.no_grad()
    def step(self, closure: Any | None = None):
        if closure is not None:
            closure()
        device = self.param_groups[0]["params"][0].device
        for group in self.param_groups:
            lr = group["lr"]
            beta1, beta2 = group["betas"]
            wd, eps = group["weight_decay"], group["eps"]
            # tensors that share a step count share a step size: bucket by t
            by_t: dict[int, list[Tensor]] = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "m" not in st:
                    st["t"] = st.get("t", 1)
                    st["m"] = torch.zeros_like(p, requires_grad=False)
                    st["v"] = torch.zeros_like(p, requires_grad=False)
                by_t.setdefault(int(st["t"]), []).append(p)
            for t, ps in by_t.items():
                step_size = lr * (1 - beta2**t) ** 0.5 / (1 - beta1**t)
                self._update(ps, lr, wd, beta1, beta2, eps, step_size)
                for p in ps:
                    self.state[p]["t"] = t + 1
        return torch.zeros((), dtype=torch.float32, device=device)

    def _update(self, ps, lr, wd, beta1, beta2, eps, step_size):
        grads = [p.grad for p in ps]
        ms = [self.state[p]["m"] for p in ps]
        vs = [self.state[p]["v"] for p in ps]
        if ps[0].is_cuda:
            from sample_efficient_gpt_b200 import ops

            if ops.has_kernel("adamw"):
                shadows = [self.lowp_shadows.get(p) for p in ps]
                ops.fused_adamw(ps, grads, ms, vs, shadows, lr, wd, beta1, beta2, eps, step_size)
                return
        grads = [torch.nan_to_num(g, nan=0.0, posinf=float("inf"), neginf=float("-inf")) for g in grads]
        torch._foreach_mul_(ps, 1 - lr * wd)
        torch._foreach_lerp_(ms, grads, 1 - beta1)
        torch._foreach_mul_(vs, beta2)
        torch._foreach_addcmul_(vs, grads, grads, value=1 - beta2)
        denom = torch._foreach_sqrt(vs)
        torch._foreach_add_(denom, eps)
        torch._foreach_addcdiv_(ps, ms, denom, value=-step_size)
        for p in ps:
            sh = self.lowp_shadows.get(p)
            if sh is not None:
                sh.copy_(p)
