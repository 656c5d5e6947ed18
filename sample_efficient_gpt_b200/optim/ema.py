"""Exponential moving average of the model weights, kept during training.

The reference only averages saved checkpoints after the fact
(scripts/data_processing/sft/ema_posthoc.py:88-98: ``ema = d*ema + (1-d)*p`` with d = 0.8).  This class
applies the same recurrence every ``every`` optimizer steps on the device (one multi-tensor kernel)
and writes ``<iteration>_ema.pt`` in the ordinary checkpoint layout.
"""

from __future__ import annotations

import torch
from torch import Tensor


class WeightEMA:
    def __init__(self, model: torch.nn.Module, decay: float = 0.8, every: int = 10):
        self.decay = decay
        self.every = max(1, int(every))
        self.steps_seen = 0
        self.names: list[str] = []
        self.sources: list[Tensor] = []
        self.shadow: list[Tensor] = []
        seen: set[int] = set()
        for name, t in model.state_dict().items():
            if not torch.is_floating_point(t):
                continue
            self.names.append(name)
            self.sources.append(t)
            if id(t) in seen:
                continue
            seen.add(id(t))
        # aliases (e.g. the inert lm_head.weight) share storage with their source: average once
        self._unique_idx = []
        ptrs: dict[int, int] = {}
        for i, t in enumerate(self.sources):
            if t.data_ptr() in ptrs:
                continue
            ptrs[t.data_ptr()] = i
            self._unique_idx.append(i)
        self.shadow = [self.sources[i].detach().clone() for i in self._unique_idx]
        self._ptr_to_shadow = {self.sources[i].data_ptr(): s for i, s in zip(self._unique_idx, self.shadow)}

    @torch.no_grad()
    def maybe_update(self) -> bool:
        """Call once per optimizer step; updates on every ``every``-th call."""
        self.steps_seen += 1
        if self.steps_seen % self.every:
            return False
        self.update()
        return True

    @torch.no_grad()
    def update(self):
        srcs = [self.sources[i].detach() for i in self._unique_idx]
        if srcs and srcs[0].is_cuda:
            from sample_efficient_gpt_b200 import ops

            if ops.has_kernel("ema"):
                ops.fused_ema(self.shadow, srcs, self.decay)
                return
        torch._foreach_lerp_(self.shadow, srcs, 1.0 - self.decay)

    def state_dict(self) -> dict[str, Tensor]:
        """Averaged weights under the model's own state-dict keys (aliases included)."""
        return {n: self._ptr_to_shadow[t.data_ptr()] for n, t in zip(self.names, self.sources)}

    def load_state_dict(self, sd: dict[str, Tensor]):
        for n, t in zip(self.names, self.sources):
            if n in sd:
                self._ptr_to_shadow[t.data_ptr()].copy_(sd[n])
