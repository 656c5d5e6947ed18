"""NVTX ranges and CUDA-event phase timers.

``nvtx_range(name)`` works as a decorator and as a context manager.  It emits an NVTX range only
when ``ENABLE_PROF=1`` (same switch as utils/profiling.py:7-15 of the reference) and is free otherwise.
``PhaseTimer`` brackets phases of a step with CUDA events on the current stream, so the numbers are
device time and the host is never synchronised until ``summary()`` is called.
"""

from __future__ import annotations

import contextlib
import functools
import os

import torch

_ENABLED = os.environ.get("ENABLE_PROF", "0") == "1"


class _Range(contextlib.ContextDecorator):
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _ENABLED and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if _ENABLED and torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        return False


def nvtx_range(name: str):
    return _Range(name)


class PhaseTimer:
    """Device-side timing of named phases: ``with timer("fwd"): ...``."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._open: dict[str, list] = {}

    @contextlib.contextmanager
    def __call__(self, name: str):
        if not self.enabled:
            yield
            return
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        try:
            yield
        finally:
            end.record()
            self._open.setdefault(name, []).append((start, end))

    def summary(self, reset: bool = True) -> dict[str, float]:
        """Milliseconds per phase, summed over the calls since the last reset."""
        if not self.enabled:
            return {}
        torch.cuda.synchronize()
        out = {k: sum(s.elapsed_time(e) for s, e in v) for k, v in self._open.items()}
        if reset:
            self._open.clear()
        return out


def mem(tag: str) -> str:
    """Allocated / reserved device memory as a log line (trainer.py:48-51 of the reference)."""
    if not torch.cuda.is_available():
        return f"{tag}: cpu"
    alloc = torch.cuda.memory_allocated() / 1e9
    resv = torch.cuda.memory_reserved() / 1e9
    return f"{tag}: allocated={alloc:.2f} GB, reserved={resv:.2f} GB"
