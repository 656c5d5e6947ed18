"""Bucketed data parallelism.

Same contract as the reference's custom DDP (training/distributed/ddp_bucket.py:10-134):
  * parameters are broadcast from rank 0 at construction;
  * buckets are formed walking ``named_parameters()`` in reverse, starting a new bucket when the dtype
    changes or adding the tensor would exceed ``bucket_size_mb`` of parameter bytes (30.1 MiB);
  * when the last gradient of a bucket arrives the bucket is summed across ranks with bf16 on the wire
    (no division: the loss is pre-scaled by ``local_bs / global_bs``), overlapping the rest of backward;
  * ``no_sync()`` suppresses the reduction (gradient accumulation), and
    ``finish_gradient_synchronization()`` waits for every bucket and returns the host seconds it waited.
Differences: every gradient lives in one persistent flat fp32 buffer (``p.grad`` are views; a bucket is
a contiguous slice), so nothing is flattened or copied back; the per-bucket cast/reduce either goes
through ``torch.distributed`` (NCCL or gloo) or through this package's own NVLink kernels
(``parallel.symm.SymmComm``: reduce-scatter + all-gather over peer memory with the bf16<->fp32 casts
fused in).  Gradients can be announced by autograd hooks or, from the fused engine, by
``grads_ready(params)``.
"""

from __future__ import annotations

import time
from contextlib import contextmanager

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor


def assign_buckets(named_params: list[tuple[str, Tensor]], bucket_bytes: int) -> list[list[str]]:
    """Bucket membership (lists of names, in reverse registration order) by the reference's rule."""
    buckets: list[list[str]] = [[]]
    size, prev_dt = 0, None
    for name, p in reversed(named_params):
        nbytes = p.numel() * p.element_size()
        if (prev_dt is not None and p.dtype != prev_dt) or size + nbytes > bucket_bytes:
            if buckets[-1]:
                buckets.append([])
            size = 0
        buckets[-1].append(name)
        size += nbytes
        prev_dt = p.dtype
    return [b for b in buckets if b]


class DDP(nn.Module):
    def __init__(self, module: nn.Module, bucket_size_mb: float = 30.1, comm=None, process_group=None, is_local=None):
        """``is_local(name)``: parameters that differ per rank by design (expert-parallel experts) - neither broadcast
        nor reduced; their ``.grad`` is left to their owner."""
        super().__init__()
        assert dist.is_initialized(), "DDP needs an initialised process group"
        self.module = module
        self.group = process_group
        self.comm = comm  # SymmComm for the NVLink kernels, None for torch.distributed collectives
        self.world = dist.get_world_size(process_group)
        is_local = is_local or (lambda name: False)
        named = [(n, p) for n, p in module.named_parameters() if p.requires_grad and not is_local(n)]
        self._broadcast_parameters([p for n, p in module.named_parameters() if not is_local(n)])
        by_name = dict(named)
        self.bucket_names = assign_buckets(named, int(bucket_size_mb * 1024 * 1024))
        # flat fp32 gradient storage, bucket after bucket
        # Every gradient view starts on a 256-byte boundary (the kernels read gradients with 16-byte vector
        # accesses) and every bucket is padded to the length the reduction kernels need; padding stays zero.
        palign = 64
        align = max(comm.bucket_alignment() if comm is not None else 1, palign)
        align = (align + palign - 1) // palign * palign
        dev = named[0][1].device
        layout, start = [], 0
        for names in self.bucket_names:
            off, offs = start, []
            for n in names:
                offs.append(off)
                off = (off + by_name[n].numel() + palign - 1) // palign * palign
            end = start + (off - start + align - 1) // align * align
            layout.append((start, end, offs))
            start = end
        self.flat_grads = torch.zeros(start, dtype=torch.float32, device=dev)
        self.bucket_ranges: list[tuple[int, int]] = []
        self.param_bucket: dict[Tensor, int] = {}
        self._views: dict[Tensor, Tensor] = {}
        for bi, (names, (b_start, b_end, offs)) in enumerate(zip(self.bucket_names, layout)):
            for n, off in zip(names, offs):
                p = by_name[n]
                self._views[p] = self.flat_grads[off : off + p.numel()].view_as(p)
                p.grad = self._views[p]
                self.param_bucket[p] = bi
            self.bucket_ranges.append((b_start, b_end))
        self.bucket_sizes = [len(n) for n in self.bucket_names]
        self._pending = [0] * len(self.bucket_names)
        self._should_all_reduce = True
        self.handles: list = []
        self.total_bytes = 0
        if comm is not None:
            comm.register_buckets(self.flat_grads, self.bucket_ranges)
        for _, p in named:
            p.register_post_accumulate_grad_hook(self._autograd_hook)

    def _broadcast_parameters(self, params: list[Tensor]):
        # coalesce: one broadcast per ~256 MB instead of one per tensor
        chunk, size = [], 0
        def flush():
            nonlocal chunk, size
            if not chunk:
                return
            flat = torch.cat([p.detach().reshape(-1).float() for p in chunk])
            dist.broadcast(flat, src=0, group=self.group)
            o = 0
            for p in chunk:
                p.data.copy_(flat[o : o + p.numel()].view_as(p))
                o += p.numel()
            chunk, size = [], 0
        for p in params:
            chunk.append(p)
            size += p.numel() * 4
            if size >= 256 << 20:
                flush()
        flush()

    # ------------------------------------------------------------------ gradient arrival
    def _autograd_hook(self, p: Tensor):
        view = self._views[p]
        if p.grad is not None and p.grad.data_ptr() != view.data_ptr():
            # .grad was re-created (zero_grad(set_to_none=True) was used): move it back into the flat buffer
            view.copy_(p.grad)
            p.grad = view
        self.grads_ready([p])

    def grads_ready(self, params):
        """Mark the gradients of ``params`` as final for this step; launches complete buckets."""
        if not self._should_all_reduce:
            return
        for p in params:
            bi = self.param_bucket.get(p)
            if bi is None:
                continue
            self._pending[bi] += 1
            self.total_bytes += p.numel() * 4
            if self._pending[bi] == self.bucket_sizes[bi]:
                self._pending[bi] = 0
                self._launch(bi)

    def _launch(self, bi: int):
        s, e = self.bucket_ranges[bi]
        flat = self.flat_grads[s:e]
        if self.comm is not None:
            self.comm.all_reduce_bucket(bi)
            return
        wire = flat.to(torch.bfloat16)
        work = dist.all_reduce(wire, dist.ReduceOp.SUM, group=self.group, async_op=True)
        self.handles.append((work, wire, flat))

    @contextmanager
    def no_sync(self):
        before = self._should_all_reduce
        self._should_all_reduce = False
        try:
            yield
        finally:
            self._should_all_reduce = before

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def zero_grad(self, set_to_none: bool = False):
        self.flat_grads.zero_()

    def reduced_grad_norm(self, extra: list[Tensor] | None = None) -> Tensor | None:
        """Gradient norm from the partial sums of squares that the NVLink reduction kernels produced while reducing
        (None with the torch.distributed path).  ``extra``: gradients that did not go through the buckets (rank-local
        parameters).  Call once per step, after ``finish_gradient_synchronization``."""
        if self.comm is None:
            return None
        sq = self.comm.take_grad_sq()
        if extra:
            sq = sq + torch.stack([n.float() ** 2 for n in torch._foreach_norm(extra)]).sum()
        return sq.sqrt().squeeze(0)

    def finish_gradient_synchronization(self) -> float:
        t0 = time.monotonic()
        if self.comm is not None:
            self.comm.wait_all()
        for work, wire, flat in self.handles:
            work.wait()
            flat.copy_(wire)
        self.handles.clear()
        self.total_bytes = 0
        return time.monotonic() - t0


class NaiveDDP(nn.Module):
    """One asynchronous all-reduce per parameter (training/distributed/ddp.py:12-58); kept for comparison."""

    def __init__(self, module: nn.Module):
        super().__init__()
        assert dist.is_initialized()
        self.module = module
        self.handles = []
        for p in module.parameters():
            dist.broadcast(p.data, src=0)
            if p.requires_grad:
                p.register_post_accumulate_grad_hook(self._hook)

    def _hook(self, p: Tensor):
        self.handles.append(dist.all_reduce(p.grad, dist.ReduceOp.SUM, async_op=True))

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def finish_gradient_synchronization(self) -> float:
        t0 = time.monotonic()
        for h in self.handles:
            h.wait()
        self.handles.clear()
        return time.monotonic() - t0
