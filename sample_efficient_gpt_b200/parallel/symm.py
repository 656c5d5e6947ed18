"""Communicator for this package's NVLink kernels (csrc/comm.cu) on symmetric memory.

Buffers are allocated with ``torch.distributed._symmetric_memory`` (same size on every rank, peer-mapped into every
process, with an NVLS multicast mapping when the fabric supports it); the kernels only ever see raw pointers.
NCCL stays the bootstrap (process group, rendezvous) and the fallback.

  * ``register_buckets`` / ``all_reduce_bucket`` / ``wait_all``: the bucketed gradient all-reduce of ``parallel.ddp.DDP``
    as one kernel per bucket on a high-priority side stream (reduce-scatter + all-gather over peer memory with the
    fp32 -> bf16 -> fp32 casts fused in), ordered after the producer stream with an event and joined without a host sync.
  * ``symm_zeros`` / ``all_gather_inplace``: buffers for, and the all-gather of, the sharded Muon updates.
  * ``check()``: host read of the status word that a kernel sets when a bounded wait on a peer gave up.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from sample_efficient_gpt_b200 import ops


class CommTimeout(RuntimeError):
    pass


class SymmComm:
    def __init__(self, device: torch.device, group, use_multimem: bool, blocks: int):
        import torch.distributed._symmetric_memory as symm_mem

        if not ops.has_kernel("comm_allreduce_bucket"):
            raise RuntimeError("comm kernels are not built")
        self._sm = symm_mem
        self.device = device
        self.group = group if group is not None else dist.group.WORLD
        self.group_name = self.group.group_name
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        ext = ops.ext()
        if self.world > ext.COMM_MAX_RANKS:
            raise RuntimeError(f"at most {ext.COMM_MAX_RANKS} ranks")
        self.blocks = min(blocks, ext.COMM_MAX_BLOCKS)
        self.use_multimem = use_multimem
        self.stream = torch.cuda.Stream(device=device, priority=-1)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        # Two flag channels with their own sequence numbers: kernels of one channel run in the same order on every rank
        # (they share a stream); kernels of different channels may be in flight at the same time and must not see each
        # other's flag words.  Channel "bucket": gradient all-reduces on the side stream.  Channel "main": barriers and
        # all-gathers on the caller's stream (Muon step, expert-parallel exchange).
        self.seq = 1
        self.seq_main = 1
        self._handles: dict[int, tuple] = {}  # data_ptr -> (tensor, handle)
        self.flags, self._flags_hdl = self._alloc(ext.COMM_MAX_BLOCKS * ext.COMM_MAX_RANKS * 4, zero=True)
        self.flag_ptrs = [int(p) for p in self._flags_hdl.buffer_ptrs]
        self.flags_main, self._flags_main_hdl = self._alloc(ext.COMM_MAX_BLOCKS * ext.COMM_MAX_RANKS * 4, zero=True)
        self.flag_ptrs_main = [int(p) for p in self._flags_main_hdl.buffer_ptrs]
        self.wire = None
        # sum of squares of the reduced gradient slices this rank owns, accumulated by the bucket kernels of one step
        self.grad_sq = torch.zeros(1, dtype=torch.float32, device=device)
        self.bucket_ranges: list[tuple[int, int]] = []
        self.flat_grads: Tensor | None = None

    @classmethod
    def create(cls, device, use_multimem: bool = False, group=None, blocks: int = 32) -> "SymmComm":
        return cls(torch.device(device), group, use_multimem, blocks)

    # ------------------------------------------------------------------ allocation
    def _alloc(self, nbytes: int, zero: bool = True):
        nbytes = (nbytes + 255) // 256 * 256
        t = self._sm.empty(nbytes, dtype=torch.uint8, device=self.device)
        if zero:
            t.zero_()
        hdl = self._sm.rendezvous(t, self.group_name)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every rank has zeroed its buffer before anyone touches a peer's
        self._handles[t.data_ptr()] = (t, hdl)
        return t, hdl

    def symm_zeros(self, shape, dtype) -> Tensor:
        n = 1
        for s in shape:
            n *= s
        raw, _ = self._alloc(n * torch.empty((), dtype=dtype).element_size())
        return raw[: n * torch.empty((), dtype=dtype).element_size()].view(dtype).view(*shape)

    def _handle_of(self, t: Tensor):
        base = t.untyped_storage().data_ptr()
        ent = self._handles.get(base)
        if ent is None:
            raise ValueError("tensor was not allocated with SymmComm.symm_zeros")
        return ent[1], t.data_ptr() - base

    # ------------------------------------------------------------------ gradient buckets
    def bucket_alignment(self) -> int:
        return 8 * self.world

    def register_buckets(self, flat_grads: Tensor, ranges: list[tuple[int, int]]):
        """ranges are [start, end) element ranges of flat_grads, each a multiple of ``bucket_alignment()`` long."""
        for s, e in ranges:
            assert (e - s) % self.bucket_alignment() == 0 and s % 8 == 0, "bucket ranges must be padded for the kernels"
        self.flat_grads = flat_grads
        self.bucket_ranges = list(ranges)
        total = ranges[-1][1]
        self.wire, hdl = self._alloc(total * 2, zero=True)
        self.wire_ptrs = [int(p) for p in hdl.buffer_ptrs]
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        self.mc_ptr = mc if (self.use_multimem and mc) else 0
        if self.use_multimem and not mc:
            raise RuntimeError("NVLS multicast is not available for this allocation")

    def all_reduce_bucket(self, bi: int):
        s, e = self.bucket_ranges[bi]
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self.stream.wait_event(ev)
        with torch.cuda.stream(self.stream):
            ops.ext().comm_allreduce_bucket(self.flat_grads[s:e], self.wire_ptrs, self.flag_ptrs, self.mc_ptr, s, self.rank,
                                            self.seq, self.blocks, self.status, self.grad_sq, 0, self.wire.numel() // 2)
        ops._count()
        self.seq += 2

    def wait_all(self):
        torch.cuda.current_stream(self.device).wait_stream(self.stream)

    def take_grad_sq(self) -> Tensor:
        """Sum over ranks of the per-rank partial sums of squares gathered since the last call (= ||reduced gradients||^2 of
        everything that went through ``all_reduce_bucket``); resets the accumulator.  Call after ``wait_all``."""
        total = self.grad_sq.clone()
        self.grad_sq.zero_()
        dist.all_reduce(total, group=self.group)
        return total

    # ------------------------------------------------------------------ all-gather
    def all_gather_inplace(self, t: Tensor, chunk_rows: int):
        """``t`` ([world * chunk_rows, ...], from ``symm_zeros``): rank r's rows [r*chunk, (r+1)*chunk) are valid on entry."""
        hdl, off = self._handle_of(t)
        chunk_bytes = chunk_rows * t[0].numel() * t.element_size()
        assert chunk_bytes % 16 == 0 and off % 16 == 0
        ops.ext().comm_allgather([int(p) for p in hdl.buffer_ptrs], self.flag_ptrs_main, off, chunk_bytes, self.rank, self.seq_main,
                                 self.blocks, self.status)
        ops._count()
        self.seq_main += 2

    def peer_addresses(self, t: Tensor) -> list[int]:
        """Addresses of the other ranks' copies of ``t`` (a view of a ``symm_zeros`` buffer)."""
        hdl, off = self._handle_of(t)
        return [int(p) + off for r, p in enumerate(hdl.buffer_ptrs) if r != self.rank]

    def all_addresses(self, t: Tensor) -> list[int]:
        """Addresses of every rank's copy of ``t`` (a view of a ``symm_zeros`` buffer), in rank order, this rank's included."""
        hdl, off = self._handle_of(t)
        return [int(p) + off for p in hdl.buffer_ptrs]

    def barrier(self):
        """Device-side barrier across ranks on the current stream (a zero-byte all-gather)."""
        ops.ext().comm_allgather(self.flag_ptrs_main, self.flag_ptrs_main, 0, 0, self.rank, self.seq_main, 1, self.status)
        ops._count()
        self.seq_main += 2

    def check(self):
        """Host read (synchronises): raises when a kernel gave up waiting for a peer."""
        code = int(self.status.item())
        if code != 0:
            raise CommTimeout(f"rank {self.rank}: a comm kernel gave up waiting (code {code}: peer {code - 1000})")
