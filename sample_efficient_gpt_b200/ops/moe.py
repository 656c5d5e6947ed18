"""Mixture-of-experts primitives for the hand-scheduled engine: routing, slot assignment, the expert-parallel exchange
and the router backward.  CUDA tensors run this package's kernels (csrc/moe.cu); everything else runs the PyTorch
statements below, which are also the oracle of the kernel tests.  Specification: models/moe.py.

Layout of an exchange buffer on its owner rank: ``[E_local, world, cap, d]`` - expert, source rank, slot.
Exchanges:
  * ``TorchExchange``  - index ops + ``all_to_all_single`` (gloo on CPU, NCCL on GPUs): baseline and CPU path.
  * ``PeerExchange``   - dispatch = permutation fused with peer *stores* into the owners' symmetric buffers (the consumer
    GEMM waits per source rank on arrival flags); combine = the down-projection GEMM's epilogue stores its tiles straight
    into the source ranks' landing buffers (routed output), then a local un-permutation + weighted sum.  Without the
    overlapped mode: barrier-ordered push, and a pull (peer *loads*) for the combine.  With one rank it degenerates to
    local buffers and no barrier.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch import Tensor

from sample_efficient_gpt_b200 import ops


def capacity(n_tokens: int, top_k: int, n_experts: int, factor: float) -> int:
    return max(1, math.ceil(factor * n_tokens * top_k / n_experts))


def _cuda_ok(x: Tensor) -> bool:
    return x.is_cuda and ops.has_kernel("moe_route") and ops.kernel_enabled("moe")


# ---------------------------------------------------------------------------------------------------- routing
def route(x: Tensor, wr: Tensor, top_k: int, cap: int):
    """x [T,d], wr [E,d] fp32 -> probs [T,E] fp32, idx [T,k] int32, w [T,k] fp32, slot [T,k] int32 (-1 = dropped),
    totals [E] int32 (assignments per expert before dropping)."""
    if _cuda_ok(x) and x.dtype == torch.bfloat16:
        ops._count(3)
        probs, idx, w, off, totals = ops.ext().moe_route(x.contiguous(), wr.detach().float().contiguous(), top_k)
        return probs, idx, w, ops.ext().moe_slots(idx, off, cap), totals
    E = wr.size(0)
    probs = (x.float() @ wr.detach().float().t()).softmax(-1)
    w, idx = probs.topk(top_k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    flat = idx.reshape(-1)
    onehot = torch.nn.functional.one_hot(flat, E)
    pos = (onehot.cumsum(0) - 1).gather(1, flat[:, None]).squeeze(1).reshape(idx.shape)
    slot = torch.where(pos < cap, pos, torch.full_like(pos, -1))
    return probs, idx.int(), w, slot.int(), onehot.sum(0).int()


def route_bwd(probs: Tensor, idx: Tensor, dw: Tensor, aux_vec: Tensor) -> Tensor:
    """d(logits) [T,E] given d(renormalised weights) [T,k] and a per-expert additive term on d(probs)."""
    if _cuda_ok(probs):
        ops._count()
        return ops.ext().moe_route_bwd(probs, idx, dw.contiguous(), aux_vec.float().contiguous())
    li = idx.long()
    raw = probs.gather(1, li)
    s = raw.sum(-1, keepdim=True)
    wn = raw / s
    draw = (dw - (dw * wn).sum(-1, keepdim=True)) / s
    dp = aux_vec.float()[None, :].expand_as(probs).clone()
    dp.scatter_add_(1, li, draw)
    return probs * (dp - (dp * probs).sum(-1, keepdim=True))


# ---------------------------------------------------------------------------------------------------- exchange
class TorchExchange:
    """Exchange with index ops and (for more than one rank) ``all_to_all_single``."""

    def __init__(self, n_experts: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.n_experts, self.e_local = n_experts, n_experts // self.world

    def begin_step(self):
        pass

    def expert_output(self, key, shape, dtype, device):
        """(tensor the expert GEMM must write into or None for a fresh one, routing of its output or None)."""
        return None, None

    def _a2a(self, t: Tensor) -> Tensor:
        if self.world == 1:
            return t
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t.contiguous(), group=self.group)
        return out

    def dispatch(self, key, x: Tensor, idx: Tensor, slot: Tensor, totals: Tensor, w: Tensor | None, cap: int) -> Tensor:
        T, d = x.shape
        k, E = idx.size(1), self.n_experts
        keep = (slot >= 0).reshape(-1)
        tok = torch.arange(T, device=x.device).repeat_interleave(k)
        rows = x[tok]
        if w is not None:
            rows = (rows.float() * w.reshape(-1, 1)).to(x.dtype)
        flat = (idx.long() * cap + slot.long().clamp(min=0)).reshape(-1)
        buf = x.new_zeros(E * cap, d)
        buf.index_copy_(0, flat[keep], rows[keep])
        recv = self._a2a(buf.view(self.world, self.e_local, cap, d))  # [src, e_local, cap, d]
        return recv.permute(1, 0, 2, 3).reshape(self.e_local, self.world * cap, d).contiguous(), None

    def collect(self, key, buf: Tensor, idx: Tensor, slot: Tensor, w: Tensor | None, cap: int, out_dtype, dot_key=None,
                dot_buf: Tensor | None = None, g: Tensor | None = None):
        d = buf.size(-1)
        T, k = idx.shape

        def back(b):
            send = b.view(self.e_local, self.world, cap, d).permute(1, 0, 2, 3).contiguous()  # [dst, e_local, cap, d]
            return self._a2a(send).reshape(self.n_experts * cap, d)

        keep = (slot >= 0).reshape(-1, 1)
        flat = (idx.long() * cap + slot.long().clamp(min=0)).reshape(-1)
        rows = back(buf)[flat].float() * keep
        dots = None
        if dot_buf is not None:
            rows2 = back(dot_buf)[flat].float() * keep
            dots = (rows2.view(T, k, d) * g.float()[:, None, :]).sum(-1)
        if w is not None:
            rows = rows * w.reshape(-1, 1)
        out = rows.view(T, k, d).sum(1).to(out_dtype)
        return out, dots


class PeerExchange:
    """Exchange over symmetric memory with this package's push / pull kernels (bf16 CUDA tensors only)."""

    def __init__(self, n_experts: int, comm=None, device=None, overlap: bool | None = None):
        """``overlap``: instead of a barrier between the push and the first expert GEMM, the push signals per-destination
        flags and the GEMM's producer waits per source region, so an expert's tiles start as soon as their rows are in
        (default: on when there is more than one rank; ``SEGPT_MOE_OVERLAP=0`` switches it off)."""
        import os

        self.comm = comm
        self.world = comm.world if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.n_experts, self.e_local = n_experts, n_experts // self.world
        self.device = torch.device(device) if device is not None else (comm.device if comm is not None else torch.device("cuda"))
        self._bufs: dict = {}
        if overlap is None:
            overlap = os.environ.get("SEGPT_MOE_OVERLAP", "1") == "1"
        self.overlap = bool(overlap and comm is not None and self.world > 1)
        if self.overlap:
            self.flags = comm.symm_zeros((64,), torch.int32)  # flags[src]: last dispatch of rank src that has fully landed
            self.flag_ptrs = comm.all_addresses(self.flags)
            self.done = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.seq = 0

    def begin_step(self):
        """Nobody may push into this step's buffers before every rank is done with the previous step's."""
        if self.comm is not None:
            self.comm.barrier()

    def _buffer(self, key, cap: int, d: int) -> Tensor:
        t = self._bufs.get(key)
        if t is None or t.shape != (self.e_local, self.world, cap, d):
            shape = (self.e_local, self.world, cap, d)
            if self.comm is not None:
                t = self.comm.symm_zeros(shape, torch.bfloat16)  # zero-initialised: rows nobody wrote stay finite
            else:
                t = torch.zeros(shape, dtype=torch.bfloat16, device=self.device)
            self._bufs[key] = t
        return t

    def _addresses(self, t: Tensor) -> list[int]:
        return self.comm.all_addresses(t) if self.comm is not None else [t.data_ptr()]

    def _recv(self, key, cap: int, d: int) -> Tensor:
        """This rank's landing buffer [E, cap, d] for expert outputs that the owners' GEMMs store straight into it."""
        t = self._bufs.get(("recv", key))
        if t is None or t.shape != (self.n_experts, cap, d):
            t = self.comm.symm_zeros((self.n_experts, cap, d), torch.bfloat16)
            self._bufs[("recv", key)] = t
        return t

    def expert_output(self, key, shape, dtype, device):
        """Overlapped mode: the expert GEMM's epilogue stores every tile into the *source* rank's landing buffer (routed
        output), so the combine exchange runs inside the GEMM.  Otherwise: a symmetric buffer on this rank for the pull."""
        e_local, rows, d = shape
        cap = rows // self.world
        if self.overlap:
            recv = self._recv(key, cap, d)
            return None, (self.comm.all_addresses(recv), cap, cap * d, self.rank * self.e_local * cap * d, d)
        return self._buffer(key, cap, d).view(e_local, rows, d), None

    def dispatch(self, key, x: Tensor, idx: Tensor, slot: Tensor, totals: Tensor, w: Tensor | None, cap: int) -> Tensor:
        buf = self._buffer(key, cap, x.size(1))
        ops._count()
        view = buf.view(self.e_local, self.world * cap, x.size(1))
        if self.overlap:
            self.seq += 1
            ops.ext().moe_push(x.contiguous(), idx, slot, w, totals, self._addresses(buf), cap, self.rank, self.flag_ptrs, self.done, self.seq)
            return view, (self.flags, self.seq, cap)  # the consumer GEMM waits per source region
        ops.ext().moe_push(x.contiguous(), idx, slot, w, totals, self._addresses(buf), cap, self.rank)
        if self.comm is not None:
            self.comm.barrier()  # every rank's rows have landed before anybody's GEMMs read them
        return view, None

    def collect(self, key, buf: Tensor | None, idx: Tensor, slot: Tensor, w: Tensor | None, cap: int, out_dtype, dot_key=None,
                dot_buf: Tensor | None = None, g: Tensor | None = None):
        """``key`` / ``dot_key`` name the buffers in the overlapped mode (the rows are already here, in landing buffers);
        ``buf`` / ``dot_buf`` are the owner-side buffers of the pull mode."""
        if self.comm is not None:
            self.comm.barrier()  # every owner's output rows are written before anybody reads them
        ops._count()
        want_dots = dot_key is not None or dot_buf is not None
        gg = g.contiguous() if g is not None else None
        if self.overlap:
            d = self._bufs[("recv", key)].size(-1)
            src = [self._bufs[("recv", key)].data_ptr()]  # one local buffer [E, cap, d]: "world 1, rank 0" addressing
            src2 = [self._bufs[("recv", dot_key)].data_ptr()] if want_dots else []
            res = ops.ext().moe_pull(src, src2, idx, slot, w, gg, d, self.n_experts, cap, 0, out_dtype == torch.float32)
        else:
            res = ops.ext().moe_pull(self._addresses(buf), self._addresses(dot_buf) if want_dots else [], idx, slot, w, gg,
                                     buf.size(-1), self.n_experts, cap, self.rank, out_dtype == torch.float32)
        return res[0], (res[1] if want_dots else None)
