"""Muon, NorMuon and NorMuon with cautious weight decay, batched per matrix shape and shardable.

Update rules per matrix ``p [rows, cols]`` with (reduced) gradient ``g``, momentum ``mu``:
  buf <- buf + (1 - mu)(g - buf);  g~ = g + mu (buf - g);  v = NewtonSchulz(bf16(g~))
  Muon     (training/optimizers/muon.py:39-66):      p <- p (1 - lr wd);  p <- p - eff_lr v
  NorMuon  (training/optimizers/normuon.py:13-27,60-110): neuron-wise second-moment normalisation of v
           that keeps its Frobenius norm, then p <- p - eff_lr v   (no weight decay is applied)
  NorMuonCWD (training/optimizers/normuon_cwd.py:13-31,67-113): NorMuon, and before the update
           p <- p - lr wd p [sign(v) == sign(p)]
with ``eff_lr = lr * sqrt(max(1, rows/cols)) * p.lr_mul``.  State keys (``momentum_buffer``,
``second_momentum_buffer``), parameter groups (one per distinct shape, in Python-set order) and the
return value (``sqrt(sum ||v||_F^2) / n``) are those of the reference, so its checkpoints load.

What is different is the execution: all matrices of one shape are processed as a batch
(``[n, rows, cols]``): one momentum update, one batched Newton-Schulz chain, one batched tail.  The
reference loops over 150 matrices and runs the full step on every rank.  With ``shard=True`` and an
initialised process group each matrix has one owner rank that runs momentum + Newton-Schulz; the
orthogonalised updates are all-gathered (bf16) and every rank applies the cheap tail.  Momentum
buffers are then live only on the owner; ``consolidate_state()`` gathers them before a checkpoint.
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor

from sample_efficient_gpt_b200.optim.newton_schulz import newton_schulz
from sample_efficient_gpt_b200.utils.profiling import nvtx_range


class _ShapeBatch:
    """Stacked state for the matrices of one shape.

    ``momentum`` is ``[slots, rows, cols]`` fp32 where ``slots = world * chunk`` (``chunk`` matrices per
    rank, the tail padded); matrix i sits in slot ``owner(i) * chunk + i % chunk``.  The per-parameter
    optimizer-state entries are views into these tensors.
    """

    def __init__(self, params: list[Tensor], group_index: int, world: int, rank: int, symm_alloc=None):
        self.params = params
        n = len(params)
        self.n = n
        self.world, self.rank = world, rank
        self.chunk = math.ceil(n / world)
        self.slots = self.chunk * world
        self.rot = group_index % world
        rows, cols = params[0].shape[-2:]
        self.rows, self.cols = rows, cols
        self.slot_of = [self._slot(i) for i in range(n)]
        self.owned = [i for i in range(n) if self.owner(i) == rank]
        dev = params[0].device
        self.momentum = torch.zeros((self.slots, rows, cols), dtype=torch.float32, device=dev)
        sm_shape = (n, rows, 1) if rows >= cols else (n, 1, cols)
        self.second = torch.zeros(sm_shape, dtype=torch.float32, device=dev)
        if symm_alloc is not None:  # peer-mapped, so that the all-gather kernel can read it from other ranks
            self.update = symm_alloc((self.slots, rows, cols), torch.bfloat16)
        else:
            self.update = torch.zeros((self.slots, rows, cols), dtype=torch.bfloat16, device=dev)
        # CUDA fast path: second ping-pong buffer of the Newton-Schulz chain and slot index tables
        self.xbuf = torch.zeros_like(self.update) if dev.type == "cuda" else None
        if dev.type == "cuda":
            self.slot_all = torch.tensor(self.slot_of, dtype=torch.int32, device=dev)
            self.slot_owned = torch.tensor([self.slot_of[i] for i in self.owned], dtype=torch.int32, device=dev)

    def owner(self, i: int) -> int:
        return (i // self.chunk + self.rot) % self.world

    def _slot(self, i: int) -> int:
        return self.owner(i) * self.chunk + i % self.chunk


class Muon(torch.optim.Optimizer):
    _normalize = False
    _cautious = False
    _plain_decay = True

    def __init__(self, params, lr=0.02, weight_decay=0.01, momentum=0.95, beta2=0.95, shard: bool = False):
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum, beta2=beta2)
        params = list(params)
        sizes = {p.shape for p in params}
        param_groups = [dict(params=[p for p in params if p.shape == size]) for size in sizes]
        super().__init__(param_groups, defaults)
        self.shard = shard
        self.is_distributed = bool(shard and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1)
        self.world = dist.get_world_size() if self.is_distributed else 1
        self.rank = dist.get_rank() if self.is_distributed else 0
        self._batches: dict[int, _ShapeBatch] = {}
        self.lowp_shadows: dict[Tensor, Tensor] = {}  # param -> bf16 copy refreshed after the update
        self.comm = None  # optional parallel.symm communicator providing a fused all-gather

    # ------------------------------------------------------------------ state plumbing
    def _batch(self, gi: int) -> _ShapeBatch:
        b = self._batches.get(gi)
        if b is None:
            ps = self.param_groups[gi]["params"]
            alloc = self.comm.symm_zeros if (self.comm is not None and self.is_distributed) else None
            b = _ShapeBatch(ps, gi, self.world, self.rank, alloc)
            self._batches[gi] = b
            self._bind_state(b)
        return b

    def _bind_state(self, b: _ShapeBatch, source: dict | None = None):
        """Point ``self.state[p]`` at views of the stacked tensors (copying ``source`` values in first)."""
        for i, p in enumerate(b.params):
            st = self.state[p]
            slot = b.slot_of[i]
            if "momentum_buffer" in st and st["momentum_buffer"].data_ptr() != b.momentum[slot].data_ptr():
                b.momentum[slot].copy_(st["momentum_buffer"])
            st["momentum_buffer"] = b.momentum[slot]
            if self._normalize:
                if (
                    "second_momentum_buffer" in st
                    and st["second_momentum_buffer"].data_ptr() != b.second[i].data_ptr()
                ):
                    b.second[i].copy_(st["second_momentum_buffer"])
                st["second_momentum_buffer"] = b.second[i]

    def state_dict(self):
        sd = super().state_dict()
        # The per-parameter dicts returned by torch are the live ones: build copies instead of editing them, and
        # clone views so that a file does not drag the whole stacked storage along.
        sd["state"] = {
            k: {kk: (vv.clone() if torch.is_tensor(vv) and vv._base is not None else vv) for kk, vv in st.items()}
            for k, st in sd["state"].items()
        }
        return sd

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        self._batches.clear()
        for gi in range(len(self.param_groups)):
            if any(len(self.state[p]) for p in self.param_groups[gi]["params"]):
                self._batch(gi)

    @torch.no_grad()
    def consolidate_state(self):
        """Sharded mode: bring every owner's momentum buffers to all ranks (call on all ranks before saving)."""
        if not self.is_distributed:
            return
        for b in self._batches.values():
            mine = b.momentum[self.rank * b.chunk : (self.rank + 1) * b.chunk].contiguous()
            dist.all_gather_into_tensor(b.momentum.view(-1), mine.view(-1))

    # ------------------------------------------------------------------ the step
    @nvtx_range("muon step")
    @torch.no_grad()
    def step(self, closure: Any | None = None):
        if closure is not None:
            closure()
        device = self.param_groups[0]["params"][0].device
        sq_sum = torch.zeros((), dtype=torch.float32, device=device)
        n_total = 0
        for gi, group in enumerate(self.param_groups):
            ps = group["params"]
            if any(p.grad is None for p in ps):
                if all(p.grad is None for p in ps):
                    continue
                raise RuntimeError("Muon: either all or none of the matrices of one shape must have a gradient")
            b = self._batch(gi)
            if self._fused_ok(b):
                sq_sum += self._step_fused(b, group)
            else:
                v = self._orthogonalized_updates(b, group)  # [n, rows, cols] fp32, identical on all ranks
                sq_sum += self._apply(b, group, v)
            n_total += b.n
        return sq_sum.sqrt() / (n_total + 1e-10)

    def _fused_ok(self, b: _ShapeBatch) -> bool:
        from sample_efficient_gpt_b200 import ops

        p0 = b.params[0]
        if not (p0.is_cuda and p0.dtype == torch.float32 and ops.has_kernel("muon_tail") and ops.kernel_enabled("muon_fused")):
            return False
        if b.cols % 8 != 0 or (b.rows * b.cols) % 8 != 0:
            return False
        muls = {(getattr(p, "lr_mul", 1.0), getattr(p, "wd_mul", 1.0)) for p in b.params}
        return len(muls) == 1 and all(p.is_contiguous() and p.grad is not None and p.grad.is_contiguous() for p in b.params)

    def _step_fused(self, b: _ShapeBatch, group) -> Tensor:
        """CUDA path: 2 launches for momentum + normalisation, the GEMM chain, 3 launches for the tail."""
        from sample_efficient_gpt_b200 import ops
        from sample_efficient_gpt_b200.ops.newton_schulz import ns_iterations
        from sample_efficient_gpt_b200.optim.newton_schulz import POLAR_EXPRESS_COEFFS

        ext = ops.ext()
        idx = b.owned if self.is_distributed else list(range(b.n))
        if idx:
            ext.muon_momentum([b.params[i].grad for i in idx], b.slot_owned if self.is_distributed else b.slot_all,
                              b.momentum, b.xbuf, group["momentum"], 1e-7)
            ops._count(2)
            s0 = b.slot_of[idx[0]]
            dst = b.update[s0 : s0 + len(idx)]
            push = None
            if self.is_distributed and self.comm is not None and hasattr(self.comm, "peer_addresses"):
                # the last Newton-Schulz GEMM stores its tiles into every rank's update buffer
                push = lambda buf: self.comm.peer_addresses(buf) if buf.data_ptr() == dst.data_ptr() else None  # noqa: E731
            res = ns_iterations(b.xbuf[s0 : s0 + len(idx)], dst, POLAR_EXPRESS_COEFFS, final_extra_dst=push)
            pushed = isinstance(res, tuple)
            res = res[0] if pushed else res
            if res.data_ptr() != dst.data_ptr():
                dst.copy_(res)
        else:
            pushed = self.is_distributed and self.comm is not None and hasattr(self.comm, "peer_addresses")
        if self.is_distributed:
            if pushed and self._all_ranks_push(b):
                self.comm.barrier()  # every rank's tiles have landed everywhere
            else:
                self._gather_updates(b)
        lr, wd = group["lr"], group["weight_decay"]
        lr_mul, wd_mul = getattr(b.params[0], "lr_mul", 1.0), getattr(b.params[0], "wd_mul", 1.0)
        mode = 1 if self._plain_decay else (2 if self._cautious else 0)
        sq = torch.zeros((), dtype=torch.float32, device=b.update.device)
        shadows = [self.lowp_shadows.get(p) for p in b.params]
        shadows = shadows if all(s is not None for s in shadows) else []
        ext.muon_tail(b.update, b.slot_all, b.second, list(b.params), shadows, sq, b.rows, b.cols, group["beta2"],
                      self._normalize, lr * max(1.0, b.rows / b.cols) ** 0.5 * lr_mul, lr * wd * wd_mul, mode)
        ops._count(3)
        if not shadows:
            for p in b.params:
                sh = self.lowp_shadows.get(p)
                if sh is not None:
                    sh.copy_(p)
        return sq

    def _all_ranks_push(self, b: _ShapeBatch) -> bool:
        """The in-epilogue all-gather is used only when every rank takes it for this shape (same decision everywhere)."""
        r = min(b.rows, b.cols)
        return r % 8 == 0 and max(b.rows, b.cols) % 8 == 0 and all(
            any(b.owner(i) == rk for i in range(b.n)) for rk in range(self.world)
        )

    def _gather_updates(self, b: _ShapeBatch):
        if self.comm is not None:
            self.comm.all_gather_inplace(b.update, b.chunk)
        else:
            mine = b.update[self.rank * b.chunk : (self.rank + 1) * b.chunk].contiguous()
            dist.all_gather_into_tensor(b.update.view(-1), mine.view(-1))

    def _orthogonalized_updates(self, b: _ShapeBatch, group) -> Tensor:
        mu = group["momentum"]
        idx = b.owned if self.is_distributed else list(range(b.n))
        if idx:
            g = torch.stack([b.params[i].grad for i in idx]).float()
            slots = [b.slot_of[i] for i in idx]
            contiguous = slots == list(range(slots[0], slots[0] + len(slots)))
            m = b.momentum[slots[0] : slots[0] + len(slots)] if contiguous else b.momentum[slots]
            m.lerp_(g, 1 - mu)
            if not contiguous:
                b.momentum[slots] = m
            g.lerp_(m, mu)
            x = newton_schulz(g.bfloat16())
            if contiguous:
                b.update[slots[0] : slots[0] + len(slots)].copy_(x)
            else:
                b.update[slots] = x
        if self.is_distributed:
            self._gather_updates(b)
        if b.slot_of == list(range(b.n)):
            return b.update[: b.n].float()
        return b.update[b.slot_of].float()

    def _apply(self, b: _ShapeBatch, group, v: Tensor) -> Tensor:
        lr, wd = group["lr"], group["weight_decay"]
        ps = b.params
        mup = max(1.0, b.rows / b.cols) ** 0.5
        v_norm = v.norm(dim=(-2, -1), keepdim=True)
        if self._normalize:
            dim = -1 if b.rows >= b.cols else -2
            v_mean = v.square().mean(dim=dim, keepdim=True)
            b.second.lerp_(v_mean, 1 - group["beta2"])
            v = v * torch.rsqrt(b.second.clamp_min(1e-10))
            v = v * (v_norm / v.norm(dim=(-2, -1), keepdim=True).clamp_min(1e-10))
        vs = list(v.unbind(0))
        lr_muls = [getattr(p, "lr_mul", 1.0) for p in ps]
        wd_muls = [getattr(p, "wd_mul", 1.0) for p in ps]
        if self._plain_decay:
            torch._foreach_mul_(ps, [1 - lr * wd * w for w in wd_muls])
        elif self._cautious:
            masks = [torch.eq(torch.signbit(vi), torch.signbit(p)).to(p.dtype) for vi, p in zip(vs, ps)]
            decay = torch._foreach_mul(ps, masks)
            torch._foreach_mul_(decay, [-lr * wd * w for w in wd_muls])
            torch._foreach_add_(ps, decay)
        torch._foreach_mul_(vs, [-lr * mup * m for m in lr_muls])
        torch._foreach_add_(ps, vs)
        for p in ps:
            sh = self.lowp_shadows.get(p)
            if sh is not None:
                sh.copy_(p)
        return v_norm.square().sum()


class NorMuon(Muon):
    """Muon + neuron-wise normalisation; weight decay is accepted but never applied (as in the reference)."""

    _normalize = True
    _cautious = False
    _plain_decay = False


class NorMuonCWD(NorMuon):
    """NorMuon with cautious (sign-agreeing) decoupled weight decay: the optimizer IMU-1 was trained with."""

    _cautious = True
