"""Hand-scheduled forward + backward of the dense transformer (no autograd graph).

One call to ``forward_backward`` runs the whole training micro-step as an explicit sequence of
kernels: per block ``add+RMSNorm -> qkv GEMM -> RoPE/QK-norm/value-mix -> flash attention -> gate ->
out GEMM -> add+RMSNorm -> up GEMM -> SwiGLU -> down GEMM``, then the final norm and the fused
head-projection + cross-entropy (logits never stored), then the mirrored backward that writes
parameter gradients straight into persistent fp32 buffers (``p.grad``).  Activations are bf16, the
residual stream and all statistics fp32, weights are read from persistent bf16 shadows of the fp32
masters that the optimizers refresh.  As soon as a block's gradients are final the engine calls
``grad_ready(params)`` so that the data-parallel layer can start that bucket's reduction while the
backward of earlier blocks is still running.  Blocks below ``num_grad_checkpoint_layers`` keep only
their fp32 input and are recomputed in the backward sweep.

The same schedule runs on CPU tensors through the PyTorch statements of each op, which is how the
hand-derived backward is checked against autograd of the module path (models/transformer.py).
Semantics follow the reference model (transformer/transformer.py:47-139, attention.py:176-267).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
from torch import Tensor

from sample_efficient_gpt_b200 import ops
from sample_efficient_gpt_b200.models.transformer import Transformer
from sample_efficient_gpt_b200.training.loss import IGNORE_INDEX, LSE_SQUARE_SCALE, NATS_TO_BITS
from sample_efficient_gpt_b200.utils.profiling import nvtx_range


@dataclass
class StepOutput:
    loss: Tensor  # mean per-token loss (includes the 1e-6 * lse^2 term)
    z_loss: Tensor
    loss_bpb: Tensor | None
    kurtosis: Tensor  # [n_layers]
    loss_tok: Tensor | None = None
    aux_loss: Tensor | None = None  # sum of the load-balance terms of the mixture-of-experts blocks


def engine_supports(model: Transformer) -> bool:
    blk = model.blocks[0]
    uniform = all(b.is_moe == blk.is_moe for b in model.blocks)
    return uniform and blk.attn.gating in (False, "per-head")


class FusedEngine:
    def __init__(self, model: Transformer, act_dtype: torch.dtype = torch.bfloat16, moe_exchange=None, fuse_gate: bool | None = None):
        if not engine_supports(model):
            raise ValueError("FusedEngine: gating in {False, 'per-head'} and either all-dense or all-MoE blocks only")
        self.model = model
        self.lp = act_dtype
        self.grad_ready: Callable[[list[torch.nn.Parameter]], None] | None = None
        self.shadows: dict[Tensor, Tensor] = {}
        self._matrix_params = [p for n, p in model.named_parameters() if p.ndim == 2 and "embedding" not in n]
        for p in self._matrix_params:
            self.shadows[p] = p.detach().to(act_dtype) if act_dtype != p.dtype else p.detach()
        self._first_accum = True
        # the per-layer LayerNorm scaling factors live in device buffers of the model: read them once, not with a
        # device-to-host copy (and a stalled launch queue) in every block of every pass
        self._ln_scale = [float(b.ln1.position_scale) for b in model.blocks]
        self._final_scale = float(model.final_norm.position_scale)
        at = model.blocks[0].attn
        self.H, self.Hkv, self.hd = at.n_heads, at.n_kv_heads, at.head_dim
        self._ones = torch.ones(1, dtype=torch.float32, device=model.embedding.weight.device)
        self._loss_coef = 1.0
        # The per-head gate projection ([d] -> [H], e.g. 1152 -> 18) is far too narrow for a GEMM of its own: its weight
        # rows are appended to the qkv weight (in the low-precision shadow, padded to a multiple of 8 rows), so that the
        # gate logits, their data gradient and their weight gradient ride along with the qkv GEMMs.
        self.fuse_gate = (act_dtype != torch.float32) if fuse_gate is None else fuse_gate
        self.qkvz_w: dict[int, Tensor] = {}
        self._wg_tmp: Tensor | None = None
        if self.fuse_gate and at.gating == "per-head":
            for i, blk in enumerate(model.blocks):
                wq, wg = blk.attn.qkv.linear.weight, blk.attn.attn_gate.linear.weight
                n_qkv, H = wq.size(0), wg.size(0)
                n_ext = (n_qkv + H + 7) // 8 * 8
                cat = torch.zeros((n_ext, wq.size(1)), dtype=act_dtype, device=wq.device)
                cat[:n_qkv].copy_(wq.detach())
                cat[n_qkv : n_qkv + H].copy_(wg.detach())
                self.qkvz_w[i] = cat
                self.shadows[wq], self.shadows[wg] = cat[:n_qkv], cat[n_qkv : n_qkv + H]
        self.moe = None
        if model.blocks[0].is_moe:
            from sample_efficient_gpt_b200.training.moe_engine import MoEEngine

            self.moe = MoEEngine(self, moe_exchange)

    # ------------------------------------------------------------------ helpers
    def refresh_shadows(self):
        """Re-cast every GEMM weight from its fp32 master (after a load or an external update).  In fp32 runs most shadows
        are the masters themselves; the stacked expert weights are copies in every precision."""
        ps = [p for p in self.shadows if self.shadows[p].data_ptr() != p.data_ptr()]
        if ps:
            torch._foreach_copy_([self.shadows[p] for p in ps], [p.detach() for p in ps])
        if self.moe is not None:
            self.moe.refresh()

    def register_with(self, optimizers):
        """Let the optimizers write the shadows (bf16 copies; in fp32 runs only the stacked expert weights are copies) in the
        same kernel that updates the masters."""
        for opt in optimizers:
            if hasattr(opt, "lowp_shadows"):
                for g in opt.param_groups:
                    for p in g["params"]:
                        if p in self.shadows and self.shadows[p].data_ptr() != p.data_ptr():
                            opt.lowp_shadows[p] = self.shadows[p]

    def ensure_grads(self):
        """fp32 gradients for every parameter.  When none exists yet (single-process runs; DDP installs its own views before)
        they are carved out of one flat buffer, 256-byte aligned, so that the global gradient norm is one reduction
        (``flat_grads``) instead of one per tensor."""
        params = [p for p in self.model.parameters() if p.requires_grad]
        if params and all(p.grad is None for p in params) and getattr(self, "flat_grads", None) is None:
            offs, total = [], 0
            for p in params:
                offs.append(total)
                total += (p.numel() + 63) // 64 * 64
            self.flat_grads = torch.zeros(total, dtype=torch.float32, device=params[0].device)
            self._flat_views = {}
            for p, o in zip(params, offs):
                p.grad = self._flat_views[p] = self.flat_grads[o : o + p.numel()].view_as(p)
            return
        for p in params:
            if p.grad is None:
                p.grad = torch.zeros_like(p, dtype=torch.float32)

    def flat_grad_norm(self) -> Tensor | None:
        """Global gradient norm from the flat buffer; None when some gradient no longer lives there."""
        flat, views = getattr(self, "flat_grads", None), getattr(self, "_flat_views", None)
        if flat is None or any(p.grad is not v for p, v in views.items()):
            return None
        return torch.linalg.vector_norm(flat)

    def _dqkvz_buffer(self, T: int, n_ext: int, like: Tensor) -> Tensor:
        """Gradient buffer of the fused qkv+gate projection, shared by all blocks (the kernels of a step run in stream order);
        its padding columns are zeroed once, at allocation, and never written afterwards."""
        buf = getattr(self, "_dqkvz", None)
        if buf is None or buf.shape != (T, n_ext) or buf.dtype != like.dtype or buf.device != like.device:
            buf = self._dqkvz = torch.zeros((T, n_ext), dtype=like.dtype, device=like.device)
        return buf

    def _w(self, p: Tensor) -> Tensor:
        return self.shadows[p]

    def _acc(self, p: torch.nn.Parameter, value: Tensor):
        if self._first_accum:
            p.grad.copy_(value.reshape(p.grad.shape))
        else:
            p.grad.add_(value.reshape(p.grad.shape))

    def _wgrad(self, p: torch.nn.Parameter, dy: Tensor, x: Tensor):
        ops.wgrad_accumulate(p.grad, dy, x, self._first_accum)

    # ------------------------------------------------------------------ one block
    def _layer_fwd(self, i: int, res: Tensor, delta: Tensor | None, v1: Tensor | None, B: int, S: int, want_kurt=True, train=True):
        blk = self.model.blocks[i]
        at = blk.attn
        H, Hkv, hd = self.H, self.Hkv, self.hd
        T = B * S
        scale = self._ln_scale[i]
        x, n1, rstd1, kurt = ops.add_rmsnorm_fwd(res, delta, blk.ln1.gain, scale, blk.ln1.eps, self.lp, want_kurt)
        if i in self.qkvz_w:
            n_qkv = at.qkv.linear.weight.size(0)
            qkvz = ops.matmul_nt(n1, self.qkvz_w[i])
            qkv, z = qkvz[:, :n_qkv], qkvz[:, n_qkv : n_qkv + H]  # column views: the kernels take the row stride
        else:
            qkv = ops.matmul_nt(n1, self._w(at.qkv.linear.weight))
            z = ops.matmul_nt(n1, self._w(at.attn_gate.linear.weight)) if at.gating else None
        qgain = at.sdpa_qknorm.gain if at.qknorm else self._ones
        q, k, v = ops.qkv_post_fwd(
            qkv, v1, at.rope.cos, at.rope.sin, qgain, at.alpha1, at.alpha2, at.scale, B, S, H, Hkv, hd, at.qknorm
        )
        o, lse = ops.attention_fwd(q, k, v, True, 0, for_backward=train)
        g = ops.gate_fwd(o.view(T, H, hd), z) if at.gating else o.view(T, H * hd)
        a = ops.matmul_nt(g, self._w(at.out.linear.weight))
        y, n2, rstd2, _ = ops.add_rmsnorm_fwd(x, a, blk.ln2.gain, scale, blk.ln2.eps, self.lp, False)
        if blk.is_moe:
            m, u = self.moe.forward(i, n2, train, record=want_kurt or not train)  # u: what the expert backward needs
            f = None
        else:
            u, f = ops.up_swiglu(n2, self._w(blk.ffn.up.linear.weight))
            m = ops.matmul_nt(f, self._w(blk.ffn.down.linear.weight))
        saved = (x, n1, rstd1, qkv, z, q, k, v, o, lse, g, y, n2, rstd2, u, f)
        return y, m, v, kurt, saved

    def _layer_bwd(self, i, saved, v1, dres, dres_lp, dv1_acc, B, S):
        blk = self.model.blocks[i]
        at = blk.attn
        H, Hkv, hd = self.H, self.Hkv, self.hd
        T = B * S
        x, n1, rstd1, qkv, z, q, k, v, o, lse, g, y, n2, rstd2, u, f = saved
        scale = self._ln_scale[i]
        w_out, w_qkv = at.out.linear.weight, at.qkv.linear.weight

        if blk.is_moe:
            dn2 = self.moe.backward(i, dres_lp, n2, u, self._loss_coef, self._first_accum)
        else:
            w_down, w_up = blk.ffn.down.linear.weight, blk.ffn.up.linear.weight
            du = ops.down_dgrad_swiglu(dres_lp, self._w(w_down), u)
            self._wgrad(w_down, dres_lp, f)
            dn2 = ops.matmul_nn(du, self._w(w_up))
            self._wgrad(w_up, du, n2)
        dy, dy_lp, dgain2 = ops.add_rmsnorm_bwd(dn2, dres, y, blk.ln2.gain, rstd2, scale, self.lp)
        self._acc(blk.ln2.gain, dgain2)

        dg = ops.matmul_nn(dy_lp, self._w(w_out))
        self._wgrad(w_out, dy_lp, g)
        fused = i in self.qkvz_w
        dqkvz = None
        if fused:  # [dqkv | dz | zero padding], the layout of the fused projection's output; both kernels write into it
            n_qkv, n_ext = w_qkv.size(0), self.qkvz_w[i].size(0)
            dqkvz = self._dqkvz_buffer(T, n_ext, qkv)
        if at.gating:
            do, dz = ops.gate_bwd(dg, o.view(T, H, hd), z, dz_out=dqkvz[:, n_qkv : n_qkv + H] if fused else None)
        else:
            do, dz = dg, None
        dq, dk, dv = ops.attention_bwd(do.view(B, S, H, hd), q, k, v, o, lse, True, 0)
        if i == 0 and dv1_acc is not None:
            dv = dv.float() + dv1_acc
        qgain = at.sdpa_qknorm.gain if at.qknorm else self._ones
        dqkv, dv1, dqg, da1, da2, dvs = ops.qkv_post_bwd(
            dq, dk, dv, qkv, v1, at.rope.cos, at.rope.sin, qgain, at.alpha1, at.alpha2, at.scale, B, S, H, Hkv, hd, at.qknorm,
            dqkv_out=dqkvz[:, :n_qkv] if fused else None, dv1_acc=dv1_acc if v1 is not None else None,
        )
        if dv1 is not None:
            dv1_acc = dv1  # the kernel added this block's part to the running sum (or started it)
        if at.qknorm:
            self._acc(at.sdpa_qknorm.gain, dqg)
        if at.value_residual:
            self._acc(at.alpha1, da1)
            self._acc(at.alpha2, da2)
            self._acc(at.scale, dvs)
        if fused:
            w_gate = at.attn_gate.linear.weight
            dn1 = ops.matmul_nn(dqkvz, self.qkvz_w[i])
            if self._wg_tmp is None or self._wg_tmp.shape != (n_ext, w_qkv.size(1)):
                self._wg_tmp = torch.empty((n_ext, w_qkv.size(1)), dtype=torch.float32, device=qkv.device)
            ops.wgrad_accumulate(self._wg_tmp, dqkvz, n1, True)
            self._acc(w_qkv, self._wg_tmp[:n_qkv])
            self._acc(w_gate, self._wg_tmp[n_qkv : n_qkv + H])
        else:
            dn1 = ops.matmul_nn(dqkv, self._w(w_qkv))
            self._wgrad(w_qkv, dqkv, n1)
            if at.gating:
                w_gate = at.attn_gate.linear.weight
                dn1.addmm_(dz, self._w(w_gate))
                self._wgrad(w_gate, dz, n1)
        dx, dx_lp, dgain1 = ops.add_rmsnorm_bwd(dn1, dy, x, blk.ln1.gain, rstd1, scale, self.lp)
        self._acc(blk.ln1.gain, dgain1)
        if self.grad_ready is not None:
            self.grad_ready([p for p in blk.parameters() if p.requires_grad])
        return dx, dx_lp, dv1_acc

    # ------------------------------------------------------------------ whole model
    @torch.no_grad()
    def forward_backward(
        self,
        tokens: Tensor,
        targets: Tensor,
        loss_coef: float = 1.0,
        byte_len: Tensor | None = None,
        first_micro_step: bool = True,
    ) -> StepOutput:
        """Gradients of ``loss_coef * mean_tokens(loss)`` are written (first micro-step) or added to ``p.grad``."""
        model = self.model
        self.ensure_grads()
        self._first_accum = first_micro_step
        self._loss_coef = loss_coef
        if self.moe is not None:
            self.moe.begin_step()
        B, S = tokens.shape
        T = B * S
        L = model.n_layers
        n_ckpt = min(model.num_grad_checkpoint_layers, L)
        ids = tokens.reshape(-1).long()
        with nvtx_range("forward"):
            res = model.embedding.weight.detach()[ids].float()
            delta, v1 = None, None
            saved_all, v1_in, kurts = [], [], []
            for i in range(L):
                with nvtx_range(f"block {i}"):
                    y, m, v, kurt, saved = self._layer_fwd(i, res, delta, v1, B, S)
                v1_in.append(v1)
                saved_all.append((saved[0],) if i < n_ckpt else saved)
                if v1 is None:
                    v1 = v
                res, delta = y, m
                kurts.append(kurt)
            fn = model.final_norm
            xf, hf, rstdf, _ = ops.add_rmsnorm_fwd(res, delta, fn.gain, self._final_scale, fn.eps, self.lp, False)
        head = model.lm_head.linear.weight
        with nvtx_range("cross entropy"):
            if first_micro_step:
                head.grad.zero_()
            loss_tok, z_tok, dh, _ = ops.linear_ce_fwd_bwd(
                hf, self._w(head), targets.reshape(-1), LSE_SQUARE_SCALE, IGNORE_INDEX, loss_coef / T, model.output_mult, dw_out=head.grad
            )
        with nvtx_range("backward"):
            dres, dres_lp, dgain_f = ops.add_rmsnorm_bwd(dh, None, xf, fn.gain, rstdf, self._final_scale, self.lp)
            self._acc(fn.gain, dgain_f)
            if self.grad_ready is not None:
                self.grad_ready([head, fn.gain])
            dv1_acc = None
            for i in reversed(range(L)):
                saved = saved_all[i]
                if len(saved) == 1:  # recompute this block from its fp32 input
                    _, _, _, _, saved = self._layer_fwd(i, saved[0], None, v1_in[i], B, S, want_kurt=False)
                saved_all[i] = None
                with nvtx_range(f"block {i} bwd"):
                    dres, dres_lp, dv1_acc = self._layer_bwd(i, saved, v1_in[i], dres, dres_lp, dv1_acc, B, S)
                del saved
            emb = model.embedding.weight
            if first_micro_step:
                emb.grad.zero_()
            emb.grad.index_add_(0, ids, dres)
            if self.grad_ready is not None:
                self.grad_ready([emb])
        bpb = None
        if byte_len is not None:
            bl = byte_len[targets.reshape(-1).clamp_min(0).long()]
            bpb = (loss_tok * bl).sum() / bl.sum() * NATS_TO_BITS
        aux = self.moe.aux_loss() if self.moe is not None else None
        return StepOutput(loss_tok.mean(), z_tok.mean(), bpb, torch.stack(kurts) / T, loss_tok, aux)

    @torch.no_grad()
    def forward_loss(self, tokens: Tensor, targets: Tensor, byte_len: Tensor | None = None) -> StepOutput:
        """Evaluation: the same kernel sequence without saving activations or producing gradients."""
        model = self.model
        B, S = tokens.shape
        T = B * S
        if self.moe is not None:
            self.moe.begin_step()
        res = model.embedding.weight.detach()[tokens.reshape(-1).long()].float()
        delta, v1, kurts = None, None, []
        for i in range(model.n_layers):
            res, delta, v, kurt, _ = self._layer_fwd(i, res, delta, v1, B, S, train=False)
            if v1 is None:
                v1 = v
            kurts.append(kurt)
        fn = model.final_norm
        _, hf, _, _ = ops.add_rmsnorm_fwd(res, delta, fn.gain, self._final_scale, fn.eps, self.lp, False)
        loss_tok, z_tok, _, _ = ops.linear_ce_fwd_bwd(
            hf, self._w(model.lm_head.linear.weight), targets.reshape(-1), LSE_SQUARE_SCALE, IGNORE_INDEX, 0.0,
            model.output_mult, need_grad=False,
        )
        bpb = None
        if byte_len is not None:
            bl = byte_len[targets.reshape(-1).clamp_min(0).long()]
            bpb = (loss_tok * bl).sum() / bl.sum() * NATS_TO_BITS
        return StepOutput(loss_tok.mean(), z_tok.mean(), bpb, torch.stack(kurts) / T, loss_tok)
