"""Decoder-only transformer (pre-norm blocks, value residual from the first block, untied head).

Module tree and parameter names are those of transformer/transformer.py:15-139 of the reference, so
``state_dict()`` is interchangeable with its checkpoints:
``embedding``, ``blocks.{i}.{ln1,attn,ln2,ffn}``, ``final_norm``, ``lm_head.linear`` (+ the inert
``lm_head.weight`` alias when ``weight_tying`` is set: the alias is stored but the head keeps its own
matrix, exactly as in the reference).  ``forward`` returns ``(logits, kurtosis[n_layers])``.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor
from torch.utils.checkpoint import checkpoint

from sample_efficient_gpt_b200.models.attention import KVCache, MultiHeadSelfAttention
from sample_efficient_gpt_b200.models.core import Embedding, Linear, RMSNorm, SwiGLU, softmax
from sample_efficient_gpt_b200.utils.profiling import nvtx_range


def block_kurtosis(x: Tensor) -> Tensor:
    """Mean over tokens of E[x^4] / max(E[x^2], 1e-8)^2 along the feature axis, in fp32, detached."""
    xf = x.detach().float()
    m2 = xf.square().mean(-1).clamp_min(1e-8)
    m4 = xf.pow(4).mean(-1)
    return (m4 / (m2 * m2)).mean()


class Block(nn.Module):
    def __init__(
        self,
        d_model: int,
        n_heads: int,
        d_ff: int,
        attn_qknorm: bool = False,
        attn_val_residual: bool = False,
        attn_gating: bool | str = False,
        n_kv_heads: int | None = None,
        theta: float = 10_000,
        position: int | None = None,
        max_seq_len: int = 8192,
        head_dim: int | None = None,
        moe: dict | None = None,
        device=None,
        dtype=None,
    ):
        super().__init__()
        self.ln1 = RMSNorm(d_model, position=position, device=device, dtype=dtype)
        self.attn = MultiHeadSelfAttention(
            d_model,
            n_heads,
            n_kv_heads=n_kv_heads,
            theta=theta,
            max_seq_len=max_seq_len,
            qknorm=attn_qknorm,
            value_residual=attn_val_residual,
            gating=attn_gating,
            head_dim=head_dim,
            device=device,
            dtype=dtype,
        )
        self.ln2 = RMSNorm(d_model, position=position, device=device, dtype=dtype)
        if moe:
            from sample_efficient_gpt_b200.models.moe import MoEFeedForward

            self.ffn = MoEFeedForward(d_model, device=device, dtype=dtype, **moe)
        else:
            self.ffn = SwiGLU(d_model, d_ff, device=device, dtype=dtype)
        self.is_moe = bool(moe)

    def forward(self, x: Tensor, token_positions=None, v1: Tensor | None = None, kv_cache: KVCache | None = None):
        attn_out, v = self.attn(self.ln1(x), token_positions, v1=v1, kv_cache=kv_cache)
        kurt = block_kurtosis(x)
        y = x + attn_out
        return y + self.ffn(self.ln2(y)), kurt, v


class Transformer(nn.Module):
    def __init__(
        self,
        n_layers: int,
        vocab_size: int,
        d_model: int,
        n_heads: int,
        d_ff: int,
        attn_qknorm: bool = False,
        attn_val_residual: bool = False,
        attn_gating: bool | str = False,
        layernorm_scaling: bool = False,
        theta: float = 10_000,
        n_kv_heads: int | None = None,
        device=None,
        dtype=None,
        weight_tying: bool = False,
        num_grad_checkpoint_layers: int = 0,
        head_dim: int | None = None,
        max_seq_len: int = 8192,
        mup_base_width: int | None = None,
        moe: dict | None = None,
    ):
        super().__init__()
        self.n_layers = n_layers
        self.vocab_size = vocab_size
        self.d_model = d_model
        self.num_grad_checkpoint_layers = num_grad_checkpoint_layers
        # muP readout multiplier: 1 at the base width, base/width above it.  None keeps the reference's
        # parametrisation (init std 1/sqrt(fan_in) plus the Muon sqrt(max(1, out/in)) lr factor only).
        self.output_mult = 1.0 if not mup_base_width else float(mup_base_width) / float(d_model)
        self.embedding = Embedding(vocab_size, d_model, device, dtype)
        self.blocks = nn.ModuleList(
            [
                Block(
                    d_model,
                    n_heads,
                    d_ff,
                    n_kv_heads=n_kv_heads,
                    theta=theta,
                    attn_qknorm=attn_qknorm,
                    attn_val_residual=attn_val_residual,
                    attn_gating=attn_gating,
                    position=pos if layernorm_scaling else None,
                    max_seq_len=max_seq_len,
                    head_dim=head_dim,
                    moe=moe,
                    device=device,
                    dtype=dtype,
                )
                for pos in range(1, n_layers + 1)
            ]
        )
        self.final_norm = RMSNorm(d_model, device=device, dtype=dtype)
        self.lm_head = Linear(d_model, vocab_size, device, dtype)
        if weight_tying:
            # Stored alias only; the head's own matrix (lm_head.linear.weight) is what forward uses.
            self.lm_head.weight = self.embedding.weight

    def aux_loss(self) -> Tensor | None:
        """Sum of the MoE load-balance losses recorded by the last forward (None for dense models)."""
        losses = [b.ffn.last_aux_loss for b in self.blocks if b.is_moe and b.ffn.last_aux_loss is not None]
        return torch.stack(losses).sum() if losses else None

    def hidden_states(self, ids: Tensor, kv_cache: list[KVCache] | None = None) -> tuple[Tensor, Tensor]:
        """Final-normed hidden states ``[B,S,d]`` and the per-block kurtosis vector."""
        x = self.embedding(ids)
        kurt = torch.zeros((len(self.blocks),), dtype=x.dtype, device=x.device)
        v1 = None
        for i, layer in enumerate(self.blocks):
            cache_i = kv_cache[i] if kv_cache is not None else None
            with nvtx_range(f"block {i}"):
                if i < self.num_grad_checkpoint_layers and torch.is_grad_enabled():
                    x, k, v = checkpoint(
                        lambda x_, v1_, layer=layer, cache_i=cache_i: layer(x_, v1=v1_, kv_cache=cache_i),
                        x,
                        v1,
                        use_reentrant=False,
                    )
                else:
                    x, k, v = layer(x, v1=v1, kv_cache=cache_i)
            if v1 is None:
                v1 = v
            kurt[i] = k
        return self.final_norm(x), kurt

    def forward(self, ids: Tensor, kv_cache: list[KVCache] | None = None) -> tuple[Tensor, Tensor]:
        h, kurt = self.hidden_states(ids, kv_cache)
        logits = self.lm_head(h)
        if self.output_mult != 1.0:
            logits = logits * self.output_mult
        return logits, kurt

    @torch.inference_mode()
    def generate(
        self,
        prompt: Tensor,
        eos_token_id: int,
        top_p: float = 0.4,
        temperature: float = 0.7,
        max_steps: int = 32,
        eos_prob_multiplier: float = 1.0,
    ) -> tuple[Tensor, Tensor | None]:
        """KV-cache decoding: greedy at temperature 0, else temperature + nucleus sampling.

        Returns the prompt with the sampled tokens appended and the EOS probability after each step.
        """
        caches = [KVCache() for _ in range(self.n_layers)]
        step_in = prompt
        out_seq = prompt
        eos_trace: list[Tensor] = []
        for _ in range(max_steps):
            logits, _ = self.forward(step_in, kv_cache=caches)
            probs = softmax(logits[:, -1, :].float(), dim=-1, temperature=temperature)
            if temperature == 0:
                nxt = probs.argmax(dim=-1, keepdim=True)
            else:
                probs[:, eos_token_id] *= eos_prob_multiplier
                if top_p < 1.0:
                    sorted_p, sorted_i = probs.sort(-1, descending=True)
                    keep = sorted_p.cumsum(-1) <= top_p
                    keep[:, 0] = True
                    mask = torch.zeros_like(probs, dtype=torch.bool).scatter_(-1, sorted_i, keep)
                    probs = probs * mask
                probs = probs / probs.sum(-1, keepdim=True)
                nxt = torch.multinomial(probs, 1)
            out_seq = torch.cat([out_seq, nxt], dim=-1)
            step_in = nxt
            eos_trace.append(probs[:, eos_token_id])
            if bool((nxt == eos_token_id).all()):
                break
        return out_seq, (torch.cat(eos_trace, dim=-1) if eos_trace else None)


def build_model(mcfg, device="cpu", dtype=torch.float32, ep_group=None) -> Transformer:
    """Instantiate from a ``ModelConfig`` (fp32 master weights, as trainer.py:99-117 of the reference)."""
    moe = None
    if getattr(mcfg, "n_experts", 0):
        moe = dict(
            n_experts=mcfg.n_experts,
            top_k=mcfg.moe_top_k,
            d_ff=mcfg.moe_d_ff or mcfg.d_ff,
            capacity_factor=mcfg.moe_capacity_factor,
            aux_loss_weight=mcfg.moe_aux_loss_weight,
            ep_group=ep_group,
        )
    return Transformer(
        mcfg.n_layers,
        mcfg.vocab_size,
        mcfg.d_model,
        mcfg.n_heads,
        mcfg.d_ff,
        n_kv_heads=mcfg.n_kv_heads,
        attn_qknorm=mcfg.attn_qknorm,
        attn_val_residual=mcfg.attn_val_residual,
        attn_gating=mcfg.attn_gating,
        layernorm_scaling=mcfg.layernorm_scaling,
        theta=mcfg.theta,
        num_grad_checkpoint_layers=mcfg.num_grad_checkpoint_layers,
        weight_tying=mcfg.weight_tying,
        head_dim=getattr(mcfg, "head_dim", None),
        max_seq_len=getattr(mcfg, "max_seq_len", 8192),
        mup_base_width=getattr(mcfg, "mup_base_width", None),
        moe=moe,
        device=device,
        dtype=dtype,
    )
