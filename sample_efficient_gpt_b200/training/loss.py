"""Language-model losses.

``efficient_cross_entropy`` returns ``(loss, z_loss, loss_bpb)`` with the reference's definitions
(training/loss.py:69-99, transformer/ops/cross_entropy.py:96-247): per token
``l = lse - x_y + 1e-6 * lse^2``, ``z = 1e-6 * lse^2``; ``loss = mean(l)`` (so it already contains the
z term), ``z_loss = mean(z)``; targets equal to -100 contribute 0 but count in the mean; bits per
byte ``= sum(l * bytes(y)) / sum(bytes(y)) * 1.44269``.  The gradient carries the in-kernel z term
``2e-6 * lse * softmax`` and nothing flows through the returned ``z_loss``.
``cross_entropy`` is the plain max-shifted variant with ``z = logsumexp(shifted)^2``.
"""

from __future__ import annotations

import torch
from torch import Tensor

from sample_efficient_gpt_b200 import ops
from sample_efficient_gpt_b200.utils.profiling import nvtx_range

LSE_SQUARE_SCALE = 1e-6
IGNORE_INDEX = -100
NATS_TO_BITS = 1.44269


@nvtx_range("cross entropy")
def cross_entropy(logits: Tensor, targets: Tensor) -> tuple[Tensor, Tensor]:
    """Per-token loss and squared log-partition of the max-shifted logits (training/loss.py:10-66)."""
    lf = logits.float()
    m = lf.max(dim=-1, keepdim=True)[0]
    shifted_lse = torch.logsumexp(lf - m, dim=-1)
    tgt = lf.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1)
    return m.squeeze(-1) - tgt + shifted_lse, shifted_lse**2


def bits_per_byte(per_token_loss: Tensor, targets: Tensor, per_token_byte_lengths: Tensor) -> Tensor:
    byte_len = per_token_byte_lengths[targets.reshape(-1).clamp_min(0).long()].view_as(targets)
    nats_per_byte = (per_token_loss.detach().view_as(targets) * byte_len).sum() / byte_len.sum()
    return nats_per_byte * NATS_TO_BITS


@nvtx_range("cross entropy")
def efficient_cross_entropy(
    logits: Tensor, targets: Tensor, weight=None, per_token_byte_lengths: Tensor | None = None
) -> tuple[Tensor, Tensor, Tensor | None]:
    loss_tok, z_tok = ops.softmax_cross_entropy(
        logits.reshape(-1, logits.size(-1)), targets.reshape(-1), LSE_SQUARE_SCALE, IGNORE_INDEX
    )
    bpb = None
    if per_token_byte_lengths is not None:
        bpb = bits_per_byte(loss_tok, targets, per_token_byte_lengths)
    return loss_tok.mean(), z_tok.mean(), bpb


def fused_linear_cross_entropy(
    hidden: Tensor,
    head_weight: Tensor,
    targets: Tensor,
    per_token_byte_lengths: Tensor | None = None,
    logit_scale: float = 1.0,
) -> tuple[Tensor, Tensor, Tensor | None]:
    """Same three values computed from the final hidden states without storing ``[tokens, vocab]`` logits."""
    loss, z_tok, loss_tok = ops.linear_cross_entropy(
        hidden.reshape(-1, hidden.size(-1)), head_weight, targets.reshape(-1), LSE_SQUARE_SCALE, IGNORE_INDEX, logit_scale
    )
    bpb = None
    if per_token_byte_lengths is not None:
        bpb = bits_per_byte(loss_tok, targets, per_token_byte_lengths)
    return loss, z_tok.mean(), bpb
