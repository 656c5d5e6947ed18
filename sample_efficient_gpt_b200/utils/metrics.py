"""Throughput / MFU bookkeeping and metric sinks.

MFU formula of the reference (training/trainer.py:139-144,584-592):
``P = L (4 d^2 + 2 d + 2 d d_ff) + d V``; ``FLOPs/token = 6 P + 12 L H hd T``;
``MFU = FLOPs/token * tokens/s / (0.9 * peak * world)``.  The reference hard-codes peaks for a
consumer GPU, a 4-GPU box and 8 H200s and has no entry for other world sizes; here the peak is
looked up from the device name (dense bf16, nominal) and can be overridden with
``SEGPT_PEAK_TFLOPS`` (per GPU), so every world size has a value.
"""

from __future__ import annotations

import json
import os
import time
from pathlib import Path

import torch

NOMINAL_BF16_TFLOPS = {
    "B200": 2250.0,
    "B100": 1750.0,
    "H200": 989.0,
    "H100": 989.0,
    "A100": 312.0,
    "RTX 5090": 209.5,
    "RTX 4090": 165.2,
}


def device_peak_flops(device_name: str | None = None) -> float:
    env = os.environ.get("SEGPT_PEAK_TFLOPS")
    if env:
        return float(env) * 1e12
    if device_name is None:
        device_name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    for key, tf in NOMINAL_BF16_TFLOPS.items():
        if key in device_name:
            return tf * 1e12
    return 1e12  # unknown device (CPU): 1 TFLOP/s so the number is at least finite


def non_embedding_params(mcfg) -> int:
    layer = 4 * mcfg.d_model**2 + 2 * mcfg.d_model + 2 * mcfg.d_model * mcfg.d_ff
    return mcfg.n_layers * layer + mcfg.d_model * mcfg.vocab_size


def flops_per_token(mcfg, seq_len: int) -> float:
    hd = mcfg.head_dim or (mcfg.d_model // mcfg.n_heads)
    return 6.0 * non_embedding_params(mcfg) + 12.0 * mcfg.n_layers * mcfg.n_heads * hd * seq_len


def mfu(mcfg, seq_len: int, tokens_per_s: float, world: int, use_fp8: bool = False, peak: float | None = None) -> float:
    peak = device_peak_flops() if peak is None else peak
    mult = 1.6 if use_fp8 else 0.9
    return flops_per_token(mcfg, seq_len) * tokens_per_s / (peak * mult * world)


class JsonlSink:
    """Offline stand-in for wandb: one JSON object per ``log`` call, same keys."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.id = f"jsonl-{int(time.time())}"

    def log(self, data: dict, step: int | None = None):
        rec = {"_step": step, "_time": time.time()}
        for k, v in data.items():
            if torch.is_tensor(v):
                v = v.item() if v.numel() == 1 else v.tolist()
            rec[k] = v
        with open(self.path, "a") as f:
            f.write(json.dumps(rec, default=str) + "\n")

    def finish(self):
        pass
