"""Shared plumbing of the offline data-curation tools: row files (jsonl / jsonl.gz / parquet), rank sharding as under
torchrun (``LOCAL_RANK`` / ``WORLD_SIZE``; no collectives are needed), batched scoring with a Hugging Face
sequence-classification model."""

from __future__ import annotations

import gzip
import json
import os
from pathlib import Path


def rank_world(rank=None, world=None) -> tuple[int, int]:
    return (rank if rank is not None else int(os.environ.get("LOCAL_RANK", 0)),
            world if world is not None else int(os.environ.get("WORLD_SIZE", 1)))


def contiguous_shard(n: int, rank: int, world: int) -> range:
    """ceil(n / world) consecutive items per rank."""
    per = (n + world - 1) // world
    return range(min(n, rank * per), min(n, rank * per + per))


def read_rows(path) -> list[dict]:
    path = Path(path)
    if path.suffix == ".parquet":
        import pyarrow.parquet as pq

        return pq.read_table(path).to_pylist()
    opener = gzip.open if path.suffix == ".gz" else open
    with opener(path, "rt", encoding="utf-8") as f:
        return [json.loads(line) for line in f if line.strip()]


def write_rows(path, rows: list[dict]) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    if path.suffix == ".parquet":
        import pyarrow as pa
        import pyarrow.parquet as pq

        pq.write_table(pa.Table.from_pylist(rows), path, compression="zstd")
        return
    with open(path, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")


def device_for(rank: int) -> str:
    import torch

    if torch.cuda.is_available():
        torch.cuda.set_device(rank)
        return f"cuda:{rank}"
    return "cpu"


class ClassifierScorer:
    """texts -> float scores of a single-logit sequence-classification model (quality / reward / safety heads)."""

    def __init__(self, repo: str, device: str, max_length: int | None = None, dtype=None):
        import torch
        from transformers import AutoModelForSequenceClassification, AutoTokenizer

        self.torch = torch
        self.tok = AutoTokenizer.from_pretrained(repo)
        self.model = AutoModelForSequenceClassification.from_pretrained(repo).to(device, dtype=dtype or torch.bfloat16).eval()
        self.device, self.max_length = device, max_length

    def __call__(self, texts: list[str], batch_size: int = 128) -> list[float]:
        torch = self.torch
        out: list[float] = []
        with torch.inference_mode():
            for i in range(0, len(texts), batch_size):
                enc = self.tok(texts[i : i + batch_size], return_tensors="pt", padding="longest", truncation=True, max_length=self.max_length)
                enc = {k: v.to(self.device) for k, v in enc.items()}
                logits = self.model(**enc).logits
                out.extend(logits[:, 0].float().cpu().tolist() if logits.dim() == 2 else logits.float().cpu().tolist())
        return out


def int_score(score: float) -> int:
    """Quality classifiers regress 0..5: clamp and round."""
    return int(round(max(0.0, min(score, 5.0))))
