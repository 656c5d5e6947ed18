"""Per-sample scoring of SFT data, sharded over GPUs under torchrun (no collectives; one output file per rank).

    torchrun --nproc_per_node 8 -m sample_efficient_gpt_b200.scripts.data_processing.sft.score loss \
        --checkpoint hf_dir --data-file train.jsonl --output-dir out/
    python -m sample_efficient_gpt_b200.scripts.data_processing.sft.score filter --input-path out/loss.jsonl --output-path kept.jsonl

Tasks (the reference's scripts/data_processing/sft/infer_hf_{loss,embedding,reward,safety}.py):
  loss       mean next-token loss over the assistant tokens of ``input.messages + output`` (chat template with the
             assistant mask; without a template: the tokens of the reply), on this package's model or a HF causal LM;
  embedding  mean-pooled last hidden state of an encoder over the rendered conversation (``embedding`` column);
  reward     scalar reward of ``output`` and of every ``generated_outputs`` candidate (``rewards`` column);
  safety     classifier score of the reply (``safety`` column);
  filter     keep samples by loss: below 0.95 x the ``keep_pct`` percentile, plus the band 1.5-1.75 x that percentile.
Rows: ``{"index", "input": {"messages": [...]}, "output": str, ...}``.
"""

from __future__ import annotations

import argparse
from pathlib import Path

import numpy as np
import torch

from sample_efficient_gpt_b200.scripts.data_processing.common import (ClassifierScorer, contiguous_shard, device_for, rank_world,
                                                                      read_rows, write_rows)


def conversation(row: dict) -> list[dict]:
    return row["input"]["messages"] + [{"role": "assistant", "content": row["output"]}]


def tokenize_with_mask(tokenizer, conv: list[dict], max_length: int):
    """ids and a 0/1 mask of the assistant tokens."""
    if getattr(tokenizer, "chat_template", None):
        out = tokenizer.apply_chat_template(conv, return_assistant_tokens_mask=True, return_dict=True, add_generation_prompt=False)
        ids, mask = list(out["input_ids"]), list(out["assistant_masks"])
    else:  # no template: prompt text, then the reply
        prompt = "".join(f"{m['role'].capitalize()}: {m['content']}\n" for m in conv[:-1]) + "Assistant:"
        a = tokenizer.encode(prompt, add_special_tokens=False)
        b = tokenizer.encode(" " + conv[-1]["content"], add_special_tokens=False)
        ids, mask = a + b, [0] * len(a) + [1] * len(b)
    return ids[:max_length], mask[:max_length]


@torch.no_grad()
def sample_loss(model, ids: list[int], mask: list[int], device) -> float:
    x = torch.tensor([ids], dtype=torch.long, device=device)
    out = model(x)
    logits = out[0] if isinstance(out, tuple) else out.logits
    per_tok = torch.nn.functional.cross_entropy(logits[0, :-1].float(), x[0, 1:], reduction="none")
    keep = torch.tensor(mask[1:], device=device, dtype=torch.bool)  # a target counts when it is an assistant token
    return float(per_tok[keep].mean()) if bool(keep.any()) else float("nan")


def load_causal_lm(checkpoint: str, device: str):
    """A converted HF directory or native checkpoint of this package, else any HF causal LM."""
    try:
        from sample_efficient_gpt_b200.evals.generation import load_engine

        eng = load_engine(checkpoint, device)
        return eng.model, eng.tokenizer
    except Exception:
        from transformers import AutoModelForCausalLM, AutoTokenizer

        model = AutoModelForCausalLM.from_pretrained(checkpoint, torch_dtype=torch.bfloat16, local_files_only=True).to(device).eval()
        return model, AutoTokenizer.from_pretrained(checkpoint)


def run_loss(rows, model, tokenizer, device, max_length: int) -> list[dict]:
    ctx = torch.autocast("cuda", torch.bfloat16) if str(device).startswith("cuda") else torch.autocast("cpu", enabled=False)
    out = []
    with ctx:
        for row in rows:
            ids, mask = tokenize_with_mask(tokenizer, conversation(row), max_length)
            out.append({"index": row.get("index"), "input": row["input"], "output": row["output"], "loss": sample_loss(model, ids, mask, device)})
    return out


@torch.no_grad()
def run_embedding(rows, checkpoint: str, device: str, max_length: int, batch_size: int = 32) -> list[dict]:
    from transformers import AutoModel, AutoTokenizer

    tok = AutoTokenizer.from_pretrained(checkpoint)
    model = AutoModel.from_pretrained(checkpoint).to(device).eval()
    texts = ["\n".join(f"{m['role']}: {m['content']}" for m in conversation(r)) for r in rows]
    out = []
    for at in range(0, len(texts), batch_size):
        enc = tok(texts[at : at + batch_size], return_tensors="pt", padding=True, truncation=True, max_length=max_length).to(device)
        h = model(**enc).last_hidden_state
        m = enc["attention_mask"][..., None].to(h.dtype)
        emb = torch.nn.functional.normalize((h * m).sum(1) / m.sum(1).clamp_min(1), dim=-1)
        for r, e in zip(rows[at : at + batch_size], emb.float().cpu().tolist()):
            out.append({**r, "embedding": e})
    return out


def render_for_reward(tokenizer, conv: list[dict]) -> str:
    text = tokenizer.apply_chat_template(conv, tokenize=False)
    bos = getattr(tokenizer, "bos_token", None)
    return text[len(bos):] if bos and text.startswith(bos) else text


def run_reward(rows, scorer: ClassifierScorer, batch_size: int = 8) -> list[dict]:
    out = []
    for row in rows:
        cands = [row["output"]] + list(row.get("generated_outputs", []))
        texts = [render_for_reward(scorer.tok, row["input"]["messages"] + [{"role": "assistant", "content": c}]) for c in cands]
        out.append({**row, "rewards": scorer(texts, batch_size)})
    return out


def run_safety(rows, scorer: ClassifierScorer, batch_size: int = 32) -> list[dict]:
    scores = scorer([r["output"] for r in rows], batch_size)
    return [{**r, "safety": s} for r, s in zip(rows, scores)]


def filter_dataset_by_loss(input_path, output_path, keep_pct: float = 0.25) -> int:
    rows = read_rows(input_path)
    losses = np.array([r["loss"] if r["loss"] is not None else np.nan for r in rows], dtype=float)
    valid = ~np.isnan(losses)
    thresh = np.percentile(losses[valid], int(keep_pct * 100))
    keep = valid & ((losses < 0.95 * thresh) | ((losses < 1.75 * thresh) & (losses > 1.5 * thresh)))
    order = list(np.nonzero(valid & (losses < 0.95 * thresh))[0]) + list(np.nonzero(valid & (losses < 1.75 * thresh) & (losses > 1.5 * thresh))[0])
    write_rows(output_path, [rows[i] for i in order])
    print(f"loss threshold {thresh:.4f}: keeping {keep.sum() / len(rows):.3f} of the samples")
    return int(keep.sum())


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("task", choices=["loss", "embedding", "reward", "safety", "filter"])
    p.add_argument("--checkpoint")
    p.add_argument("--data-file")
    p.add_argument("--output-dir", type=Path, default=Path("."))
    p.add_argument("--output-prefix", default=None)
    p.add_argument("--max-length", type=int, default=1024)
    p.add_argument("--batch-size", type=int, default=8)
    p.add_argument("--world-size", type=int, default=None)
    p.add_argument("--rank", type=int, default=None)
    p.add_argument("--start", type=int, default=None)
    p.add_argument("--end", type=int, default=None)
    p.add_argument("--input-path")
    p.add_argument("--output-path")
    p.add_argument("--keep-pct", type=float, default=0.3)
    a = p.parse_args(argv)
    if a.task == "filter":
        return filter_dataset_by_loss(a.input_path, a.output_path, a.keep_pct)
    rank, world = rank_world(a.rank, a.world_size)
    device = device_for(rank)
    rows = read_rows(a.data_file)[a.start or 0 : a.end]
    mine = contiguous_shard(len(rows), rank, world)
    if len(mine) == 0:
        raise ValueError(f"Rank {rank} has no data to process")
    rows = [rows[i] for i in mine]
    if a.task == "loss":
        model, tok = load_causal_lm(a.checkpoint, device)
        res = run_loss(rows, model, tok, device, a.max_length)
    elif a.task == "embedding":
        res = run_embedding(rows, a.checkpoint, device, a.max_length, a.batch_size)
    else:
        scorer = ClassifierScorer(a.checkpoint, device, a.max_length)
        res = run_reward(rows, scorer, a.batch_size) if a.task == "reward" else run_safety(rows, scorer, a.batch_size)
    write_rows(a.output_dir / f"{a.output_prefix or a.task}_rank{rank}.jsonl", res)


if __name__ == "__main__":
    main()
