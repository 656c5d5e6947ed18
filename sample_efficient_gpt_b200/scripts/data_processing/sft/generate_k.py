"""K sampled replies per prompt for a slice of an SFT dataset, on this package's generation engine.

    torchrun --nproc_per_node 4 -m sample_efficient_gpt_b200.scripts.data_processing.sft.generate_k \
        --model-dir hf_dir --data-file train.jsonl --k 8 --output-dir out/

Same data flow as the reference's scripts/data_processing/sft/infer_vllm_k.py:86-254 (which serves the model through
vLLM data-parallel workers): conversations are cut to whole turns within a character limit and must end with a user turn,
K replies are sampled (temperature, top-k, stop at the end-of-turn tokens) and stored as ``generated_outputs``; rows are
split over the ranks, one output file per rank.
"""

from __future__ import annotations

import argparse
from pathlib import Path

from sample_efficient_gpt_b200.scripts.data_processing.common import contiguous_shard, device_for, rank_world, read_rows, write_rows


def truncate_messages(messages: list[dict], limit: int = 3456) -> list[dict]:
    """Whole (user, assistant) turns while they fit into ``limit`` characters; the result ends with a user message."""
    used, kept = 0, []
    i = 0
    while i < len(messages):
        pair = messages[i : i + 2] if i + 1 < len(messages) and messages[i + 1]["role"] == "assistant" else messages[i : i + 1]
        size = sum(len(m["content"]) for m in pair)
        if used + size > limit:
            break
        kept.extend(pair)
        used += size
        i += 2
    if kept and kept[-1]["role"] == "assistant":
        kept = kept[:-1]
    return kept


def generate_rows(rows: list[dict], engine, k: int, max_new_tokens: int, temperature: float, top_k: int, batch_size: int = 16) -> list[dict]:
    from sample_efficient_gpt_b200.evals.generation import SamplingParams

    params = SamplingParams(n=k, max_tokens=max_new_tokens, temperature=temperature, top_k=top_k, stop_token_ids=engine.default_stop_ids())
    out = []
    usable = [(r, truncate_messages(r["input"]["messages"])) for r in rows]
    usable = [(r, m) for r, m in usable if m]
    for at in range(0, len(usable), batch_size):
        chunk = usable[at : at + batch_size]
        replies = engine.chat([m for _, m in chunk], params)
        for (r, m), texts in zip(chunk, replies):
            out.append({**r, "input": {"messages": m}, "generated_outputs": texts})
    return out


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--model-dir", required=True)
    p.add_argument("--data-file", required=True, type=Path)
    p.add_argument("--output-dir", type=Path, default=Path("data_sft_stage2"))
    p.add_argument("--prefix", default="train_k.jsonl")
    p.add_argument("--start_idx", type=int, default=-1)
    p.add_argument("--end_idx", type=int, default=-1)
    p.add_argument("--limit", type=int, default=0)
    p.add_argument("--k", type=int, default=8)
    p.add_argument("--max-new-tokens", type=int, default=384)
    p.add_argument("--temperature", type=float, default=0.7)
    p.add_argument("--top-k", type=int, default=30)
    a = p.parse_args(argv)
    from sample_efficient_gpt_b200.evals.generation import load_engine

    rank, world = rank_world()
    rows = read_rows(a.data_file)
    if a.start_idx >= 0:
        rows = rows[a.start_idx : (a.end_idx if a.end_idx >= 0 else None)]
    if a.limit > 0:
        rows = rows[: a.limit]
    rows = [rows[i] for i in contiguous_shard(len(rows), rank, world)]
    engine = load_engine(a.model_dir, device_for(rank))
    write_rows(a.output_dir / f"{Path(a.prefix).stem}_rank{rank}.jsonl", generate_rows(rows, engine, a.k, a.max_new_tokens, a.temperature, a.top_k))


if __name__ == "__main__":
    main()
