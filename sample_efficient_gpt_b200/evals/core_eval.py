"""CORE metric evaluation (DCLM, arXiv 2406.11794): multiple choice, schema and language-modelling tasks.

Behaviour follows evals/core_eval.py:19-304 of the reference: few-shot prompts (examples drawn with
``random.Random(1234 + idx)``), answer span located by the common prefix (multiple choice) or common suffix (schema) of
the tokenised prompts, a BOS token prepended when the tokenizer has one, per-example forward, mean continuation loss
(or exact greedy match for language modelling), examples strided over ranks and two scalar all-reduces per task.
Prompts are assembled with plain string operations (no template engine).
"""

from __future__ import annotations

import random

import torch
import torch.distributed as dist


def _fewshot_block(lines: list[str]) -> str:
    """Few-shot examples, each followed by a blank line."""
    return "".join(line + "\n\n" for line in lines)


def render_prompts_mc(item, delim, fewshot=None) -> list[str]:
    head = _fewshot_block([f"{ex['query']}{delim}{ex['choices'][ex['gold']]}" for ex in (fewshot or [])])
    return [f"{head}{item['query']}{delim}{choice}" for choice in item["choices"]]


def render_prompts_schema(item, delim, fewshot=None) -> list[str]:
    head = _fewshot_block([f"{ex['context_options'][ex['gold']]}{delim}{ex['continuation']}" for ex in (fewshot or [])])
    return [f"{head}{ctx}{delim}{item['continuation']}" for ctx in item["context_options"]]


def render_prompts_lm(item, delim, fewshot=None) -> list[str]:
    """Two prompts: without and with the continuation.  Contexts are trimmed (some datasets carry trailing blanks) and
    the prompt without the continuation is stripped so that it tokenises to a clean prefix of the other one."""
    head = _fewshot_block([f"{ex['context'].strip()}{delim}{ex['continuation']}" for ex in (fewshot or [])])
    base = f"{head}{item['context'].strip()}{delim}"
    return [base.strip(), base + item["continuation"]]


def find_common_length(seqs, direction: str = "left") -> int:
    n = min(len(s) for s in seqs)
    for i in range(n):
        idx = i if direction == "left" else -1 - i
        if any(s[idx] != seqs[0][idx] for s in seqs):
            return i
    return n


def stack_sequences(tokens, pad_id: int) -> torch.Tensor:
    out = torch.full((len(tokens), max(len(t) for t in tokens)), pad_id, dtype=torch.long)
    for i, t in enumerate(tokens):
        out[i, : len(t)] = torch.tensor(t, dtype=torch.long)
    return out


def bos_token_id(tokenizer):
    for getter in ("get_bos_token_id",):
        fn = getattr(tokenizer, getter, None)
        if callable(fn):
            try:
                v = fn()
                if v is not None:
                    return v
            except TypeError:
                pass
    for attr in ("bos_token_id", "eos_token_id"):
        v = getattr(tokenizer, attr, None)
        if v is not None:
            return v
    added = getattr(tokenizer, "added_tokens_decoder", None)
    return next(iter(added), None) if added else None


def encode_prompts(tokenizer, prompts: list[str]) -> list[list[int]]:
    enc = tokenizer(prompts, add_special_tokens=False)
    ids = enc["input_ids"] if isinstance(enc, dict) or hasattr(enc, "keys") else getattr(enc, "input_ids", enc)
    bos = bos_token_id(tokenizer)
    return [([bos] if bos is not None else []) + list(s) for s in ids]


def answer_spans(task_type: str, tokens):
    """(token lists, start indices, end indices) of the scored continuation per prompt."""
    if task_type == "multiple_choice":
        start = find_common_length(tokens, "left")
        return tokens, [start] * len(tokens), [len(t) for t in tokens]
    if task_type == "schema":
        suf = find_common_length(tokens, "right")
        return tokens, [len(t) - suf for t in tokens], [len(t) for t in tokens]
    without, with_ = tokens
    assert len(without) < len(with_) and with_[: len(without)] == without, "prompt without the continuation must be a prefix"
    return [with_], [len(without)], [len(with_)]


@torch.no_grad()
def forward_model(model, input_ids: torch.Tensor):
    """Per-position next-token loss (last column NaN) and argmax predictions."""
    out = model(input_ids)
    logits = out[0] if isinstance(out, tuple) else out.logits
    B, T = input_ids.shape
    targets = torch.roll(input_ids, shifts=-1, dims=1)
    losses = torch.nn.functional.cross_entropy(logits.reshape(B * T, -1).float(), targets.reshape(-1), reduction="none").view(B, T)
    losses[:, -1] = float("nan")
    return losses, logits.argmax(dim=-1)


RENDER = {"multiple_choice": render_prompts_mc, "schema": render_prompts_schema, "language_modeling": render_prompts_lm}


@torch.no_grad()
def evaluate_example(idx, model, tokenizer, data, device, task_meta) -> bool:
    item = data[idx]
    ttype, k, delim = task_meta["task_type"], task_meta["num_fewshot"], task_meta["continuation_delimiter"]
    if ttype not in RENDER:
        raise ValueError(f"Unsupported task type: {ttype}")
    fewshot = []
    if k > 0:
        rng = random.Random(1234 + idx)
        fewshot = [data[i] for i in rng.sample([i for i in range(len(data)) if i != idx], k)]
    prompts = RENDER[ttype](item, delim, fewshot)
    tokens, starts, ends = answer_spans(ttype, encode_prompts(tokenizer, prompts))
    max_len = getattr(model, "max_seq_len", None)
    if max_len:
        cropped = [(t[-max_len:], s - max(0, len(t) - max_len), e - max(0, len(t) - max_len)) for t, s, e in zip(tokens, starts, ends)]
        tokens, starts, ends = map(list, zip(*cropped))
    pad = getattr(tokenizer, "pad_token_id", None)
    pad = pad if pad is not None else (bos_token_id(tokenizer) or 0)
    input_ids = stack_sequences(tokens, pad).to(device)
    losses, preds = forward_model(model, input_ids)
    if ttype == "language_modeling":
        s, e = starts[0], ends[0]
        return bool(torch.all(preds[0, s - 1 : e - 1] == input_ids[0, s:e]).item())
    means = [losses[i, s - 1 : e - 1].mean().item() for i, (s, e) in enumerate(zip(starts, ends))]
    return means.index(min(means)) == item["gold"]


def evaluate_task(model, tokenizer, data, device, task_meta, batch_size: int = 8) -> float:
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    mine = list(range(rank, len(data), world))
    correct = sum(float(evaluate_example(i, model, tokenizer, data, device, task_meta)) for i in mine)
    c = torch.tensor(correct, device=device)
    n = torch.tensor(float(len(mine)), device=device)
    if world > 1:
        dist.barrier()
        dist.all_reduce(c)
        dist.all_reduce(n)
    return (c / n).item() if n.item() > 0 else 0.0
