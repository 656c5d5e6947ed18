"""Chat-model evaluation (ARC, MMLU, GSM8K variants, HumanEval -> ChatCORE) on this package's own generation engine.

    torchrun --nproc-per-node=4 -m sample_efficient_gpt_b200.evals.chat_eval --checkpoint /path/to/hf_checkpoint

Same tasks, sampling settings, rank striding, letter picking, centred mean and CSV as evals/chat_eval.py:37-388 of the
reference.  Data parallel: every rank holds a replica and takes problems ``rank::world``; the two counters are summed
with one all-reduce.  Generation is ``generation.ChatEngine`` (the reference hands this to vLLM); any object with
``chat(conversations, SamplingParams) -> list[list[str]]`` can be passed instead.
"""

from __future__ import annotations

import argparse
import os
from functools import partial
from pathlib import Path

import torch
import torch.distributed as dist

from sample_efficient_gpt_b200.evals.generation import SamplingParams, load_engine

ALL_TASKS = ["ARC-Easy", "ARC-Challenge", "MMLU", "GSM8K", "GSM8K_5shot", "GSM8K_5shot_cot", "HumanEval"]
BASELINE_ACCURACY = {"ARC-Easy": 0.25, "ARC-Challenge": 0.25, "MMLU": 0.25}  # the others: 0


def task_factory(name: str):
    from sample_efficient_gpt_b200.evals.tasks.arc import ARC
    from sample_efficient_gpt_b200.evals.tasks.gsm8k import GSM8K
    from sample_efficient_gpt_b200.evals.tasks.humaneval import HumanEval
    from sample_efficient_gpt_b200.evals.tasks.mmlu import MMLU

    return {
        "HumanEval": HumanEval,
        "MMLU": partial(MMLU, subset="all", split="test"),
        "ARC-Easy": partial(ARC, subset="ARC-Easy", split="test"),
        "ARC-Challenge": partial(ARC, subset="ARC-Challenge", split="test"),
        "GSM8K": partial(GSM8K, subset="main", split="test", few_shot=False),
        "GSM8K_5shot": partial(GSM8K, subset="main", split="test", few_shot=True),
        "GSM8K_5shot_cot": partial(GSM8K, subset="main", split="test", few_shot=True, use_llama_system_prompt=True),
    }[name]


def pick_letter(text: str, letters) -> str | None:
    """First character of the reply that (upper-cased) is one of the allowed letters."""
    return next((ch.upper() for ch in text.strip() if ch.upper() in letters), None)


def _sum_over_ranks(passed: int, total: int, device) -> tuple[int, int]:
    if dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([passed, total], dtype=torch.long, device=device)
        dist.all_reduce(t)
        passed, total = int(t[0]), int(t[1])
    return passed, total


def _log(log_file, *fields):
    if log_file is not None:
        Path(log_file).parent.mkdir(exist_ok=True, parents=True)
        with Path(log_file).open("a") as f:
            f.write(",".join(str(x) for x in fields) + "\n")


def run_eval(task, engine, params: SamplingParams, batch_size: int, rank: int, world_size: int, reduce_device,
             max_problems: int | None = None, log_file=None, quiet: bool = False) -> float:
    """One pass over the task; generative tasks pass if any of the n samples passes, categorical ones compare the
    picked letter."""
    n = len(task) if max_problems is None else min(len(task), max_problems)
    mine = list(range(rank, n, world_size))
    categorical = task.eval_type == "categorical"
    passed = total = 0
    for at in range(0, len(mine), batch_size):
        idxs = mine[at : at + batch_size]
        convs = [task[i] for i in idxs]
        replies = engine.chat([c["messages"][:-1] for c in convs], params)  # the gold reply is dropped
        for i, conv, texts in zip(idxs, convs, replies):
            if categorical:
                letter = pick_letter(texts[0], conv["letters"])
                ok = bool(task.evaluate(conv, letter)) if letter else False
                _log(log_file, type(task).__name__, i, letter, ok)
            else:
                outcomes = [bool(task.evaluate(conv, t)) for t in texts]
                ok = any(outcomes)
                _log(log_file, type(task).__name__, i, texts[0], outcomes[0])
            passed += int(ok)
            total += 1
        if not quiet:
            print(f"\r\033[KRank {rank} processed {total}/{len(mine)} ({100 * passed / max(total, 1):.2f}%)", end="", flush=True)
    if not quiet:
        print()
    passed, total = _sum_over_ranks(passed, total, reduce_device)
    if rank == 0 and not quiet:
        print(f"Final: {passed}/{total} ({100 * passed / max(total, 1):.2f}%)")
    return passed / total if total > 0 else 0.0


def run_chat_eval(task_name, engine, rank, world_size, reduce_device, batch_size=1, max_new_tokens=512, temperature=0.0,
                  top_k=50, num_samples=1, max_problems=None, log_file=None, task=None, quiet=False) -> float:
    task = task if task is not None else task_factory(task_name)()
    stop = engine.default_stop_ids()
    if task.eval_type == "generative":
        params = SamplingParams(n=num_samples, max_tokens=max_new_tokens, temperature=temperature, top_k=top_k, stop_token_ids=stop)
    elif task.eval_type == "categorical":
        params = SamplingParams(n=1, max_tokens=8, temperature=0.0, top_k=top_k, stop_token_ids=stop)
    else:
        raise ValueError(f"Unsupported task evaluation type: {task.eval_type}")
    return run_eval(task, engine, params, batch_size, rank, world_size, reduce_device, max_problems, log_file, quiet)


def chatcore(results: dict[str, float]) -> float | None:
    """Mean of the baseline-centred accuracies, defined only when every task was run."""
    if not all(t in results for t in ALL_TASKS):
        return None
    centred = [(acc - BASELINE_ACCURACY.get(t, 0.0)) / (1.0 - BASELINE_ACCURACY.get(t, 0.0)) for t, acc in results.items()]
    return sum(centred) / len(centred)


def parse_args(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--checkpoint", type=str, required=True, help="converted HF directory or native .pt checkpoint")
    p.add_argument("--base-dir", type=str, default="evals/results", help="directory for the csv results")
    p.add_argument("-a", "--task-name", type=str, default=None, help="Default = all tasks. Use | to split multiple tasks.")
    p.add_argument("-d", "--dtype", type=str, default="bfloat16", choices=["float32", "bfloat16", "auto"])
    p.add_argument("-t", "--temperature", type=float, default=0.0)
    p.add_argument("-m", "--max-new-tokens", type=int, default=1024)
    p.add_argument("-n", "--num-samples", type=int, default=1)
    p.add_argument("-k", "--top-k", type=int, default=30)
    p.add_argument("-b", "--batch-size", type=int, default=32)
    p.add_argument("-x", "--max-problems", type=int, default=None)
    p.add_argument("--log-file", type=Path, default=None)
    p.add_argument("--device-type", type=str, default="", choices=["", "cuda", "cpu"], help="empty => autodetect")
    return p.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    out_csv = Path(args.base_dir) / "chat_eval" / ("_".join(Path(args.checkpoint).parts[-3:]) + ".csv")
    out_csv.parent.mkdir(exist_ok=True, parents=True)
    cuda = torch.cuda.is_available() and args.device_type != "cpu"
    launched = "RANK" in os.environ and "WORLD_SIZE" in os.environ
    if launched and not dist.is_initialized():
        dist.init_process_group(backend="nccl" if cuda else "gloo")
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    local = int(os.environ.get("LOCAL_RANK", rank))
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    engine = load_engine(args.checkpoint, device, args.dtype, max_model_len=2048)

    log_file = args.log_file
    if log_file is not None:
        if world > 1:
            log_file = log_file.with_name(f"{log_file.stem}.rank{rank}{log_file.suffix}")
        if log_file.exists():
            log_file.unlink()

    results: dict[str, float] = {}
    for name in (ALL_TASKS if args.task_name is None else args.task_name.split("|")):
        results[name] = run_chat_eval(name, engine, rank, world, device, args.batch_size, args.max_new_tokens, args.temperature,
                                      args.top_k, args.num_samples, args.max_problems, log_file)
        if rank == 0:
            print(f"{name} accuracy: {100 * results[name]:.2f}%")
    core = chatcore(results)
    if core is not None:
        results["ChatCORE metric"] = core
    if rank == 0:
        print(results)
        with open(out_csv, "w") as f:
            f.write(f"{'Task':<35}, {'Accuracy':<10}\n")
            for label, v in results.items():
                f.write(f"{label:<35}, {v:<10.6f}\n")
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return results


if __name__ == "__main__":
    main()
