"""CORE metric driver: evaluates a checkpoint of this framework (``--type se``) or a Hugging Face model (``--type hf``)
on the DCLM eval bundle and writes a per-task CSV.

    python -m sample_efficient_gpt_b200.evals.base_eval --checkpoint ckpt.pt --base_dir ~/.cache/sample_efficient_gpt
    torchrun --nproc_per_node=8 -m sample_efficient_gpt_b200.evals.base_eval --checkpoint ckpt.pt

Same inputs and outputs as evals/base_eval.py:36-238 of the reference: ``<base_dir>/eval_bundle/{core.yaml,
eval_meta_data.csv, eval_data/*.jsonl}``, data shuffled with ``random.Random(1337)``, centred accuracy
``(acc - baseline) / (1 - baseline)`` with the baseline given in percent, CORE = mean of the centred accuracies, CSV under
``<results_dir>/base_eval_continue/<slug>.csv``.  Runs without a process group too (single process, CPU or one GPU);
the metadata table is read with the ``csv`` module.
"""

from __future__ import annotations

import csv
import json
import os
import random
import time
from argparse import ArgumentParser
from contextlib import nullcontext
from pathlib import Path

import torch
import torch.distributed as dist
import yaml

from sample_efficient_gpt_b200.evals.core_eval import evaluate_task


def _rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def print0(*args, **kwargs):
    if _rank() == 0:
        print(*args, **kwargs, flush=True)


def read_random_baselines(path: Path) -> dict[str, float]:
    with open(path, newline="") as f:
        return {row["Eval Task"]: float(row["Random baseline"]) for row in csv.DictReader(f)}


def evaluate_model(base_dir: Path, model, tokenizer, device, max_per_task: int = -1, batch_size: int = 8,
                   task: str | None = None) -> dict:
    bundle = Path(base_dir) / "eval_bundle"
    tasks = yaml.safe_load((bundle / "core.yaml").read_text())["icl_tasks"]
    if task:
        chosen = [t for t in tasks if t.get("label") == task]
        if not chosen:
            raise ValueError(f"Unknown task '{task}'. Available: {sorted({t.get('label') for t in tasks})}")
        tasks = chosen
    baselines = read_random_baselines(bundle / "eval_meta_data.csv")
    results, centered = {}, {}
    for t in tasks:
        t0 = time.monotonic()
        label = t["label"]
        meta = {
            "task_type": t["icl_task_type"],
            "dataset_uri": t["dataset_uri"],
            "num_fewshot": t["num_fewshot"][0],
            "continuation_delimiter": t.get("continuation_delimiter", " "),
        }
        print0(f"Evaluating: {label} ({meta['num_fewshot']}-shot, type: {meta['task_type']})... ", end="")
        with (bundle / "eval_data" / meta["dataset_uri"]).open() as f:
            data = [json.loads(line) for line in f if line.strip()]
        random.Random(1337).shuffle(data)  # files are often ordered; a cropped run should still be a fair sample
        if max_per_task > 0:
            data = data[:max_per_task]
        acc = evaluate_task(model, tokenizer, data, device, meta, batch_size=batch_size)
        base = 0.01 * baselines[label]
        results[label] = acc
        centered[label] = (acc - base) / (1.0 - base)
        print0(f"accuracy: {acc:.4f} | centered: {centered[label]:.4f} | time: {time.monotonic() - t0:.2f}s")
    return {"results": results, "centered_results": centered, "core_metric": sum(centered.values()) / len(centered)}


def get_model(checkpoint, device, tokenizer_path: str | None = None):
    from sample_efficient_gpt_b200.training.trainer import Trainer

    overrides = {"trainer.device": str(device)}
    if tokenizer_path:
        overrides["data.tokenizer_path"] = tokenizer_path
    tr = Trainer(load_from=checkpoint, load_components="infer", compile=False, **overrides)
    tr.model.eval()
    return tr.model, tr.tokenizer, tr.run_id, tr.cfg.project, tr.iteration


def get_model_hf(checkpoint="HuggingFaceTB/SmolLM2-360M", device="cuda", tokenizer_path=None):
    from transformers import AutoModelForCausalLM, AutoTokenizer

    model = AutoModelForCausalLM.from_pretrained(checkpoint, torch_dtype=torch.bfloat16, local_files_only=True).to(device)
    tokenizer = AutoTokenizer.from_pretrained(tokenizer_path or checkpoint)
    return model.eval(), tokenizer, "", "", 0


def write_csv(path: Path, out: dict) -> None:
    os.makedirs(path.parent, exist_ok=True)
    with open(path, "w") as f:
        f.write(f"{'Task':<35}, {'Accuracy':<10}, {'Centered':<10}\n")
        for label, acc in out["results"].items():
            f.write(f"{label:<35}, {acc:<10.6f}, {out['centered_results'][label]:<10.6f}\n")
        f.write(f"{'CORE':<35}, {'':<10}, {out['core_metric']:<10.6f}\n")


def parse_args(argv=None):
    p = ArgumentParser()
    p.add_argument("--checkpoint")
    p.add_argument("--base_dir", default=Path.home() / ".cache" / "sample_efficient_gpt", type=Path)
    p.add_argument("--results_dir", default=Path("evals/results"), type=Path)
    p.add_argument("--type", default="se", help="se or hf")
    p.add_argument("--task", default="", help="specific task, like arc_easy")
    p.add_argument("--max_per_task", type=int, default=-1, help="Max examples per task (-1 = full).")
    p.add_argument("--tokenizer_path", type=str, default="thepowerfuldeez/imu_1_base")
    p.add_argument("--batch", type=int, default=8, help="per-rank eval batch size")
    p.add_argument("--device", default=None, help="default: cuda:<local rank> when CUDA is present, else cpu")
    p.add_argument("--wandb", action="store_true", help="log the results to the training run (needs wandb)")
    return p.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    launched = "RANK" in os.environ and "WORLD_SIZE" in os.environ
    cuda = torch.cuda.is_available() and (args.device or "cuda").startswith("cuda")
    if launched:
        dist.init_process_group("nccl" if cuda else "gloo")
    local = int(os.environ.get("LOCAL_RANK", 0))
    device = args.device or (f"cuda:{local}" if cuda else "cpu")
    if cuda:
        torch.cuda.set_device(torch.device(device))

    if args.type == "hf":
        model, tokenizer, run_id, project, iteration = get_model_hf(args.checkpoint, device, args.tokenizer_path)
        slug = args.checkpoint.replace("/", "_").lower()
    else:
        model, tokenizer, run_id, project, iteration = get_model(args.checkpoint, device, args.tokenizer_path)
        slug = f"base_model_{iteration:06d}"
    ctx = torch.amp.autocast(device_type="cuda", dtype=torch.bfloat16) if cuda else nullcontext()
    with ctx:
        out = evaluate_model(args.base_dir, model, tokenizer, device, args.max_per_task, args.batch, args.task or None)

    if _rank() == 0:
        path = args.results_dir / "base_eval_continue" / f"{slug}.csv"
        write_csv(path, out)
        print(path.read_text())
        if args.wandb and run_id:
            import wandb

            run = wandb.init(project=project, id=run_id, resume="allow")
            run.log({"core_metric": out["core_metric"], **{f"core/{k}": v for k, v in out["centered_results"].items()}})
            run.finish()
    if launched:
        dist.barrier()
        dist.destroy_process_group()
    return out


if __name__ == "__main__":
    main()
