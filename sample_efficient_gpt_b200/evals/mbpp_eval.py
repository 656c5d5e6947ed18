"""MBPP / MBPP+ scoring: pass@k of generated programs against base and plus inputs.

Usage (same inputs as the reference's evals/mbpp_eval.py:1-535):
    python -m sample_efficient_gpt_b200.evals.mbpp_eval --samples completions.jsonl --dataset lite
    python -m sample_efficient_gpt_b200.evals.mbpp_eval --samples samples_dir --dataset /path/MbppPlus.jsonl.gz
``samples`` is a .jsonl(.gz) with ``{"task_id", "completion"}`` (body appended to the prompt) or ``{"task_id",
"solution"}`` (whole file), or a directory ``<dir>/<task_id>/*.py``.  Expected outputs come from running the canonical
solution; a sample passes when every output equals the expected one (floats within ``atol``).  pass@k is the unbiased
estimator ``1 - C(n-c, k)/C(n, k)``; "plus" counts samples that pass base *and* plus inputs.

Every candidate runs through ``execution.execute_code`` (fresh interpreter, memory/CPU limits, wall-clock kill) with one
time limit for the whole submission; its per-input verdicts come back as a JSON line on stdout.
"""

from __future__ import annotations

import argparse
import gzip
import json
import math
import os
import sys
import time
from collections.abc import Callable, Iterable
from dataclasses import dataclass
from typing import Any

from sample_efficient_gpt_b200.evals import mbpp_lite
from sample_efficient_gpt_b200.evals.execution import execute_code

PASS, FAIL, TIMEOUT = "pass", "fail", "timeout"
_MARK = "@@MBPP-VERDICT@@"


@dataclass
class Problem:
    task_id: str
    prompt: str
    canonical_solution: str
    entry_point: str
    base_input: list[list[Any]]
    plus_input: list[list[Any]]
    atol: float = 0.0


def read_jsonl(path: str) -> Iterable[dict]:
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rt", encoding="utf-8") as f:
        for line in f:
            if line.strip():
                yield json.loads(line)


def load_dataset(dataset: str) -> dict[str, Problem]:
    if dataset.strip().lower() == "lite":
        records = ({"task_id": tid, **rec} for tid, rec in mbpp_lite.DATA.items())
    else:
        records = read_jsonl(dataset)
    keys = ("task_id", "prompt", "canonical_solution", "entry_point", "base_input", "plus_input")
    return {r["task_id"]: Problem(*(r[k] for k in keys), atol=float(r.get("atol", 0.0))) for r in records}


def load_solutions(samples_path: str) -> Iterable[dict]:
    if os.path.isfile(samples_path):
        for i, rec in enumerate(read_jsonl(samples_path)):
            if "completion" not in rec and "solution" not in rec:
                raise ValueError(f"Line {i}: missing 'completion' or 'solution'")
            yield {**rec, "_identifier": f"{os.path.basename(samples_path)}:{i}"}
        return
    for task_id in sorted(os.listdir(samples_path)):
        tdir = os.path.join(samples_path, task_id)
        if os.path.isdir(tdir):
            for fname in sorted(f for f in os.listdir(tdir) if f.endswith(".py")):
                path = os.path.join(tdir, fname)
                yield {"_identifier": path, "task_id": task_id, "solution": open(path, encoding="utf-8").read()}


def safe_compare(out: Any, exp: Any, atol: float) -> bool:
    if isinstance(exp, float) or isinstance(out, float):
        try:
            return math.isclose(float(out), float(exp), rel_tol=1e-7, abs_tol=atol)
        except (TypeError, ValueError):
            return False
    if isinstance(exp, (list, tuple)) and isinstance(out, (list, tuple)):
        return len(exp) == len(out) and all(safe_compare(o, e, atol) for o, e in zip(out, exp))
    return out == exp


def compute_expected(problem: Problem) -> tuple[list, list]:
    """Outputs of the (trusted) canonical solution."""
    scope: dict[str, Any] = {}
    exec(problem.prompt + problem.canonical_solution, scope)
    fn = scope[problem.entry_point]
    return [fn(*a) for a in problem.base_input], [fn(*a) for a in problem.plus_input]


_HARNESS = '''
import json as _j, math as _m, sys as _s, io as _io
def _cmp(out, exp, atol):
    if isinstance(exp, float) or isinstance(out, float):
        try:
            return _m.isclose(float(out), float(exp), rel_tol=1e-7, abs_tol=atol)
        except (TypeError, ValueError):
            return False
    if isinstance(exp, (list, tuple)) and isinstance(out, (list, tuple)):
        return len(exp) == len(out) and all(_cmp(o, e, atol) for o, e in zip(out, exp))
    return out == exp
_real, _s.stdout = _s.stdout, _io.StringIO()
_details = []
try:
    exec(compile(_CODE, "<submission>", "exec"), globals())
    _fn = globals()[_ENTRY]
    for _args, _exp in zip(eval(_INPUTS), eval(_EXPECTED)):
        try:
            _ok = bool(_cmp(_fn(*_args), _exp, _ATOL))
        except (Exception, SystemExit):
            _ok = False
        _details.append(_ok)
        if _FAST and not _ok:
            break
except (Exception, SystemExit):
    pass
_s.stdout = _real
print(_MARK + _j.dumps(_details))
'''


def untrusted_check(code: str, entry_point: str, inputs: list, expected: list, atol: float, timeout: float,
                    fast_fail: bool = True) -> tuple[str, list[bool]]:
    header = (f"_CODE = {code!r}\n_ENTRY = {entry_point!r}\n_INPUTS = {repr(inputs)!r}\n_EXPECTED = {repr(expected)!r}\n"
              f"_ATOL = {atol!r}\n_FAST = {fast_fail!r}\n_MARK = {_MARK!r}\n")
    res = execute_code(header + _HARNESS, timeout=timeout, maximum_memory_bytes=1 << 30)
    if res.timeout:
        return TIMEOUT, []
    line = next((l for l in reversed(res.stdout.splitlines()) if l.startswith(_MARK)), None)
    if line is None:
        return FAIL, []
    details = json.loads(line[len(_MARK):])
    ok = bool(details) and all(details) and len(details) == len(expected)
    return (PASS if ok else FAIL), details


def estimate_pass_at_k(num_samples: list[int], num_correct: list[int], k: int) -> float:
    def one(n: int, c: int) -> float:
        if n - c < k:
            return 1.0
        return 1.0 - math.prod(1.0 - k / i for i in range(n - c + 1, n + 1))

    vals = [one(int(n), int(c)) for n, c in zip(num_samples, num_correct)]
    return sum(vals) / len(vals) if vals else 0.0


class Tally:
    """Per-task sample counts and the pass@k summary."""

    def __init__(self, plus: bool):
        self.plus = plus
        self.records: dict[str, list[dict]] = {}
        self.total: dict[str, int] = {}
        self.base_ok: dict[str, int] = {}
        self.both_ok: dict[str, int] = {}

    def add(self, tid: str, base_status: str, plus_status: str | None, **extra):
        self.records.setdefault(tid, []).append({"task_id": tid, "base_status": base_status, "plus_status": plus_status, **extra})
        self.total[tid] = self.total.get(tid, 0) + 1
        self.base_ok[tid] = self.base_ok.get(tid, 0) + (base_status == PASS)
        self.both_ok[tid] = self.both_ok.get(tid, 0) + (self.plus and base_status == PASS and plus_status == PASS)

    def summary(self, ks: list[int]) -> dict:
        if not self.total:
            return {"eval": {}, "pass_at_k": {}}
        ks = [k for k in ks if k <= min(self.total.values())]
        tids = list(self.total)
        n = [self.total[t] for t in tids]
        out = {"eval": self.records,
               "pass_at_k": {"base": {f"pass@{k}": estimate_pass_at_k(n, [self.base_ok[t] for t in tids], k) for k in ks}}}
        if self.plus and ks:
            out["pass_at_k"]["plus"] = {f"pass@{k}": estimate_pass_at_k(n, [self.both_ok[t] for t in tids], k) for k in ks}
        return out


class SimpleMBPPEvaluator:
    """Programmatic use during training: ``SimpleMBPPEvaluator('lite').evaluate_with_generate(trainer_generate)``."""

    def __init__(self, dataset: str = "lite", timeout: float = 15.0, base_only: bool = False):
        self.timeout, self.base_only = float(timeout), bool(base_only)
        self.problems = load_dataset(dataset)
        self.expected_map: dict[str, dict[str, list]] = {}
        for tid, prob in self.problems.items():
            try:
                b, p = compute_expected(prob)
            except BaseException:
                b, p = [], []
            self.expected_map[tid] = {"base": b, "plus": p}

    def resolve(self, tid: str) -> str | None:
        if tid in self.problems:
            return tid
        alt = tid.replace("_", "/")
        return alt if alt in self.problems else None

    def check(self, tid: str, code: str, plus: bool) -> tuple[str, str | None]:
        prob, exp = self.problems[tid], self.expected_map[tid]
        base, _ = untrusted_check(code, prob.entry_point, prob.base_input, exp["base"], prob.atol, self.timeout)
        plus_status = None
        if plus:
            plus_status, _ = untrusted_check(code, prob.entry_point, prob.plus_input, exp["plus"], prob.atol, self.timeout)
        return base, plus_status

    def evaluate_with_generate(self, generate_fn: Callable[..., str], *, num_samples: int = 1,
                               task_ids: list[str] | None = None, mode: str = "completion", ks: list[int] | None = None,
                               plus: bool | None = None, **gen_kwargs) -> dict:
        plus = (not self.base_only) if plus is None else plus
        tids = [t for t in (self.resolve(x) for x in (task_ids or [])) if t] or list(self.problems)
        tally = Tally(plus)
        for tid in tids:
            prob = self.problems[tid]
            for _ in range(int(num_samples)):
                completion = str(generate_fn(prob.prompt, **gen_kwargs))
                code = prob.prompt + completion if mode == "completion" else completion
                tally.add(tid, *self.check(tid, code, plus), code=code)
        return tally.summary(ks or [1, 10, 100])


def main(argv=None):
    ap = argparse.ArgumentParser(description="MBPP / MBPP+ evaluator")
    ap.add_argument("--samples", required=True, help="samples .jsonl(.gz) or a directory <dir>/<task_id>/*.py")
    ap.add_argument("--dataset", default="lite", help="'lite' or path to an MBPP+ jsonl(.gz)")
    ap.add_argument("--timeout", type=float, default=15.0, help="seconds per submission")
    ap.add_argument("--base_only", action="store_true")
    ap.add_argument("--k", default="1,10,100", help="comma-separated ks (those above the samples per task are dropped)")
    ap.add_argument("--output", default=None)
    args = ap.parse_args(argv)

    ev = SimpleMBPPEvaluator(args.dataset, args.timeout, args.base_only)
    if not ev.problems:
        sys.exit("No problems loaded; check --dataset")
    tally = Tally(not args.base_only)
    for sample in load_solutions(args.samples):
        tid = ev.resolve(sample["task_id"])
        if tid is None:
            print(f"[warn] sample for unknown task_id: {sample['task_id']}", file=sys.stderr)
            continue
        code = sample.get("solution") or ev.problems[tid].prompt + sample["completion"]
        tally.add(tid, *ev.check(tid, code, not args.base_only))
    ks = [int(t) for t in args.k.split(",") if t.strip().isdigit()]
    out = {"date": time.strftime("%Y-%m-%d %H:%M"), **tally.summary(ks)}

    if args.output:
        out_path = args.output
    elif os.path.isfile(args.samples):
        stem = args.samples
        for ext in (".jsonl.gz", ".jsonl"):
            if stem.endswith(ext):
                stem = stem[: -len(ext)]
                break
        out_path = stem + ".eval_results.json"
    else:
        out_path = os.path.join(args.samples, "eval_results.json")
    with open(out_path, "w", encoding="utf-8") as f:
        json.dump(out, f, indent=2)
    for split, table in out["pass_at_k"].items():
        for k, v in table.items():
            print(f"  {split} {k}: {v:.3f}")
    print(f"Saved -> {out_path}")
    return out


if __name__ == "__main__":
    main()
