"""Task = an indexable set of conversations (+ how to score a reply).  Mirrors evals/tasks/common.py:11-135 of the
reference: strided logical views (``start/stop/step``), ``TaskMixture`` (deterministic shuffle, seed 42) and
``TaskSequence`` (curriculum), and the multiple-choice rendering with the letter *after* the choice.

``load_rows`` is the one place datasets come from: a local mirror first (``$SEGPT_DATASETS_DIR/<repo with '/' as
'__'>/[<subset>/]<split>.{jsonl,parquet}``), the ``datasets`` hub library second; rows are permuted the way
``Dataset.shuffle(seed)`` does (``numpy.random.default_rng(seed).permutation``).
"""

from __future__ import annotations

import json
import os
import random
from pathlib import Path


class Rows:
    """A list of dict rows with an optional index permutation."""

    def __init__(self, rows, order=None):
        self.rows, self.order = rows, order

    def __len__(self):
        return len(self.rows) if self.order is None else len(self.order)

    def __getitem__(self, i):
        return self.rows[int(i if self.order is None else self.order[i])]

    def __iter__(self):
        return (self[i] for i in range(len(self)))

    def shuffle(self, seed: int) -> "Rows":
        import numpy as np

        return Rows(self.rows, np.random.default_rng(seed).permutation(len(self.rows)))

    def select(self, idx) -> "Rows":
        return Rows([self[i] for i in idx])


def _local_file(repo: str, subset: str | None, split: str) -> Path | None:
    root = os.environ.get("SEGPT_DATASETS_DIR")
    if not root:
        return None
    base = Path(root) / repo.replace("/", "__")
    for d in ([base / subset] if subset else []) + [base]:
        for ext in (".jsonl", ".parquet"):
            if (d / f"{split}{ext}").exists():
                return d / f"{split}{ext}"
    return None


def load_rows(repo: str, subset: str | None = None, split: str = "train", seed: int | None = 42):
    path = _local_file(repo, subset, split)
    if path is not None:
        if path.suffix == ".jsonl":
            rows = [json.loads(line) for line in path.read_text().splitlines() if line.strip()]
        else:
            import pyarrow.parquet as pq

            rows = pq.read_table(path).to_pylist()
        ds = Rows(rows)
    else:
        try:
            from datasets import load_dataset
        except ImportError as e:
            raise RuntimeError(f"{repo}: no local mirror under $SEGPT_DATASETS_DIR and `datasets` is not installed") from e
        ds = load_dataset(repo, subset, split=split) if subset else load_dataset(repo, split=split)
    return ds.shuffle(seed=seed) if seed is not None else ds


class Task:
    def __init__(self, start: int = 0, stop: int | None = None, step: int = 1):
        assert start >= 0, f"Start must be non-negative, got {start}"
        assert stop is None or stop >= start, f"Stop should be greater than or equal to start, got {stop} and {start}"
        assert step >= 1, f"Step must be strictly positive, got {step}"
        self.start, self.stop, self.step = start, stop, step

    @property
    def eval_type(self) -> str:  # 'generative' | 'categorical'
        raise NotImplementedError

    def num_examples(self) -> int:
        raise NotImplementedError

    def get_example(self, index: int):
        raise NotImplementedError

    def evaluate(self, conversation, completion):
        raise NotImplementedError

    def __len__(self) -> int:
        stop = self.num_examples() if self.stop is None else self.stop
        return max(0, -(-(stop - self.start) // self.step))

    def __getitem__(self, index: int):
        assert isinstance(index, int), f"Index must be an integer, got {type(index)}"
        return self.get_example(self.start + index * self.step)

    def __iter__(self):
        return (self[i] for i in range(len(self)))


class TaskMixture(Task):
    """All examples of several tasks in one deterministic shuffle (pass a task twice to oversample it)."""

    def __init__(self, tasks, **kwargs):
        super().__init__(**kwargs)
        self.tasks = tasks
        self.lengths = [len(t) for t in tasks]
        self.num_conversations = sum(self.lengths)
        self.index_map = [(ti, li) for ti, n in enumerate(self.lengths) for li in range(n)]
        random.Random(42).shuffle(self.index_map)

    def num_examples(self):
        return self.num_conversations

    def get_example(self, index):
        assert 0 <= index < self.num_conversations, f"Index {index} out of range for mixture with {self.num_conversations} conversations"
        ti, li = self.index_map[index]
        return self.tasks[ti][li]


class TaskSequence(Task):
    """Tasks one after another (a training curriculum)."""

    def __init__(self, tasks, **kwargs):
        super().__init__(**kwargs)
        self.tasks = tasks
        self.lengths = [len(t) for t in tasks]
        self.num_conversations = sum(self.lengths)

    def num_examples(self):
        return self.num_conversations

    def get_example(self, index):
        assert 0 <= index < self.num_conversations, f"Index {index} out of range for sequence with {self.num_conversations} conversations"
        for task, n in zip(self.tasks, self.lengths):
            if index < n:
                return task[index]
            index -= n


def render_mc(question: str, letters, choices) -> str:
    """Letter after the choice (binds better for small models) and no blank between '=' and the letter, so the prompt
    carries the same token the assistant must answer with."""
    lines = "".join(f"- {c}={l}\n" for l, c in zip(letters, choices))
    return f"Multiple Choice question: {question}\n{lines}\nRespond only with the letter of the correct answer."


class ConversationTask(Task):
    """A plain SFT conversation dataset: rows with a ``messages`` list."""

    def __init__(self, rows, **kwargs):
        super().__init__(**kwargs)
        self.ds = rows
        self.length = len(rows)

    def num_examples(self):
        return self.length

    def get_example(self, index):
        return {"messages": self.ds[index]["messages"]}
