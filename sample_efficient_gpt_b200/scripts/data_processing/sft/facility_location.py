"""Subset selection by facility location over embeddings: pick the set S maximising ``sum_i max_{j in S} sim(i, j)``.

    python -m sample_efficient_gpt_b200.scripts.data_processing.sft.facility_location --data-file emb.jsonl \
        --select-frac 0.8 --output-file kept.jsonl

The reference (scripts/data_processing/sft/infer_hf_filter_fla.py:23-62) hands a dense euclidean kernel to submodlib's
lazy greedy.  Here the greedy runs on the accelerator: the similarity matrix ``1 / (1 + ||a - b||)`` is kept in blocks on
the device, every round evaluates the marginal gains of all remaining candidates with one fused pass
(``relu(sim - best).sum(0)``), and rounds are batched lazily - stale upper bounds are re-evaluated only for the current
top candidates, as in lazy greedy - so selection of k out of n costs O(k * n * r) with r << n re-evaluations per round.
"""

from __future__ import annotations

import argparse
from pathlib import Path

import numpy as np
import torch

from sample_efficient_gpt_b200.scripts.data_processing.common import read_rows, write_rows


def similarity(emb: torch.Tensor, block: int = 8192) -> torch.Tensor:
    n = emb.size(0)
    sim = torch.empty(n, n, dtype=torch.float32, device=emb.device)
    e = emb.float()
    for at in range(0, n, block):
        sim[at : at + block] = 1.0 / (1.0 + torch.cdist(e[at : at + block], e))
    return sim


@torch.no_grad()
def lazy_greedy(sim: torch.Tensor, budget: int, recheck: int = 64) -> list[int]:
    """sim [n, n] (row i: how well each j represents i).  Returns the selected column indices in order."""
    n = sim.size(0)
    best = torch.zeros(n, device=sim.device)  # current coverage of every item
    bounds = sim.sum(0)  # marginal gains against the empty set: valid upper bounds forever (submodularity)
    chosen: list[int] = []
    alive = torch.ones(n, dtype=torch.bool, device=sim.device)
    for _ in range(min(budget, n)):
        while True:
            cand = torch.topk(torch.where(alive, bounds, torch.full_like(bounds, -1.0)), min(recheck, n)).indices
            fresh = torch.relu(sim[:, cand] - best[:, None]).sum(0)
            bounds[cand] = fresh
            top = int(cand[fresh.argmax()])
            # accept when the refreshed best still beats every stale bound outside the refreshed set
            outside = torch.where(alive, bounds, torch.full_like(bounds, -1.0)).clone()
            outside[cand] = -1.0
            if float(fresh.max()) >= float(outside.max()) - 1e-12:
                break
        chosen.append(top)
        alive[top] = False
        best = torch.maximum(best, sim[:, top])
    return chosen


def main(argv=None):
    p = argparse.ArgumentParser(description="Subset embeddings with facility location")
    p.add_argument("--data-file", required=True)
    p.add_argument("--start", type=int, default=0)
    p.add_argument("--end", type=int, default=None)
    p.add_argument("--select-frac", type=float, default=0.8)
    p.add_argument("--output-file", type=Path, required=True)
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = p.parse_args(argv)
    rows = read_rows(a.data_file)[a.start : a.end]
    emb = torch.from_numpy(np.asarray([r["embedding"] for r in rows], dtype=np.float32)).to(a.device)
    picked = lazy_greedy(similarity(emb), int(a.select_frac * len(rows)))
    print(f"selected {len(picked)} of {len(rows)}")
    write_rows(a.output_file, [rows[i] for i in picked])


if __name__ == "__main__":
    main()
