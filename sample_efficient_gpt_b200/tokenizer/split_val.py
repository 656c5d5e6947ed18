"""Carve a validation set off the front of a tokenised dataset at a document boundary
(tokenizer/split_val.py:19-45 of the reference): the first ~``--val-tokens`` tokens of the first ``.npy`` file go to
``<save-dir>/<filename>`` (plus ``offsets_<filename>``), the source file and its offsets are shortened in place."""

from __future__ import annotations

import os
from argparse import ArgumentParser
from bisect import bisect_right
from pathlib import Path

import numpy as np


def split_validation(tokenized_dir: Path, save_dir: Path, filename: str = "val.npy", val_tokens: int = 20_000_000) -> int:
    save_dir.mkdir(exist_ok=True, parents=True)
    files = sorted(f for f in tokenized_dir.glob("*.npy") if "offsets_" not in f.stem)
    base = files[0].stem
    tokens = np.load(tokenized_dir / f"{base}.npy", mmap_mode="r")
    offsets = np.load(tokenized_dir / f"offsets_{base}.npy")
    cut_doc = max(bisect_right(offsets, val_tokens) - 1, 0)
    cut_tok = int(offsets[cut_doc])
    np.save(save_dir / filename, np.asarray(tokens[:cut_tok]))
    np.save(save_dir / f"offsets_{filename}", offsets[: cut_doc + 1])
    # the source is memory-mapped: write the remainder next to it and swap the files afterwards
    tmp_tok, tmp_off = tokenized_dir / f"{base}_temp.npy", tokenized_dir / f"offsets_{base}_temp.npy"
    np.save(tmp_tok, np.array(tokens[cut_tok:], copy=True))
    np.save(tmp_off, offsets[cut_doc:] - cut_tok)
    del tokens
    os.replace(tmp_tok, tokenized_dir / f"{base}.npy")
    os.replace(tmp_off, tokenized_dir / f"offsets_{base}.npy")
    return cut_tok


if __name__ == "__main__":
    p = ArgumentParser()
    p.add_argument("--tokenized-data-path", type=Path, required=True)
    p.add_argument("--save-dir", type=Path, required=True)
    p.add_argument("--filename", default="val.npy")
    p.add_argument("--val-tokens", type=int, default=20_000_000)
    a = p.parse_args()
    print(f"moved {split_validation(a.tokenized_data_path, a.save_dir, a.filename, a.val_tokens)} tokens to {a.save_dir / a.filename}")
