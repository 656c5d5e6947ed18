"""BPE encoder / decoder over the pickled vocabulary and merges (tokenizer/tokenizer.py:104-351 of the reference).

``encode`` splits on special tokens, pre-tokenises each piece with the native scanner, and merges every pre-token
lowest-rank-first (cached per distinct pre-token).  With ``superbpe_transition_idx`` the merges from that index on form
a second stage that is applied across pre-token boundaries of a piece.  The CLI measures bytes/token on validation
text and writes uint16 ``.npy`` token files.
"""

from __future__ import annotations

import json
import math
import pickle
import time
from argparse import ArgumentParser
from functools import lru_cache
from pathlib import Path

import numpy as np
import regex as re

from sample_efficient_gpt_b200.utils.logger import logger


def merge_by_rank(ids: list[int], ranks: dict[tuple[int, int], int], merge_map: dict[tuple[int, int], int]) -> list[int]:
    """Repeatedly merge the adjacent pair of lowest rank (leftmost on ties) until none is mergeable."""
    while len(ids) >= 2:
        best, best_i = None, -1
        for i, p in enumerate(zip(ids, ids[1:])):
            r = ranks.get(p)
            if r is not None and (best is None or r < best):
                best, best_i = r, i
        if best is None:
            break
        p = (ids[best_i], ids[best_i + 1])
        new_id = merge_map[p]
        out, i = [], 0
        while i < len(ids):  # merge every occurrence of that pair, left to right
            if i + 1 < len(ids) and (ids[i], ids[i + 1]) == p:
                out.append(new_id)
                i += 2
            else:
                out.append(ids[i])
                i += 1
        ids = out
    return ids


class Tokenizer:
    def __init__(self, vocab: dict[int, bytes], merges: list[tuple[bytes, bytes]], special_tokens: list[str] | None = None,
                 superbpe_transition_idx: int | None = None, use_native: bool = True):
        from sample_efficient_gpt_b200.tokenizer.fastsplit import Splitter

        self.special_tokens = special_tokens or []
        self.vocab = vocab
        self.byte2int = {v: k for k, v in vocab.items()}
        self.lut256 = [self.byte2int[bytes([b])] for b in range(256)]
        toks = sorted(self.special_tokens, reverse=True) or ["<|endoftext|>"]
        self.split_re = "(" + "|".join(re.escape(t) for t in toks) + ")"
        self._split = re.compile(self.split_re)
        self._scanner = Splitter("")
        self.superbpe_transition_idx = superbpe_transition_idx
        second = []
        if superbpe_transition_idx is not None:
            merges, second = merges[:superbpe_transition_idx], merges[superbpe_transition_idx:]
        self.merge_map, self.bpe_ranks = self._init_merge_map(merges, 0)
        self.merge_map_superbpe, self.bpe_ranks_superbpe = self._init_merge_map(second, len(merges))
        self._cached = lru_cache(maxsize=2_000_000)(self._encode_bytes)
        # native encoder (tokenizer/csrc/segtok.cpp::Encoder): same merges, same order; the Python statements below stay as
        # the fallback and as its oracle (``use_native=False``)
        self.use_native = use_native
        self._native = None
        if use_native:
            from sample_efficient_gpt_b200.tokenizer.fastsplit import _mod

            if hasattr(_mod, "Encoder"):
                as_rows = lambda mm, rk: [(l, r, mm[(l, r)], rk[(l, r)]) for (l, r) in sorted(rk, key=rk.get)]  # noqa: E731
                self._native = _mod.Encoder(self.lut256, as_rows(self.merge_map, self.bpe_ranks),
                                            as_rows(self.merge_map_superbpe, self.bpe_ranks_superbpe))

    def _init_merge_map(self, merges, base_rank):
        merge_map, ranks = {}, {}
        for rank, (l, r) in enumerate(merges):
            new_id = self.byte2int.get(l + r)
            if new_id is None or l not in self.byte2int or r not in self.byte2int:
                continue
            pair = (self.byte2int[l], self.byte2int[r])
            merge_map[pair] = new_id
            ranks[pair] = base_rank + rank
        return merge_map, ranks

    @classmethod
    def from_files(cls, vocab_filepath, merges_filepath, special_tokens=None, superbpe_transition_idx=None):
        return cls(pickle.loads(Path(vocab_filepath).read_bytes()), pickle.loads(Path(merges_filepath).read_bytes()),
                   special_tokens, superbpe_transition_idx)

    def _encode_bytes(self, tok_bytes: bytes) -> tuple[int, ...]:
        return tuple(merge_by_rank([self.lut256[b] for b in tok_bytes], self.bpe_ranks, self.merge_map))

    def encode(self, text: str) -> list[int]:
        out: list[int] = []
        for piece in self._split.split(text):
            if not piece:
                continue
            if piece in self.special_tokens:
                out.append(self.byte2int[piece.encode()])
                continue
            if self._native is not None:
                out.extend(self._native.encode_ordinary(piece))
                continue
            ids: list[int] = []
            for tok in self._scanner.pretokens(piece):
                ids.extend(self._cached(tok.encode("utf-8")))
            if self.superbpe_transition_idx is not None:
                ids = merge_by_rank(ids, self.bpe_ranks_superbpe, self.merge_map_superbpe)
            out.extend(ids)
        return out

    def encode_batch(self, texts: list[str], threads: int = 8) -> list[list[int]]:
        """Many documents at once; with the native encoder the ordinary pieces of all of them are encoded on native threads."""
        if self._native is None:
            return [self.encode(t) for t in texts]
        plans, pieces = [], []
        for text in texts:
            plan = []
            for piece in self._split.split(text):
                if not piece:
                    continue
                if piece in self.special_tokens:
                    plan.append(self.byte2int[piece.encode()])
                else:
                    plan.append(None)
                    pieces.append(piece)
            plans.append(plan)
        encoded = iter(self._native.encode_batch(pieces, threads))
        outs = []
        for plan in plans:
            ids: list[int] = []
            for item in plan:
                if item is None:
                    ids.extend(next(encoded))
                else:
                    ids.append(item)
            outs.append(ids)
        return outs

    def encode_iterable(self, iterable):
        for line in iterable:
            yield from self.encode(line)

    def encode_file(self, filepath, chunk_size: int = 1024 * 1024, threads: int = 8) -> list[int]:
        from sample_efficient_gpt_b200.tokenizer.pretokenization import find_chunk_boundaries

        path = Path(filepath)
        n_chunks = max(1, math.ceil(path.stat().st_size / chunk_size))
        with path.open("rb") as f:
            bounds = find_chunk_boundaries(f, n_chunks, b" ")
            tokens: list[int] = []
            spans = list(zip(bounds[:-1], bounds[1:]))
            group = 64 if self._native is not None else 1  # chunks encoded together on native threads
            for g0 in range(0, len(spans), group):
                texts = []
                for s, e in spans[g0 : g0 + group]:
                    f.seek(s)
                    texts.append(f.read(e - s).decode("utf-8", errors="ignore"))
                for ids in self.encode_batch(texts, threads=threads):
                    tokens.extend(ids)
        return tokens

    def decode(self, ids) -> str:
        if not isinstance(ids, (list, tuple)):
            ids = [ids]
        return b"".join(self.vocab.get(i, b"") if isinstance(i, int) else i for i in ids).decode("utf-8", errors="replace")


def parse_args():
    p = ArgumentParser()
    p.add_argument("--vocab-path", required=True)
    p.add_argument("--merges-path", required=True)
    p.add_argument("--data-path", required=True, help="folder with *train*.txt / *val*.txt")
    p.add_argument("--tokenized-data-path", required=True)
    p.add_argument("--superbpe-transition-idx", default=None, type=int)
    p.add_argument("--stats-name", default="stats.json")
    p.add_argument("--include-val-data", default=0, type=int)
    return p.parse_args()


if __name__ == "__main__":
    a = parse_args()
    tok = Tokenizer.from_files(a.vocab_path, a.merges_path, ["<|endoftext|>"], a.superbpe_transition_idx)
    src = Path(a.data_path)
    ratios = {}
    for f in src.glob("*val*.txt"):
        rs = [len(d.encode()) / max(1, len(tok.encode(d))) for d in re.split(tok.split_re, f.read_text())[:200]
              if d and d != "<|endoftext|>"]
        ratios[f.name] = float(np.mean(rs)) if rs else 0.0
        print(f"{f.name} compression ratio: {ratios[f.name]:.2f}")
    (src / a.stats_name).write_text(json.dumps(ratios))
    dst = Path(a.tokenized_data_path)
    dst.mkdir(exist_ok=True, parents=True)
    files = list(src.glob("*train*.txt")) + (list(src.glob("*val*.txt")) if a.include_val_data == 1 else [])
    for fp in files:
        t0 = time.monotonic()
        ids = tok.encode_file(fp, chunk_size=8 * 1024 * 1024)
        dt = time.monotonic() - t0
        logger.info(f"{fp}: {dt:.1f} s, {fp.stat().st_size / 2**20 / dt:.2f} MB/s")
        np.save(str((dst / fp.name).with_suffix(".npy")), np.array(ids, dtype="uint16"))
