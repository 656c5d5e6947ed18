"""Byte-pair-encoding trainer.

``BPE(special_tokens, vocab_size).train(path)`` pre-tokenises the file, learns merges and stores ``vocab.pickle``
(``{id: bytes}``: 256 bytes, then the special tokens, then the merges in order) and ``merges.pickle``
(``[(left bytes, right bytes)]``), the layout of tokenizer/train_bpe.py:24-665 of the reference.  The merge loop
runs in the native trainer by default (``use_native=True``, the reference's ``--use-rust-bpe`` path) or in the
pure-Python incremental trainer below, which is also the oracle the native one is tested against: the most
frequent pair wins, ties go to the largest ``(left bytes, right bytes)`` tuple.  ``resume_train`` continues from
saved pickles, optionally as a SuperBPE second stage whose merges may span pre-token boundaries inside a document.
"""

from __future__ import annotations

import heapq
import pickle
import time
from argparse import ArgumentParser
from collections import defaultdict
from pathlib import Path

import regex as re

from sample_efficient_gpt_b200.tokenizer.pretokenization import Splitter, pre_tokenize
from sample_efficient_gpt_b200.utils.logger import logger

PAT_STR = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""
PAT = re.compile(PAT_STR)


class _RevBytes:
    """Orders heap entries so that the *largest* (left, right) byte tuple pops first among equal counts."""

    __slots__ = ("k",)

    def __init__(self, k):
        self.k = k

    def __lt__(self, other):
        return self.k > other.k


def train_merges_python(words: list[list[int]], counts: list[int], token_bytes: list[bytes], num_merges: int):
    """Incremental merge loop on id sequences; returns [(left id, right id)] and extends ``token_bytes`` in place."""
    pair_counts: dict[tuple[int, int], int] = defaultdict(int)
    where: dict[tuple[int, int], set[int]] = defaultdict(set)
    for wi, (ids, c) in enumerate(zip(words, counts)):
        for p in zip(ids, ids[1:]):
            pair_counts[p] += c
            where[p].add(wi)
    heap = [(-c, _RevBytes((token_bytes[p[0]], token_bytes[p[1]])), p) for p, c in pair_counts.items() if c > 0]
    heapq.heapify(heap)
    merges = []
    while len(merges) < num_merges and heap:
        negc, _, pair = heapq.heappop(heap)
        cur = pair_counts.get(pair, 0)
        if -negc != cur:
            if cur > 0:
                heapq.heappush(heap, (-cur, _RevBytes((token_bytes[pair[0]], token_bytes[pair[1]])), pair))
            continue
        if cur <= 0:
            break
        a, b = pair
        new_id = len(token_bytes)
        token_bytes.append(token_bytes[a] + token_bytes[b])
        merges.append(pair)
        touched = where.pop(pair, set())
        created = set()
        for wi in touched:
            ids, c = words[wi], counts[wi]
            out, i, n = [], 0, len(ids)
            while i < n:
                if i + 1 < n and ids[i] == a and ids[i + 1] == b:
                    if out:
                        pair_counts[(out[-1], a)] -= c
                        pair_counts[(out[-1], new_id)] += c
                        where[(out[-1], new_id)].add(wi)
                        created.add((out[-1], new_id))
                    pair_counts[pair] -= c
                    if i + 2 < n:
                        pair_counts[(b, ids[i + 2])] -= c
                        pair_counts[(new_id, ids[i + 2])] += c
                        where[(new_id, ids[i + 2])].add(wi)
                        created.add((new_id, ids[i + 2]))
                    out.append(new_id)
                    i += 2
                else:
                    out.append(ids[i])
                    i += 1
            words[wi] = out
        for p in created:
            c = pair_counts.get(p, 0)
            if c > 0:
                heapq.heappush(heap, (-c, _RevBytes((token_bytes[p[0]], token_bytes[p[1]])), p))
    return merges


class BPE:
    def __init__(self, special_tokens: list[str], vocab_size: int = 355, save_every: int = 10000, save_dir: str = "."):
        self.vocab_size = vocab_size
        self.special_tokens = special_tokens
        self.special_tokens_bytes = [x.encode() for x in special_tokens]
        self.splitter = Splitter("<|endoftext|>")
        self.vocab: dict[int, bytes] = {i: bytes([i]) for i in range(256)}
        for i, s in enumerate(self.special_tokens_bytes):
            self.vocab[256 + i] = s
        self.merges_tuples: list[tuple[bytes, bytes]] = []
        self.save_dir = Path(save_dir)
        self.save_dir.mkdir(exist_ok=True, parents=True)
        self.save_every = save_every
        self.vocab_name, self.merges_name = "vocab.pickle", "merges.pickle"

    @property
    def cur_vocab_size(self) -> int:
        return len(self.vocab)

    def _install(self, merges_bytes: list[tuple[bytes, bytes]]):
        next_id = 256 + len(self.special_tokens_bytes) + len(self.merges_tuples)
        for l, r in merges_bytes:
            self.vocab[next_id] = l + r
            self.merges_tuples.append((l, r))
            next_id += 1

    def train(self, filepath: str, num_processes: int = 1, use_native: bool = True):
        t0 = time.monotonic()
        counts = pre_tokenize(self.splitter, str(filepath), num_processes=num_processes)
        logger.info(f"Pre-tokenization finished in {time.monotonic() - t0:.1f} s, {len(counts)} distinct pre-tokens")
        return self.train_from_counts(counts, use_native)

    def train_from_counts(self, counts: dict[str, int], use_native: bool = True):
        target_no_specials = self.vocab_size - len(self.special_tokens)
        assert target_no_specials >= 256
        pre = [(k.encode("utf-8"), v) for k, v in counts.items()]
        if use_native:
            from sample_efficient_gpt_b200.tokenizer.cppbpe import Tokenizer as NativeBPE

            nt = NativeBPE()
            nt.train_from_pretokens(pre, target_no_specials)
            merges_bytes = nt.export_merges_bytes()
        else:
            token_bytes = [bytes([i]) for i in range(256)]
            words = [list(b) for b, _ in pre]
            merges = train_merges_python(words, [c for _, c in pre], token_bytes, target_no_specials - 256)
            merges_bytes = [(token_bytes[a], token_bytes[b]) for a, b in merges]
        self._install(merges_bytes)
        self.save()
        return self.vocab, self.merges_tuples

    def resume_train(self, tokenized_docs: list[list[int]], vocab_size: int, superbpe: bool = True):
        """Learn further merges on already tokenised documents (ids of the current vocabulary).

        With ``superbpe`` the sequences are whole documents, so new tokens may cross the pre-token boundaries of the
        first stage; special tokens never take part in a merge."""
        n_new = vocab_size - self.cur_vocab_size
        if n_new <= 0:
            return self.vocab, self.merges_tuples
        max_id = max(self.vocab) + 1
        token_bytes = [self.vocab.get(i, b"") for i in range(max_id)]
        specials = set(range(256, 256 + len(self.special_tokens)))
        words, counts = [], []
        for doc in tokenized_docs:
            seg: list[int] = []
            for t in doc:
                if t in specials:
                    if len(seg) > 1:
                        words.append(seg)
                        counts.append(1)
                    seg = []
                else:
                    seg.append(int(t))
            if len(seg) > 1:
                words.append(seg)
                counts.append(1)
        merges = train_merges_python(words, counts, token_bytes, n_new)
        self._install([(token_bytes[a], token_bytes[b]) for a, b in merges])
        self.vocab_size = vocab_size
        self.save()
        return self.vocab, self.merges_tuples

    def save(self):
        (self.save_dir / self.vocab_name).write_bytes(pickle.dumps(self.vocab))
        (self.save_dir / self.merges_name).write_bytes(pickle.dumps(self.merges_tuples))

    @classmethod
    def load(cls, save_dir: str, special_tokens: list[str]) -> "BPE":
        vocab = pickle.loads((Path(save_dir) / "vocab.pickle").read_bytes())
        merges = pickle.loads((Path(save_dir) / "merges.pickle").read_bytes())
        obj = cls(special_tokens, vocab_size=len(vocab), save_dir=save_dir)
        obj.vocab, obj.merges_tuples = vocab, merges
        return obj


def parse_args():
    p = ArgumentParser(description="Train a byte-level BPE tokenizer")
    p.add_argument("--data-path", required=True)
    p.add_argument("--vocab-size", type=int, default=32000)
    p.add_argument("--save-dir", default="tokenizer_out")
    p.add_argument("--num-processes", type=int, default=8)
    p.add_argument("--use-rust-bpe", "--use-native-bpe", dest="use_native", type=int, default=1)
    p.add_argument("--n-reserved", type=int, default=20)
    return p.parse_args()


if __name__ == "__main__":
    a = parse_args()
    specials = ["<|endoftext|>"] + [f"<|reserved_{i}|>" for i in range(a.n_reserved)]
    bpe = BPE(specials, vocab_size=a.vocab_size, save_dir=a.save_dir)
    t0 = time.monotonic()
    bpe.train(a.data_path, num_processes=a.num_processes, use_native=bool(a.use_native))
    logger.info(f"trained {len(bpe.merges_tuples)} merges in {time.monotonic() - t0:.1f} s -> {a.save_dir}")
