"""CPU timings of the native tokenizer tools against their Python statements, on a synthetic corpus (no downloads).

    python -m sample_efficient_gpt_b200.tokenizer.bench_tokenizer --mb 64 --vocab-size 4096 --threads 8

  * pre-tokenisation: the C++ scanner (``Splitter.seek_and_split``, one and several threads) against ``regex.findall`` with
    the same pattern plus a Python ``Counter`` (what the reference's pure-Python path does, tokenizer/pretokenization.py);
  * encoding with the learned vocabulary: the Python merge loop with its cache against the native encoder
    (``tokenizer/csrc/segtok.cpp::Encoder``), one thread and several; the ids must be identical;
  * BPE training on the resulting pre-token counts: the C++ incremental trainer (the stand-in for the reference's Rust
    ``rustbpe``) against the Python merge loop (``train_merges_python``: the reference's optimised loop with the sort
    heuristic, tokenizer/train_bpe.py:168 there).  Both must produce the same merges.
The corpus is Zipf-distributed pseudo-words with punctuation, digits, contractions, a few non-ASCII words and document
separators, so the pre-token statistics have the long tail that real text has.
"""

from __future__ import annotations

import argparse
import json
import random
import tempfile
import time
from collections import Counter
from pathlib import Path


def make_corpus(path: Path, mb: int, seed: int = 0) -> int:
    import numpy as np

    rnd = random.Random(seed)
    rng = np.random.default_rng(seed)
    letters = "etaoinshrdlcumwfgypbvkjxqz"
    words = ["".join(rnd.choice(letters) for _ in range(rnd.randint(1, 11))) for _ in range(60000)]
    words += ["naïve", "façade", "Übung", "señor", "データ", "模型", "привет", "don't", "it's", "we'll", "I'm", "they've"]
    prob = np.array([1.0 / (i + 1) ** 1.05 for i in range(len(words))])
    prob /= prob.sum()
    seps = [" "] * 79 + [". ", ", ", "; ", "? ", "! ", ":\n", "\n\n", " (", ") ", " - ", "  "] * 2
    target, written = mb << 20, 0
    with path.open("w", encoding="utf-8") as f:
        while written < target:
            n = int(rng.integers(400, 3200))
            idx = rng.choice(len(words), size=n, p=prob)
            caps = rng.random(n) < 0.08
            sep = rng.integers(0, len(seps), size=n)
            nums = rng.random(n) < 0.03
            parts = []
            for i in range(n):
                w = words[idx[i]]
                parts.append(w.capitalize() if caps[i] else w)
                parts.append(f" {int(sep[i]) * 977 % 100000} " if nums[i] else seps[sep[i]])
            doc = "".join(parts) + "<|endoftext|>"
            f.write(doc)
            written += len(doc.encode("utf-8"))
    return written


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--mb", type=int, default=64)
    p.add_argument("--vocab-size", type=int, default=4096)
    p.add_argument("--threads", type=int, default=8)
    p.add_argument("--python-mb", type=int, default=8, help="the Python pre-tokeniser is timed on this many MB only")
    a = p.parse_args()

    from sample_efficient_gpt_b200.tokenizer.cppbpe import Tokenizer as NativeBPE
    from sample_efficient_gpt_b200.tokenizer.fastsplit import Splitter
    from sample_efficient_gpt_b200.tokenizer.pretokenization import pre_tokenize
    from sample_efficient_gpt_b200.tokenizer.train_bpe import PAT, train_merges_python

    out = {"corpus_mb": a.mb}
    with tempfile.TemporaryDirectory() as d:
        path = Path(d) / "corpus.txt"
        nbytes = make_corpus(path, a.mb)
        sp = Splitter("<|endoftext|>")
        t0 = time.monotonic()
        counts = pre_tokenize(sp, str(path), num_processes=1)
        t1 = time.monotonic()
        counts_mt = pre_tokenize(sp, str(path), num_processes=a.threads)
        t2 = time.monotonic()
        assert counts == counts_mt
        out["pretokenize_native_1_thread_mb_s"] = round(nbytes / (t1 - t0) / 2**20, 1)
        out[f"pretokenize_native_{a.threads}_threads_mb_s"] = round(nbytes / (t2 - t1) / 2**20, 1)
        out["distinct_pretokens"] = len(counts)

        text = path.read_bytes()[: a.python_mb << 20].decode("utf-8", errors="ignore")
        t0 = time.monotonic()
        py = Counter()
        for seg in text.split("<|endoftext|>"):
            py.update(PAT.findall(seg))
        t1 = time.monotonic()
        out["pretokenize_python_regex_mb_s"] = round(len(text.encode("utf-8")) / (t1 - t0) / 2**20, 1)

    pre = [(k.encode("utf-8"), v) for k, v in counts.items()]
    target = a.vocab_size
    t0 = time.monotonic()
    nt = NativeBPE()
    nt.train_from_pretokens(pre, target)
    native_merges = nt.export_merges_bytes()
    t1 = time.monotonic()
    token_bytes = [bytes([i]) for i in range(256)]
    merges = train_merges_python([list(b) for b, _ in pre], [c for _, c in pre], token_bytes, target - 256)
    t2 = time.monotonic()
    py_merges = [(token_bytes[x], token_bytes[y]) for x, y in merges]
    out["bpe_merges"] = target - 256
    out["bpe_native_s"] = round(t1 - t0, 3)
    out["bpe_python_s"] = round(t2 - t1, 3)
    out["bpe_speedup"] = round((t2 - t1) / max(t1 - t0, 1e-9), 1)
    out["bpe_same_merges"] = native_merges == py_merges

    # encoding with the learned vocabulary: Python merge loop with its per-pre-token cache, the native encoder, and the
    # native encoder on several threads (documents of the same corpus; the Python path is timed on a slice)
    from sample_efficient_gpt_b200.tokenizer.tokenizer import Tokenizer

    vocab = {i: bytes([i]) for i in range(256)}
    vocab[256] = b"<|endoftext|>"
    for k, (l, r) in enumerate(native_merges):
        vocab[257 + k] = l + r
    docs = [d + "<|endoftext|>" for d in text.split("<|endoftext|>") if d]
    py_tok = Tokenizer(vocab, native_merges, ["<|endoftext|>"], use_native=False)
    na_tok = Tokenizer(vocab, native_merges, ["<|endoftext|>"])
    py_docs = docs[: max(1, len(docs) // 4)]
    t0 = time.monotonic()
    py_ids = [py_tok.encode(d) for d in py_docs]
    t1 = time.monotonic()
    na_ids = [na_tok.encode(d) for d in docs]
    t2 = time.monotonic()
    na_batch = na_tok.encode_batch(docs, threads=a.threads)
    t3 = time.monotonic()
    nb = lambda ds: sum(len(d.encode("utf-8")) for d in ds)  # noqa: E731
    out["encode_python_mb_s"] = round(nb(py_docs) / (t1 - t0) / 2**20, 2)
    out["encode_native_mb_s"] = round(nb(docs) / (t2 - t1) / 2**20, 2)
    out[f"encode_native_{a.threads}_threads_mb_s"] = round(nb(docs) / (t3 - t2) / 2**20, 2)
    out["encode_same_ids"] = na_ids[: len(py_ids)] == py_ids and na_batch == na_ids
    out["bytes_per_token"] = round(nb(docs) / max(1, sum(len(x) for x in na_ids)), 3)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
