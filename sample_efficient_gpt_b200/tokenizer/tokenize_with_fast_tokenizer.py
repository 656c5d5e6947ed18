"""Dataset tokeniser: parquet / jsonl.gz / txt corpora -> ``uint16`` token shards + ``int64`` document offsets.

Same outputs and rules as tokenizer/tokenize_with_fast_tokenizer.py:22-356 of the reference: per-dataset quality-score
thresholds chosen by the ``STAGE`` environment variable (1, 2 or 3), ``<|endoftext|>`` appended to every document,
stage-3 chat wrapping (``<|bos|>...`` and the ``\\n<think>`` query/response split) with a 4000-character minimum,
``<name>.npy`` + ``offsets_<name>.npy`` per input file (document i is ``tokens[offsets[i]:offsets[i+1]]``), finished
shards skipped, optional token ``--limit``.  Files are read with pyarrow / gzip directly and encoded in batches by the
fast tokenizer (which threads internally); no dataset-library cache is involved.
"""

from __future__ import annotations

import gzip
import json
import logging
import math
import os
import time
from argparse import ArgumentParser
from pathlib import Path

import numpy as np

from sample_efficient_gpt_b200.tokenizer.pretokenization import find_chunk_boundaries

logger = logging.getLogger(__name__)

EOT = "<|endoftext|>"
STAGE3_LENGTH_THRESHOLD = 4000  # characters

#            dataset tag                     stage 1  stage 2  stage 3
THRESHOLDS = {
    "cosmopedia": (2.0, 2.3, 2.5),
    "finemath": (3.7, 4.1, 4.25),
    "dclm_edu": (2.75, 3.2, 3.2),
    "stack_edu": (3.75, 4.1, 4.25),
    "finepdfs": (1.75, 2.1, 2.4),
    "pleias_synth": (1.65, 1.85, 2.1),
}
# path substring -> (threshold tag, how to read the score of a row)
SCORE_RULES = [
    ("dclm-edu", "dclm_edu", lambda r: r["metadata"]["edu_score"]),
    ("finemath", "finemath", lambda r: r["score"]),
    ("cosmopedia-v2-textbook-7b", "cosmopedia", lambda r: r["score"]),
    ("stack_edu_375plus_20B", "stack_edu", lambda r: r["score"]),
    ("finepdfs_en_2020plus_edu", "finepdfs", lambda r: r["score"]),
    ("finepdfs-edu", "finepdfs", lambda r: min(r["metadata"]["fw_edu_scores"])),
    ("pleias_synth", "pleias_synth", lambda r: r["score"]),
]


def current_stage() -> int:
    s = int(os.getenv("STAGE", "1"))
    return s if s in (2, 3) else 1


def threshold(tag: str, stage: int | None = None) -> float:
    return THRESHOLDS[tag][(stage or current_stage()) - 1]


class TokenizerProcessor:
    def __init__(self, tokenizer_name, special_tokens=(EOT,), batch_size: int = 2048):
        from transformers import PreTrainedTokenizerFast

        self.tok = tokenizer_name if hasattr(tokenizer_name, "encode") else PreTrainedTokenizerFast.from_pretrained(tokenizer_name)
        self.special_tokens = list(special_tokens)
        self.batch_size = batch_size
        import regex as re

        escaped = [re.escape(t) for t in sorted(self.special_tokens, reverse=True)] or [re.escape(EOT)]
        self.split_re = re.compile(f"({'|'.join(escaped)})")

    # ---- text rules -------------------------------------------------------------------------------------------------
    def preprocess_text(self, text: str) -> str:
        if current_stage() == 3:
            if "\n<think>" in text:
                at = text.index("\n<think>")
                return f"<|bos|><|user_start|>{text[:at]}<|user_end|><|assistant_start|>{text[at:]}<|assistant_end|>{EOT}"
            return f"<|bos|>{text}{EOT}"
        return f"{text}{EOT}"

    def keep_row(self, row: dict, source: str) -> bool:
        for tag, name, score in SCORE_RULES:
            if tag in source and not score(row) > threshold(name):
                return False
        return not (current_stage() == 3 and len(row["text"]) <= STAGE3_LENGTH_THRESHOLD)

    # ---- encoding ---------------------------------------------------------------------------------------------------
    def encode_docs(self, docs: list[str]) -> tuple[np.ndarray, np.ndarray]:
        """Flat uint16 tokens and int64 offsets (len(docs)+1)."""
        pieces, lens = [], []
        for at in range(0, len(docs), self.batch_size):
            ids = self.tok(docs[at : at + self.batch_size], add_special_tokens=True)["input_ids"]
            lens.extend(len(x) for x in ids)
            pieces.extend(np.asarray(x, dtype=np.int64) for x in ids)
        flat = np.concatenate(pieces) if pieces else np.zeros(0, dtype=np.int64)
        if flat.size and flat.max() >= (1 << 16):
            raise ValueError("Token ids exceed uint16 range; choose uint32 instead.")
        offsets = np.zeros(len(lens) + 1, dtype=np.int64)
        np.cumsum(lens, out=offsets[1:])
        return flat.astype(np.uint16), offsets

    def _rows_to_shard(self, rows, source: str, out_path: Path, offsets_path: Path, filtered: bool, wrapped: bool) -> int:
        docs = []
        for row in rows:
            if filtered and not self.keep_row(row, source):
                continue
            docs.append(self.preprocess_text(row["text"]) if wrapped else row["text"])
        tokens, offsets = self.encode_docs(docs)
        np.save(str(out_path), tokens)
        np.save(str(offsets_path), offsets)
        return int(tokens.shape[0])

    def encode_hf(self, filepath, tokenized_path, limit: int = -1) -> int:
        """Parquet files (recursively) or ``*.jsonl.gz`` files (in groups of 50) under ``filepath``."""
        path, tokenized_path = Path(filepath), Path(tokenized_path)
        tokenized_path.mkdir(parents=True, exist_ok=True)
        count = 0
        parquet = sorted(path.glob("**/*.parquet"))
        if parquet:
            jobs = [([p], "".join(p.name.split(".")[:-1]), p.stem) for p in parquet]
        else:
            files = sorted(path.glob("*.jsonl.gz"))
            jobs = [(files[i : i + 50], str(i // 50), str(i // 50)) for i in range(0, len(files), 50)]
        for members, name, offsets_name in jobs:
            out_path = (tokenized_path / name).with_suffix(".npy")
            if out_path.exists():
                if limit > 0:
                    count += np.load(str(out_path), mmap_mode="r").shape[0]
                logger.info(f"{out_path} exists, skipping")
                continue
            if limit > 0 and count > limit:
                logger.info("reached limit")
                break
            source = str(members[0])
            chat = "all_chat" in source
            try:
                rows = list(self._read_rows(members))
            except (OSError, ValueError, json.JSONDecodeError) as e:
                logger.info(f"error while reading {source} ({e}); skipping")
                continue
            count += self._rows_to_shard(rows, source, out_path, tokenized_path / f"offsets_{offsets_name}.npy",
                                         filtered=not chat, wrapped=not chat and "the_stack_v2_" not in source)
            logger.info(f"current count: {count}")
        return count

    @staticmethod
    def _read_rows(files):
        for f in files:
            if f.suffix == ".parquet":
                import pyarrow.parquet as pq

                yield from pq.read_table(f).to_pylist()
            else:
                with gzip.open(f, "rt", encoding="utf-8") as fh:
                    for line in fh:
                        if line.strip():
                            yield json.loads(line)

    # ---- plain text files ---------------------------------------------------------------------------------------------
    def _split_text_file(self, filepath, chunk_size: int = 32 * 1024 * 1024):
        path = Path(filepath)
        n_chunks = max(1, math.ceil(path.stat().st_size / chunk_size))
        with path.open("rb") as f:
            bounds = find_chunk_boundaries(f, n_chunks, b" ")
            for start, end in zip(bounds[:-1], bounds[1:]):
                f.seek(start)
                yield f.read(end - start).decode("utf-8", errors="ignore")

    def _process_text_chunk(self, text: str) -> list[str]:
        return [doc + EOT for doc in self.split_re.split(text) if doc and doc not in self.special_tokens]

    def encode(self, text: str):
        return self.encode_docs(self._process_text_chunk(text))

    def encode_file(self, filepath, tokenized_path, chunk_size: int = 32 * 1024 * 1024) -> np.ndarray:
        out = Path(tokenized_path) / (Path(filepath).stem + ".npy")
        parts = []
        for i, chunk in enumerate(self._split_text_file(filepath, chunk_size)):
            parts.append(self.encode(chunk)[0])
            if (i + 1) % 5 == 0:  # periodic save of the partial result
                np.save(str(out), np.concatenate(parts))
        tokens = np.concatenate(parts) if parts else np.zeros(0, dtype=np.uint16)
        np.save(str(out), tokens)
        return tokens

    def encode_hf_txt(self, filepath, tokenized_path, chunk_size: int = 128 * 1024 * 1024):
        filepath = Path(filepath)
        for txt in list(filepath.glob("*val*.txt")) + list(filepath.glob("*train*.txt")):
            self.encode_file(txt, tokenized_path, chunk_size)

    def compression_ratios(self, input_dir: Path, sample_docs: int = 200) -> dict[str, float]:
        """Bytes per token over the first documents of every ``*val*.txt``."""
        out = {}
        for f in Path(input_dir).glob("*val*.txt"):
            ratios = []
            for doc in self.split_re.split(f.read_text())[:sample_docs]:
                if doc and doc != EOT:
                    n_tokens = len(self.encode(doc)[0])
                    if n_tokens:
                        ratios.append(len(doc.encode()) / n_tokens)
            out[f.name] = float(np.mean(ratios)) if ratios else 0.0
            logger.info(f"{f.name} compression ratio: {out[f.name]:.2f}")
        return out


def parse_args(argv=None):
    p = ArgumentParser()
    p.add_argument("--tokenizer-name", required=True)
    p.add_argument("--data-path", required=True)
    p.add_argument("--tokenized-data-path", required=True)
    p.add_argument("--stats-name", default="stats.json")
    p.add_argument("--include-val-data", default=0, type=int)
    p.add_argument("--is-hf", default=1, type=int, help="1: parquet/jsonl.gz (or txt) shards; 0: txt with compression stats")
    p.add_argument("--limit", default=-1, type=int)
    return p.parse_args(argv)


def main(argv=None):
    logging.basicConfig(level=logging.INFO)
    a = parse_args(argv)
    proc = TokenizerProcessor(a.tokenizer_name, special_tokens=[EOT])
    src, dst = Path(a.data_path), Path(a.tokenized_data_path)
    dst.mkdir(parents=True, exist_ok=True)
    t0 = time.monotonic()
    has_txt = bool(list(src.glob("*train*.txt")))
    if a.is_hf and not has_txt:
        proc.encode_hf(src, dst, limit=a.limit)
    elif a.is_hf:
        proc.encode_hf_txt(src, dst)
    else:
        (src / a.stats_name).write_text(json.dumps(proc.compression_ratios(src)))
        files = list(src.glob("*train.txt")) + (list(src.glob("*val*.txt")) if a.include_val_data == 1 else [])
        for f in files:
            t1 = time.monotonic()
            proc.encode_file(f, dst, chunk_size=128 * 1024 * 1024)
            dt = time.monotonic() - t1
            logger.info(f"Processed {f} in {dt:.1f} s ({f.stat().st_size / 2**20 / max(dt, 1e-9):.2f} MB/s)")
    logger.info(f"Took {time.monotonic() - t0:.1f} s.")


if __name__ == "__main__":
    main()
