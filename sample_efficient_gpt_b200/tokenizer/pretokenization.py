"""Chunked, parallel pre-tokenisation of a text file (tokenizer/pretokenization.py:13-90 of the reference).

``find_chunk_boundaries`` cuts a file into pieces that end on a delimiter (so no pre-token straddles two pieces),
``pre_tokenize`` counts pre-tokens of all pieces with the native ``Splitter`` (GIL released, so plain threads scale).
"""

from __future__ import annotations

import os
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import BinaryIO

from sample_efficient_gpt_b200.tokenizer.fastsplit import Splitter


def find_chunk_boundaries(file: BinaryIO, desired_num_chunks: int, split_special_token: bytes) -> list[int]:
    """Byte offsets (sorted, unique) of at most ``desired_num_chunks`` pieces, each starting at a delimiter."""
    assert isinstance(split_special_token, bytes), "Must represent special token as a bytestring"
    file.seek(0, os.SEEK_END)
    size = file.tell()
    step = size // desired_num_chunks
    bounds = [i * step for i in range(desired_num_chunks + 1)]
    bounds[-1] = size
    probe = 4096
    for bi in range(1, len(bounds) - 1):
        pos = bounds[bi]
        file.seek(pos)
        while True:
            buf = file.read(probe)
            if buf == b"":
                bounds[bi] = size
                break
            hit = buf.find(split_special_token)
            if hit != -1:
                bounds[bi] = pos + hit
                break
            pos += probe
    return sorted(set(bounds))


def pre_tokenize(splitter: Splitter, filepath: str, num_processes: int = 1, special_token: str = "<|endoftext|>") -> dict[str, int]:
    if num_processes > 1 and hasattr(splitter, "count_file"):
        return splitter.count_file(str(filepath), num_processes)  # native threads, one dict at the end
    with Path(filepath).open("rb") as fh:
        bounds = find_chunk_boundaries(fh, num_processes * 4, special_token.encode())
    spans = list(zip(bounds[:-1], bounds[1:]))
    total: dict[str, int] = {}

    def merge(part: dict[str, int]):
        for k, v in part.items():
            total[k] = total.get(k, 0) + v

    if num_processes > 1:
        with ThreadPoolExecutor(num_processes) as pool:
            for part in pool.map(lambda se: splitter.seek_and_split(str(filepath), se[0], se[1]), spans):
                merge(part)
    else:
        for s, e in spans:
            merge(splitter.seek_and_split(str(filepath), s, e))
    return total


if __name__ == "__main__":
    import sys

    t0 = time.monotonic()
    counts = pre_tokenize(Splitter("<|endoftext|>"), sys.argv[1], num_processes=int(sys.argv[2]) if len(sys.argv) > 2 else 1)
    print(f"{len(counts)} distinct pre-tokens in {time.monotonic() - t0:.2f}s")
