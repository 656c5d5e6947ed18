"""Token datasets over memory-mapped ``.npy`` files.

Behaviour follows training/data.py:16-261 of the reference:
  * a path is a single ``.npy`` file, a directory of ``*.npy`` (sorted; names containing ``offsets_``
    are document-offset side files and are skipped) or a JSON ``{directory: token_budget}`` mix that
    takes files from each directory until the budget is exceeded;
  * training batches are windows of ``context_length + 1`` tokens at uniformly random starts drawn
    with ``torch.randint(0, N, (local_bs,), generator=Generator().manual_seed(seed))`` where
    ``N = total_tokens - context_length``; inputs are ``w[:-1]``, targets ``w[1:]``, int32 on the CPU;
  * with ``world_size > 1`` a rank draws only its share ``bs // world (+1 for rank < bs % world)``;
  * ``get_batch`` is served by one prefetch thread that pins the batch for an asynchronous H2D copy;
  * ``get_iterator`` walks a single-file dataset in order (validation), dropping the ragged tail.
A single file is accepted as a training path too (the reference's loader fails on that input).
"""

from __future__ import annotations

import json
import queue
import threading
from collections.abc import Iterator
from pathlib import Path

import numpy as np
import torch
from torch import Tensor

from sample_efficient_gpt_b200.utils.logger import logger


def local_batch_size(batch_size: int, world_size: int, rank: int) -> int:
    if world_size <= 1:
        return batch_size
    if batch_size < world_size:
        raise ValueError(f"batch_size ({batch_size}) must be >= world_size ({world_size}).")
    return batch_size // world_size + (1 if rank < batch_size % world_size else 0)


class MemoryMappedDataset:
    def __init__(
        self,
        path_or_ds: str | Path | np.ndarray,
        context_length: int,
        device: str | torch.device = "cpu",
        seed: int | None = None,
        world_size: int = 1,
        rank: int = 0,
        prefetch: int = 2,
    ):
        self.context_length = context_length
        self.device = device
        self.world_size, self.rank = world_size, rank
        self.is_distributed = world_size > 1
        self.local_batch_size: int | None = None
        self.g = torch.Generator().manual_seed(seed) if seed is not None else None

        self.ds: list[np.ndarray] = []
        if isinstance(path_or_ds, np.ndarray):
            self.ds.append(path_or_ds)
        else:
            path = Path(path_or_ds)
            if path.suffix == ".json":
                mapping = json.loads(path.read_text())
                logger.info(mapping)
                for folder, budget in mapping.items():
                    self.ds.extend(self._read_folder(Path(folder), budget))
            elif path.is_dir():
                self.ds.extend(self._read_folder(path))
            else:
                self.ds.append(np.load(path, mmap_mode="r"))
        sizes = np.array([a.shape[0] for a in self.ds], dtype=np.int64)
        self.chunk_sizes = sizes
        self.chunk_starts = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)  # len = n_chunks + 1
        self.total_length = int(self.chunk_starts[-1])
        assert self.total_length > 0, "dataset is empty"
        self.N = self.total_length - self.context_length
        logger.info(f"Dataset length: {self.total_length}")

        self._span = np.arange(context_length + 1, dtype=np.int64)
        self._queue: queue.Queue | None = None
        self._thread: threading.Thread | None = None
        self._prefetch_depth = max(1, prefetch)
        self._prefetch_batch_size: int | None = None

    @staticmethod
    def _read_folder(path: Path, token_budget: int | None = None) -> list[np.ndarray]:
        arrays, taken = [], 0
        for fp in sorted(path.glob("*.npy")):
            if token_budget is not None and taken > token_budget:
                break
            if "offsets_" in fp.name:
                continue
            arr = np.load(fp, mmap_mode="r")
            taken += arr.shape[0]
            arrays.append(arr)
        return arrays

    def __len__(self) -> int:
        return self.N

    # ------------------------------------------------------------------ gathering
    def _gather(self, starts: np.ndarray) -> np.ndarray:
        """Windows ``[len(starts), ctx+1]`` int32 for global token offsets ``starts``."""
        span = self.context_length + 1
        out = np.empty((starts.shape[0], span), dtype=np.int32)
        chunk = np.searchsorted(self.chunk_starts, starts, side="right") - 1
        off = starts - self.chunk_starts[chunk]
        inside = off + span <= self.chunk_sizes[chunk]
        for c in np.unique(chunk[inside]):
            rows = np.nonzero((chunk == c) & inside)[0]
            out[rows] = self.ds[c][off[rows, None] + self._span[None, :]]
        for r in np.nonzero(~inside)[0]:  # window runs over a file boundary: stitch
            c, o, filled = int(chunk[r]), int(off[r]), 0
            while filled < span and c < len(self.ds):
                take = min(self.ds[c].shape[0] - o, span - filled)
                out[r, filled : filled + take] = self.ds[c][o : o + take]
                filled += take
                c, o = c + 1, 0
        return out

    def _get_batch_internal(self, batch_size: int) -> tuple[Tensor, Tensor]:
        lbs = local_batch_size(batch_size, self.world_size, self.rank)
        self.local_batch_size = lbs
        starts = torch.randint(low=0, high=len(self), size=(lbs,), generator=self.g)
        windows = self._gather(starts.numpy())
        return torch.from_numpy(windows[:, :-1]), torch.from_numpy(windows[:, 1:])

    # ------------------------------------------------------------------ prefetch
    def _prefetch_loop(self):
        pin = torch.cuda.is_available()
        while True:
            try:
                inputs, targets = self._get_batch_internal(self._prefetch_batch_size)
                # contiguous pinned copies so that .to(device, non_blocking=True) is a true async DMA
                inputs, targets = inputs.contiguous(), targets.contiguous()
                if pin:
                    inputs, targets = inputs.pin_memory(), targets.pin_memory()
            except BaseException as e:  # handed to the consumer: get_batch() raises it instead of waiting forever
                self._queue.put(e)
                return
            self._queue.put((inputs, targets))

    def get_batch(self, batch_size: int) -> tuple[Tensor, Tensor]:
        if self._thread is None:
            self._prefetch_batch_size = batch_size
            self.local_batch_size = local_batch_size(batch_size, self.world_size, self.rank)
            self._queue = queue.Queue(maxsize=self._prefetch_depth)
            self._thread = threading.Thread(target=self._prefetch_loop, daemon=True)
            self._thread.start()
        elif batch_size != self._prefetch_batch_size:
            raise ValueError(f"get_batch() batch_size changed: {batch_size} != {self._prefetch_batch_size}")
        item = self._queue.get()
        if isinstance(item, BaseException):
            self._queue.put(item)  # later calls fail the same way
            raise RuntimeError("the data prefetch thread failed") from item
        return item

    def get_iterator(self, batch_size: int) -> Iterator[tuple[Tensor, Tensor]]:
        """Sequential, non-overlapping windows of a single-file dataset; the last partial batch is dropped."""
        assert len(self.ds) == 1, "Only validation is supported (len(ds) == 1)"
        span = self.context_length + 1
        step = batch_size * span
        for first in range(0, self.N - step, step):
            starts = np.arange(first, first + step, span, dtype=np.int64)
            w = self._gather(starts)
            yield torch.from_numpy(w[:, :-1]), torch.from_numpy(w[:, 1:])
