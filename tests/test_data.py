import json

import numpy as np
import pytest
import torch

from sample_efficient_gpt_b200.training.data import MemoryMappedDataset, local_batch_size


@pytest.fixture
def shards(tmp_path):
    d = tmp_path / "train"
    d.mkdir()
    np.save(d / "a.npy", np.arange(600, dtype=np.uint16))
    np.save(d / "b.npy", np.arange(600, 1000, dtype=np.uint16))
    np.save(d / "offsets_a.npy", np.arange(5))
    return d


def test_golden_window_starts(shards):
    # reference loader, same inputs: local batch 3, starts [422, 787, 604]
    ds = MemoryMappedDataset(shards, 8, "cpu", seed=42, world_size=2, rank=1)
    assert len(ds) == 992
    x, y = ds._get_batch_internal(6)
    assert x.dtype == torch.int32 and x.shape == (3, 8) and ds.local_batch_size == 3
    assert x[:, 0].tolist() == [422, 787, 604]
    assert torch.equal(y, x + 1)


def test_window_across_file_boundary(shards):
    ds = MemoryMappedDataset(shards, 8, "cpu", seed=0)
    w = ds._gather(np.array([596, 0, 991]))
    assert w[0].tolist() == list(range(596, 605)) and w[2].tolist() == list(range(991, 1000))


def test_single_file_train_and_iterator(tmp_path):
    f = tmp_path / "val.npy"
    np.save(f, np.arange(1000, dtype=np.uint16))
    ds = MemoryMappedDataset(f, 8, "cpu", seed=1)
    x, _ = ds._get_batch_internal(4)  # a single file works as a training set too
    assert x.shape == (4, 8)
    it = ds.get_iterator(2)
    x0, y0 = next(it)
    assert x0[:, 0].tolist() == [0, 9] and x0.shape == (2, 8) and torch.equal(y0, x0 + 1)
    n = 1 + sum(1 for _ in it)
    assert n == len(range(0, 992 - 18, 18))


def test_json_mix_budget(tmp_path, shards):
    mix = tmp_path / "mix.json"
    mix.write_text(json.dumps({str(shards): 100}))
    ds = MemoryMappedDataset(mix, 8, "cpu", seed=0)
    assert ds.total_length == 600  # the second shard is beyond the 100-token budget


def test_prefetch_and_split(shards):
    ds = MemoryMappedDataset(shards, 8, "cpu", seed=3, world_size=4, rank=0)
    a, b = ds.get_batch(10)
    assert a.shape == (3, 8)
    with pytest.raises(ValueError):
        ds.get_batch(12)
    assert [local_batch_size(10, 4, r) for r in range(4)] == [3, 3, 2, 2]
    with pytest.raises(ValueError):
        local_batch_size(2, 4, 0)
