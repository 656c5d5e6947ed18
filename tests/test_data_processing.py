"""Offline data-curation tools on CPU with stand-in scorers and models."""

import json

import numpy as np
import pytest
import torch

from sample_efficient_gpt_b200.scripts.data_processing import classifier_filter as CF
from sample_efficient_gpt_b200.scripts.data_processing import common as C
from sample_efficient_gpt_b200.scripts.data_processing import format_stack as FS
from sample_efficient_gpt_b200.scripts.data_processing.sft import facility_location as FL
from sample_efficient_gpt_b200.scripts.data_processing.sft import generate_k as GK
from sample_efficient_gpt_b200.scripts.data_processing.sft import score as SC


def length_scorer(texts, batch_size=128):  # "quality" = number of words, so that thresholds are easy to reason about
    return [float(len(t.split())) for t in texts]


def test_sharding_and_row_files(tmp_path):
    assert [list(C.contiguous_shard(10, r, 4)) for r in range(4)] == [[0, 1, 2], [3, 4, 5], [6, 7, 8], [9]]
    assert list(C.contiguous_shard(2, 3, 4)) == []
    rows = [{"a": 1, "t": "x"}, {"a": 2, "t": "y"}]
    for name in ("r.jsonl", "r.parquet"):
        C.write_rows(tmp_path / name, rows)
        assert C.read_rows(tmp_path / name) == rows
    assert [C.int_score(s) for s in (-1, 2.4, 2.6, 9)] == [0, 2, 3, 5]


def test_classifier_filters(tmp_path):
    src = tmp_path / "in"
    src.mkdir()
    for i in range(3):
        C.write_rows(src / f"{i}.parquet", [{"text": "w " * n} for n in (1, 3, 5 + i)])
    for rank in range(2):
        CF.filter_parquet_dir(src, tmp_path / "out", length_scorer, 3, rank, 2)
    kept = C.read_rows(tmp_path / "out" / "2.parquet")
    assert [r["int_score"] for r in kept] == [3, 5] and kept[1]["score"] == 7.0 and kept[0]["length"] == 6
    assert CF.filter_parquet_dir(src, tmp_path / "out", length_scorer, 3, 0, 2) == []  # finished files are skipped
    txt = tmp_path / "c.txt"
    txt.write_text("a<|endoftext|>a b c<|endoftext|>a b c d<|endoftext|>")
    out = CF.filter_txt(txt, tmp_path / "txt_out", length_scorer, 3, 0, 1)
    assert out.read_text() == "a b c<|endoftext|>a b c d<|endoftext|>"
    row = CF.filter_repo_row({"repo_name": "o/r", "text": "x<|endoftext|>x y z w<|endoftext|>"}, length_scorer, 2)
    assert row["text"] == "x y z w<|endoftext|>" and row["results"] == [{"score": 4.0, "int_score": 4}] and row["repo_name"] == "o/r"


def test_format_stack(tmp_path):
    import tarfile

    repo = tmp_path / "src" / "repo-main"
    (repo / "pkg").mkdir(parents=True)
    (repo / "pkg" / "a.py").write_text("x = 1\n")
    (repo / "blob.txt").write_text("deadbeef" * 50)
    (repo / "unlisted.py").write_text("y = 2\n")
    mirrors = tmp_path / "mirrors"
    mirrors.mkdir()
    with tarfile.open(mirrors / "o__r.tar.gz", "w:gz") as tar:
        tar.add(repo, arcname="repo-main")
    meta = [{"repo_name": "o/r", "files": str([{"path": "pkg/a.py"}, {"path": "blob.txt"}])}, {"repo_name": "no/archive", "files": []}]
    out = FS.process(meta, mirrors, fmt=False)
    assert out == [{"repo_name": "o/r", "text": "x = 1\n<|endoftext|>"}]
    assert FS.is_mostly_hex("abcdef0123") and not FS.is_mostly_hex("hello world") and not FS.is_mostly_hex("")


def test_facility_location_matches_plain_greedy():
    torch.manual_seed(0)
    emb = torch.randn(60, 8)
    sim = FL.similarity(emb, block=16)
    got = FL.lazy_greedy(sim, 12, recheck=5)
    best, want = torch.zeros(60), []
    for _ in range(12):
        gains = torch.relu(sim - best[:, None]).sum(0)
        gains[want] = -1
        j = int(gains.argmax())
        want.append(j)
        best = torch.maximum(best, sim[:, j])
    assert got == want and len(set(got)) == 12


class _Tok:
    chat_template = None
    bos_token = None

    def encode(self, text, add_special_tokens=False):
        return [ord(c) % 50 for c in text]


class _LM(torch.nn.Module):
    def forward(self, ids):  # predicts (id + 1) % 50
        logits = torch.full((*ids.shape, 50), -10.0)
        logits.scatter_(-1, ((ids + 1) % 50)[..., None], 10.0)
        return logits, None


def test_sft_loss_scoring_and_filter(tmp_path):
    rows = [{"index": i, "input": {"messages": [{"role": "user", "content": "q"}]}, "output": "abc" if i % 2 else "zzz"} for i in range(4)]
    res = SC.run_loss(rows, _LM(), _Tok(), "cpu", 64)
    assert [r["index"] for r in res] == [0, 1, 2, 3]
    assert res[1]["loss"] < res[0]["loss"]  # 'abc' continues by +1 twice, 'zzz' never does
    ids, mask = SC.tokenize_with_mask(_Tok(), SC.conversation(rows[1]), 64)
    assert sum(mask) == 4 and len(ids) == len(mask)
    scored = [{"index": i, "loss": v} for i, v in enumerate([0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, None, 0.65])]
    C.write_rows(tmp_path / "l.jsonl", scored)
    n = SC.filter_dataset_by_loss(tmp_path / "l.jsonl", tmp_path / "k.jsonl", keep_pct=0.5)
    kept = [r["index"] for r in C.read_rows(tmp_path / "k.jsonl")]
    thr = np.percentile([0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.65], 50)
    assert n == len(kept) and all(scored[i]["loss"] < 0.95 * thr or 1.5 * thr < scored[i]["loss"] < 1.75 * thr for i in kept) and 8 not in kept


def test_generate_k_truncation_and_flow():
    msgs = [{"role": "user", "content": "a" * 10}, {"role": "assistant", "content": "b" * 10}, {"role": "user", "content": "c" * 10},
            {"role": "assistant", "content": "d" * 10}, {"role": "user", "content": "e" * 10}]
    assert GK.truncate_messages(msgs, 100) == msgs
    assert [m["content"][0] for m in GK.truncate_messages(msgs, 45)] == ["a", "b", "c"]  # the last user turn does not fit; the reply 'd' is dropped
    assert [m["content"][0] for m in GK.truncate_messages(msgs, 25)] == ["a"]
    assert [m["content"][0] for m in GK.truncate_messages(msgs[:3], 100)] == ["a", "b", "c"]
    assert GK.truncate_messages(msgs, 5) == []

    class Engine:
        def default_stop_ids(self):
            return [0]

        def chat(self, convs, params):
            return [[f"r{i}" for i in range(params.n)] for _ in convs]

    rows = [{"index": 0, "input": {"messages": msgs[:1]}, "output": "x"}, {"index": 1, "input": {"messages": []}, "output": "y"}]
    out = GK.generate_rows(rows, Engine(), 3, 16, 0.7, 30)
    assert len(out) == 1 and out[0]["generated_outputs"] == ["r0", "r1", "r2"] and out[0]["index"] == 0
