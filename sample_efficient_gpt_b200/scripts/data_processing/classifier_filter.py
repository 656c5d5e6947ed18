"""Quality filtering with the FineWeb-edu / Stack-edu style classifiers, sharded over GPUs by file or by row.

    torchrun --nproc_per_node 8 -m sample_efficient_gpt_b200.scripts.data_processing.classifier_filter \
        parquet --input data/ --output data_filtered/ --classifier HuggingFaceFW/fineweb-edu-classifier --min-int-score 2

Modes (the reference's scripts/data_processing/{edu_filter_ds,edu_filter_ds_pleias,edu_filter_txt,python_code_filter}.py):
  parquet  every ``*.parquet`` under ``--input`` (files split over ranks): keep rows whose rounded score >= the
           threshold; output rows carry ``text, length, score, int_score``; finished outputs are skipped;
  txt      a text corpus with ``<|endoftext|>`` separated documents, cut at document boundaries into chunks that are
           split over ranks; kept documents are written to ``<output>/part_<rank>.txt``;
  repos    rows ``{repo_name, text}`` whose text is several files joined by ``<|endoftext|>``: every file is scored and
           only files with a rounded score > the threshold stay (rows split over ranks, ``<output>/part_<rank>.parquet``).
``score_fn`` arguments let tests (and other classifiers) replace the Hugging Face model.
"""

from __future__ import annotations

import argparse
from pathlib import Path

from sample_efficient_gpt_b200.scripts.data_processing.common import (ClassifierScorer, contiguous_shard, device_for, int_score,
                                                                      rank_world, read_rows, write_rows)

EOT = "<|endoftext|>"


def filter_docs(docs: list[str], score_fn, min_int_score: int, batch_size: int = 128) -> list[dict]:
    scores = score_fn(docs, batch_size)
    return [{"text": d, "length": len(d), "score": s, "int_score": int_score(s)} for d, s in zip(docs, scores) if int_score(s) >= min_int_score]


def filter_parquet_dir(src: Path, dst: Path, score_fn, min_int_score: int, rank: int, world: int, text_key: str = "text") -> list[Path]:
    files = sorted(Path(src).glob("*.parquet"))
    done = []
    for i in contiguous_shard(len(files), rank, world):
        out = Path(dst) / files[i].name
        if out.exists():
            continue
        rows = filter_docs([r[text_key] for r in read_rows(files[i])], score_fn, min_int_score)
        write_rows(out, rows)
        done.append(out)
    return done


def filter_txt(src: Path, dst: Path, score_fn, min_int_score: int, rank: int, world: int, chunk_bytes: int = 64 << 20) -> Path:
    from sample_efficient_gpt_b200.tokenizer.pretokenization import find_chunk_boundaries

    src, dst = Path(src), Path(dst)
    dst.mkdir(parents=True, exist_ok=True)
    out = dst / f"part_{rank}.txt"
    with src.open("rb") as f, out.open("w", encoding="utf-8") as w:
        bounds = find_chunk_boundaries(f, max(world, -(-src.stat().st_size // chunk_bytes)), EOT.encode())
        spans = list(zip(bounds[:-1], bounds[1:]))
        for i in contiguous_shard(len(spans), rank, world):
            f.seek(spans[i][0])
            docs = [d for d in f.read(spans[i][1] - spans[i][0]).decode("utf-8", errors="ignore").split(EOT) if d.strip()]
            for row in filter_docs(docs, score_fn, min_int_score):
                w.write(row["text"] + EOT)
    return out


def filter_repo_row(row: dict, score_fn, min_int_score: int, batch_size: int = 128) -> dict:
    files = row["text"].split(EOT)[:-1]
    scores = score_fn(files, batch_size) if files else []
    kept = [(f, s) for f, s in zip(files, scores) if int_score(s) > min_int_score]
    text = "".join(f + EOT for f, _ in kept)
    return {"text": text, "results": [{"score": s, "int_score": int_score(s)} for _, s in kept], "length": len(text),
            "repo_name": row.get("repo_name")}


def filter_repos(src: Path, dst: Path, score_fn, min_int_score: int, rank: int, world: int) -> Path:
    rows = read_rows(src)
    out = Path(dst) / f"part_{rank}.parquet"
    write_rows(out, [filter_repo_row(rows[i], score_fn, min_int_score) for i in contiguous_shard(len(rows), rank, world)])
    return out


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("mode", choices=["parquet", "txt", "repos"])
    p.add_argument("--input", required=True, type=Path)
    p.add_argument("--output", required=True, type=Path)
    p.add_argument("--classifier", default="HuggingFaceFW/fineweb-edu-classifier")
    p.add_argument("--min-int-score", type=int, default=2)
    p.add_argument("--text-key", default="text")
    a = p.parse_args(argv)
    rank, world = rank_world()
    scorer = ClassifierScorer(a.classifier, device_for(rank))
    if a.mode == "parquet":
        filter_parquet_dir(a.input, a.output, scorer, a.min_int_score, rank, world, a.text_key)
    elif a.mode == "txt":
        filter_txt(a.input, a.output, scorer, a.min_int_score, rank, world)
    else:
        filter_repos(a.input, a.output, scorer, a.min_int_score, rank, world)


if __name__ == "__main__":
    main()
