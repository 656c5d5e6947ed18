"""Turn mirrored source repositories into one training document per repository.

For every row ``{repo_name, files: [{path, ...}]}`` of the metadata table the archive ``<mirrors>/<owner>__<repo>.tar.gz``
is unpacked, files that the metadata does not list or that are mostly hexadecimal are dropped, Python and JS/TS sources
are optionally run through a formatter, and the remaining files are joined with ``<|endoftext|>``.  Results are written
as zstd parquet shards of ``shard_size`` rows (``{repo_name, text}``).  This is the data preparation of the reference's
scripts/data_processing/format_and_upload_stack.py:23-251; the upload to a dataset hub is left to the caller
(``--upload-repo`` uses ``huggingface_hub`` when it is installed and the machine is online).
"""

from __future__ import annotations

import argparse
import ast
import shutil
import subprocess
import tarfile
import tempfile
from pathlib import Path

from sample_efficient_gpt_b200.scripts.data_processing.common import read_rows, write_rows

EOT = "<|endoftext|>"
PEEK_BYTES = 128_000
FORMATTERS = {  # suffix group -> command template (skipped when the tool is not on PATH)
    (".py", ".ipynb"): ["ruff", "format", "{dir}"],
    (".js", ".ts", ".jsx", ".tsx", ".json", ".html", ".css", ".graphql"): ["npx", "@biomejs/biome", "check", "--unsafe", "--write", "{dir}"],
}


def is_mostly_hex(text: str, threshold: float = 0.9) -> bool:
    return bool(text) and sum(c in "0123456789abcdefABCDEF" for c in text) / len(text) >= threshold


def apply_formatting(directory: Path, timeout: int = 90) -> str:
    suffixes = {p.suffix for p in Path(directory).glob("**/*") if p.is_file()}
    log = ""
    for group, cmd in FORMATTERS.items():
        if suffixes & set(group) and shutil.which(cmd[0]):
            try:
                r = subprocess.run([c.format(dir=str(directory)) for c in cmd], capture_output=True, timeout=timeout)
                log += r.stdout.decode(errors="ignore")
            except subprocess.TimeoutExpired:
                pass
    return log


def repo_document(archive: Path, listed: set[str], fmt: bool = True) -> str:
    with tempfile.TemporaryDirectory() as tmp:
        with tarfile.open(archive, "r:gz") as tar:
            tar.extractall(tmp, filter="tar")
        root = next(Path(tmp).iterdir())
        for f in sorted(root.glob("**/*")):
            if f.is_file():
                head = f.open("rb").read(PEEK_BYTES).decode("utf-8", errors="ignore")
                if str(f.relative_to(root)) not in listed or is_mostly_hex(head):
                    f.unlink()
        if fmt:
            apply_formatting(root)
        parts = []
        for f in sorted(root.glob("**/*")):
            if f.is_file():
                try:
                    parts.append(f.read_text() + EOT)
                except (UnicodeDecodeError, OSError):
                    pass
        return "".join(parts)


def process(meta_rows: list[dict], mirrors: Path, fmt: bool = True) -> list[dict]:
    out = []
    for item in meta_rows:
        files = item["files"] if not isinstance(item["files"], str) else ast.literal_eval(item["files"])
        archive = Path(mirrors) / f"{item['repo_name'].replace('/', '__')}.tar.gz"
        if archive.exists():
            out.append({"repo_name": item["repo_name"], "text": repo_document(archive, {f["path"] for f in files}, fmt)})
    return out


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--meta", required=True, type=Path, help="jsonl/parquet with repo_name and files")
    p.add_argument("--mirrors", required=True, type=Path)
    p.add_argument("--output", required=True, type=Path)
    p.add_argument("--shard-size", type=int, default=5000)
    p.add_argument("--no-format", action="store_true")
    p.add_argument("--upload-repo", default=None)
    a = p.parse_args(argv)
    rows = read_rows(a.meta)
    for n, at in enumerate(range(0, len(rows), a.shard_size), start=1):
        shard = a.output / f"train-{n:06d}.parquet"
        write_rows(shard, process(rows[at : at + a.shard_size], a.mirrors, not a.no_format))
        if a.upload_repo:
            from huggingface_hub import create_repo, upload_file

            create_repo(a.upload_repo, repo_type="dataset", exist_ok=True)
            upload_file(path_or_fileobj=str(shard), path_in_repo=f"data/{shard.name}", repo_id=a.upload_repo, repo_type="dataset")


if __name__ == "__main__":
    main()
