"""Build the native tokenizer tools (``sample_efficient_gpt_b200/tokenizer/_segtok.so``) with g++ and pybind11.

``python -m sample_efficient_gpt_b200.tokenizer.build``.  No CUDA and no torch involved.
"""

from __future__ import annotations

import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "csrc" / "segtok.cpp"
TARGET = HERE / "_segtok.so"


def build(force: bool = False) -> Path:
    import pybind11

    deps = [SRC, HERE / "csrc" / "unicode_tables.h"]
    if not force and TARGET.exists() and all(TARGET.stat().st_mtime >= d.stat().st_mtime for d in deps):
        return TARGET
    cmd = ["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-pthread", f"-I{pybind11.get_include()}",
           f"-I{sysconfig.get_paths()['include']}", f"-I{HERE / 'csrc'}", str(SRC), "-o", str(TARGET)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"tokenizer build failed:\n{r.stderr}")
    return TARGET


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
