"""The stream-K schedule of the CTA-pair GEMM is plain C++ shared by host and device (csrc/gemm_pair_sched.h); this
compiles it with the host compiler and checks, for the training shapes and a set of ragged ones, that the pairs' shares
cover every k-block of every tile exactly once and that owners and contributors agree on who adds whose part."""

import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(shutil.which("g++") is None, reason="no host compiler")
def test_stream_k_schedule_covers_every_k_block_once(tmp_path):
    exe = tmp_path / "sched_check"
    inc = ROOT / "sample_efficient_gpt_b200" / "csrc"
    subprocess.run(["g++", "-O2", "-std=c++17", f"-I{inc}", str(ROOT / "tests" / "gemm_sched_check.cpp"), "-o", str(exe)], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.startswith("ok"), r.stdout + r.stderr
