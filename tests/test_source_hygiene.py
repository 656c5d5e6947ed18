"""Static checks over the source tree: no TMA/bulk load with cluster multicast anywhere (the multi-GPU paths must not be
able to reach one), none of the batched-memcpy driver calls, every spin-wait helper bounded, and no committed file
depending on the scratch folder."""

import re
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
SKIP_DIRS = {".git", "gpurun_out", "_work", "baseline", "__pycache__", ".pytest_cache", "build"}
TEXT_SUFFIXES = {".py", ".cu", ".cuh", ".h", ".hpp", ".cpp", ".cc", ".yaml", ".yml", ".toml", ".txt", ".json", ".sh", ".cfg"}


def source_files():
    for p in ROOT.rglob("*"):
        if p.is_file() and p.suffix in TEXT_SUFFIXES and not (set(p.relative_to(ROOT).parts) & SKIP_DIRS):
            yield p


def test_no_cluster_multicast_loads_and_no_batched_memcpy():
    multicast = ".multi" + "cast::" + "cluster"
    batch_calls = [a + "Memcpy" + b + "Batch" + "Async" for a in ("cuda", "cu") for b in ("", "3D")]
    for p in source_files():
        text = p.read_text(errors="ignore")
        if multicast in text:
            # only tcgen05.commit may carry the qualifier; any bulk/tensor copy with it is forbidden
            for line in text.splitlines():
                if multicast in line:
                    assert "tcgen05.commit" in line and "cp.async" not in line, f"{p}: {line.strip()}"
        for name in batch_calls:
            assert name not in text, f"{p} names {name}"


def test_every_device_wait_is_bounded():
    """Each loop that polls an mbarrier, a flag or a peer's memory lives in a helper with an iteration or time limit."""
    csrc = ROOT / "sample_efficient_gpt_b200" / "csrc"
    for p in list(csrc.glob("*.cu")) + list(csrc.glob("*.cuh")):
        text = p.read_text()
        for m in re.finditer(r"while\s*\(\s*(true|1)\s*\)|for\s*\(\s*;\s*;\s*\)", text):
            body = text[m.start(): m.start() + 900]
            assert re.search(r"globaltimer|clock64|spins|tries|iter|limit|budget", body), f"{p.name}: unbounded loop near offset {m.start()}"
        if "try_wait" in text:
            assert re.search(r"globaltimer|clock64|limit|spins", text), f"{p.name}: mbarrier wait without a bound"


def test_committed_files_do_not_use_the_scratch_folder():
    tracked = subprocess.run(["git", "ls-files"], cwd=ROOT, capture_output=True, text=True).stdout.split()
    assert not [f for f in tracked if f.startswith(("_work/", "gpurun_out/", "baseline/_ref"))]
    pat = re.compile(r"""(from|import)\s+_work|["'/]_work/""")
    for f in tracked:
        p = ROOT / f
        if p.suffix in {".py", ".cu", ".cuh", ".h", ".cpp"} and p.name != "test_source_hygiene.py" and p.exists():
            assert not pat.search(p.read_text(errors="ignore")), f"{f} refers to the scratch folder"
