import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def reference_path():
    """Path that makes ``import sample_efficient_gpt`` (the installed reference) work, or skip."""
    p = ROOT / "baseline" / "_ref"
    if not (p / "sample_efficient_gpt").exists():
        pytest.skip("reference package is not installed under baseline/_ref")
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))
    return p
