"""NVLink kernels and multi-GPU training; needs at least two GPUs (child processes under torchrun, one rank per GPU on
as many GPUs as the box has: 2, 4 or 8).

NVLS is switched off in the libraries (NCCL_NVLS_ENABLE=0) and the package's own kernels use plain peer loads and
stores unless SEGPT_TEST_MULTIMEM=1 asks for the multimem variant as well.
"""

import pytest
import torch

from test_ddp_gloo import run_workers

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _world():
    n = _ngpu()
    return 8 if n >= 8 else (4 if n >= 4 else 2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
def test_comm_kernels_match_nccl():
    run_workers("comm_gpu", _world(), 29641, timeout=420, env_extra={"NCCL_NVLS_ENABLE": "0"})


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
def test_training_with_nvlink_kernels_matches_nccl():
    run_workers("train_gpu", _world(), 29651, timeout=600, env_extra={"NCCL_NVLS_ENABLE": "0"})


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
def test_expert_parallel_exchange_and_training():
    run_workers("moe_gpu", _world(), 29661, timeout=600, env_extra={"NCCL_NVLS_ENABLE": "0"})
