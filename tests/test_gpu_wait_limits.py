"""Bounded waits that run out, on one GPU and without any fault: a flag that nobody sets makes the kernel give up after its
(here: one millisecond) limit, return, free what it holds and report a status code that the host reads; the next launch works.
"""

import time

import pytest
import torch

from sample_efficient_gpt_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
LIMIT = 2_000_000  # cycles, about a millisecond


def _rand(*shape):
    return (torch.randn(*shape, device=DEV) * 0.5).to(torch.bfloat16)


@pytest.mark.parametrize("impl", [1, 0], ids=["pair", "single"])
def test_gemm_gives_up_on_rows_that_never_arrive(impl):
    from sample_efficient_gpt_b200.ops import gemm as G

    assert ops.has_kernel("gemm")
    dev = torch.cuda.current_device()
    ops.ext().gemm_reset_status(dev)
    torch.manual_seed(0)
    a, b = _rand(512, 256), _rand(384, 256)
    flags = torch.zeros(4, dtype=torch.int32, device=DEV)  # rows [128 r, 128 r + 128) are "complete" once flags[r] >= 1: never
    t0 = time.monotonic()
    G.gemm(a, b, wait=(flags, 1, 128), wait_limit=LIMIT, impl=impl)
    torch.cuda.synchronize()
    assert time.monotonic() - t0 < 5.0, "the kernel must return after its wait limit, not hang"
    assert G.status() == 4, "status 4 = the producer's wait for a source region's arrival flag gave up"
    ops.ext().gemm_reset_status(dev)
    assert G.status() == 0
    # tensor memory was released and the barriers are in order: the same kernel runs normally afterwards
    flags.fill_(1)
    d = G.gemm(a, b, wait=(flags, 1, 128), impl=impl)
    torch.cuda.synchronize()
    want = a.float() @ b.float().t()
    assert G.status() == 0 and (d.float() - want).abs().max() <= 2e-2 * want.abs().max()
    # long contraction cut between pairs: the workspace flags were cleared by the reset as well
    x, w = _rand(8192, 256), _rand(8192, 256)
    g = G.mm_tn(x, w, out_f32=True, impl=impl)
    torch.cuda.synchronize()
    wantg = x.float().t() @ w.float()
    assert G.status() == 0 and (g - wantg).abs().max() <= 1e-2 * wantg.abs().max()


def test_comm_barrier_gives_up_on_a_peer_that_never_comes():
    """The bucket kernel as "rank 0 of 2" with both ranks' buffers on this GPU; nothing plays rank 1, so its flag stays 0."""
    assert ops.has_kernel("comm_allreduce_bucket")
    ext = ops.ext()
    blocks, n = 4, 2 * 8 * 1024
    grads = torch.randn(n, device=DEV)
    before = grads.clone()
    wires = [torch.zeros(n, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    flags = [torch.zeros(blocks * ext.COMM_MAX_RANKS, dtype=torch.int32, device=DEV) for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    t0 = time.monotonic()
    ext.comm_allreduce_bucket(grads, [w.data_ptr() for w in wires], [f.data_ptr() for f in flags], 0, 0, 0, 1, blocks, status, None, LIMIT)
    torch.cuda.synchronize()
    assert time.monotonic() - t0 < 5.0
    assert int(status.item()) == 1001, "1000 + the peer that did not show up"
    assert torch.equal(grads, before), "a block that gave up at the first barrier has not touched the gradients"
    # the device is fine: an ordinary kernel of the package runs
    y = ops.swiglu_fwd(_rand(64, 256))
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all()
