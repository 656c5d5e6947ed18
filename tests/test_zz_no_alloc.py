"""The allocation-free C entry point (csrc/noalloc.h), called the way its users call it: through the exported C symbol.

Those users are hosts that may not request device memory after start-up (a fixed arena, a no-allocation rule in a
control loop, a callback inside another framework's stream), so the test goes around the Python bindings and the
PyTorch allocator for the call itself: ctypes on the shared object, raw device pointers, the current stream handle.
The regular binding (which takes its scratch from the allocator) provides the expected values.  Two calls in a row
check that the scratch array left behind by the first call does not disturb the second.
This file is named so that pytest collects it last.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from sample_efficient_gpt_b200 import ops

    ext = ops.ext()
    assert ext is not None, f"extension not built: {ops.ext_error()!r}"
    lib = ctypes.CDLL(ext.__file__)
    fn = lib.segpt_add_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    lib.segpt_noalloc_last_error.restype = ctypes.c_char_p
    return lib, ext


def _call(lib, dy, dres_in, x, gain, rstd, scale, bf16):
    dres = torch.empty_like(x)
    dres_lp = torch.empty_like(dy)
    dgain = torch.empty_like(gain)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    rc = lib.segpt_add_rmsnorm_bwd_noalloc(
        dy.data_ptr(), dres_in.data_ptr() if dres_in is not None else None, x.data_ptr(), gain.data_ptr(), rstd.data_ptr(),
        dres.data_ptr(), dres_lp.data_ptr(), dgain.data_ptr(), x.size(0), x.size(1), scale, int(bf16),
        torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.segpt_noalloc_last_error().decode()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before  # the call itself took nothing from the allocator
    return dres, dres_lp, dgain


@pytest.mark.parametrize("bf16", [True, False])
def test_no_alloc_entry_matches_regular_binding_twice_in_a_row(bf16):
    lib, ext = _lib()
    torch.manual_seed(0)
    lp = torch.bfloat16 if bf16 else torch.float32
    for T, d in [(4096, 1152), (777, 256)]:  # second call: other shape, scratch still holds the first call's sums
        x = torch.randn(T, d, device="cuda")
        gain = torch.rand(d, device="cuda") + 0.5
        rstd = torch.rsqrt(x.square().mean(-1) + 1e-5)
        dy = torch.randn(T, d, device="cuda").to(lp)
        dres_in = torch.randn(T, d, device="cuda")
        want = ext.add_rmsnorm_bwd(dy, dres_in, x, gain, rstd, 0.5, bf16)
        got = _call(lib, dy, dres_in, x, gain, rstd, 0.5, bf16)
        for g, w, tol in zip(got, want, (1e-4, 3e-2 if bf16 else 1e-4, 1e-3)):
            err = (g.float() - w.float()).abs().max().item()
            assert err <= tol + 1e-4 * w.float().abs().max().item(), err
        want2 = ext.add_rmsnorm_bwd(dy, None, x, gain, rstd, 1.0, bf16)
        got2 = _call(lib, dy, None, x, gain, rstd, 1.0, bf16)
        assert torch.allclose(got2[2], want2[2], rtol=1e-4, atol=1e-3) and torch.allclose(got2[0], want2[0], atol=1e-4)


def test_no_alloc_entry_rejects_oversize_and_bad_arguments():
    lib, _ = _lib()
    x = torch.zeros(8, 4096, device="cuda")
    v = torch.zeros(4096, device="cuda")
    r = torch.zeros(8, device="cuda")
    args = lambda d: (x.data_ptr(), None, x.data_ptr(), v.data_ptr(), r.data_ptr(), x.data_ptr(), x.data_ptr(), v.data_ptr(), 8, d, 1.0, 0, None)  # noqa: E731
    assert lib.segpt_add_rmsnorm_bwd_noalloc(*args(4096)) == -3
    assert b"exceeds the built-in scratch" in lib.segpt_noalloc_last_error()
    assert lib.segpt_add_rmsnorm_bwd_noalloc(*args(6)) == -2
    assert lib.segpt_add_rmsnorm_bwd_noalloc(None, None, x.data_ptr(), v.data_ptr(), r.data_ptr(), x.data_ptr(), x.data_ptr(), v.data_ptr(), 8, 64, 1.0, 0, None) == -1
