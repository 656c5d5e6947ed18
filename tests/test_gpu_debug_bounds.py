"""The debug build of the extension (``_C_dbg.so``: every computed store index is checked against the extent of its
destination, csrc/bounds.cuh) in a process of its own with ``SEGPT_DEBUG_BOUNDS=1``:

  * the GEMM, kernel, attention and mixture-of-experts tests run against it on their odd shapes - any store outside its
    destination would leave a 90xx code in the status word, which is asserted to be 0 at the end;
  * outputs placed between canary rows stay inside their rows;
  * the checks do fire: with the output's extent capped below its real size, exactly the stores past the cap are refused,
    the status word says so, and nothing faults.
"""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

INNER = r'''
import torch
from sample_efficient_gpt_b200 import ops
from sample_efficient_gpt_b200.ops import gemm as G

ext = ops.ext()
assert ext.__name__.endswith("_C_dbg") and ext.DEBUG_BOUNDS, ext.__name__
dev = torch.cuda.current_device()
torch.manual_seed(0)
rnd = lambda *s: (torch.randn(*s, device="cuda") * 0.5).to(torch.bfloat16)

# canaries: the generic epilogues (addend, mirrored output, fp32 addend) write only inside their rows
for impl in (1, 0):
    for (M, N, K) in [(200, 136, 72), (300, 328, 200), (130, 264, 1104)]:
        a, b = rnd(M, K), rnd(N, K)
        c = rnd(M, N)
        big = torch.full((M + 16, N), 3.0, device="cuda", dtype=torch.bfloat16)
        G.gemm(a, b, c=c, out=big[8 : 8 + M], alpha=0.5, beta=2.0, impl=impl)
        torch.cuda.synchronize()
        want = 0.5 * (a.float() @ b.float().t()) + 2.0 * c.float()
        assert (big[8 : 8 + M].float() - want).abs().max() <= 3e-2 * want.abs().max()
        assert bool((big[:8] == 3.0).all()) and bool((big[8 + M :] == 3.0).all()), "canary rows were written"
    x = rnd(2, 264, 320)
    bigs = torch.full((2, 264 + 16, 264), 3.0, device="cuda", dtype=torch.bfloat16)
    G.gemm(x, x, out=bigs[:, 8 : 8 + 264], symmetric=True, impl=impl)
    torch.cuda.synchronize()
    assert (bigs[:, 8 : 8 + 264].float() - torch.bmm(x.float(), x.float().mT)).abs().max() < 0.5
    assert bool((bigs[:, :8] == 3.0).all()) and bool((bigs[:, 8 + 264 :] == 3.0).all())
    assert G.status() == 0, G.status()

# the checks fire: pretend the output ends after 100 rows; rows beyond stay untouched, status = 9000 + 1
for impl in (1, 0):
    M, N, K = 256, 192, 128
    a, b, c = rnd(M, K), rnd(N, K), torch.randn(M, N, device="cuda")
    out = torch.full((M, N), 7.0, device="cuda")
    ext.gemm_debug_extent_cap(100 * N)
    G.gemm(a, b, c=c, out=out, out_f32=True, alpha=1.0, beta=0.5, impl=impl)
    torch.cuda.synchronize()
    ext.gemm_debug_extent_cap(0)
    assert G.status() == 9001, G.status()
    want = a.float() @ b.float().t() + 0.5 * c
    assert (out[:100] - want[:100]).abs().max() <= 2e-2 * want.abs().max(), "stores inside the extent must still happen"
    assert bool((out[100:] == 7.0).all()), "stores past the extent must be refused"
    ext.gemm_reset_status(dev)
    out2 = G.gemm(a, b, c=c, out=torch.empty_like(out), out_f32=True, alpha=1.0, beta=0.5, impl=impl)
    torch.cuda.synchronize()
    assert G.status() == 0 and (out2 - want).abs().max() <= 2e-2 * want.abs().max()
print("DEBUG-BOUNDS-OK")
'''


def _env():
    env = dict(os.environ)
    env["SEGPT_DEBUG_BOUNDS"] = "1"
    env["PYTHONPATH"] = str(ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    return env


@pytest.mark.skipif(not (ROOT / "sample_efficient_gpt_b200" / "_C_dbg.so").exists(), reason="debug build missing: python -m sample_efficient_gpt_b200.csrc.build --debug-bounds")
def test_canaries_and_refused_stores_in_the_debug_build():
    r = subprocess.run([sys.executable, "-c", INNER], capture_output=True, text=True, timeout=600, env=_env(), cwd=ROOT)
    assert r.returncode == 0 and "DEBUG-BOUNDS-OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])


@pytest.mark.skipif(not (ROOT / "sample_efficient_gpt_b200" / "_C_dbg.so").exists(), reason="debug build missing")
def test_kernel_suites_pass_on_the_debug_build_without_a_violation():
    files = ["tests/test_gpu_gemm.py", "tests/test_gpu_kernels.py", "tests/test_gpu_moe.py", "tests/test_gpu_engine.py"]
    code = ("import sys, pytest, torch; rc = pytest.main(['-x', '-q', '-m', 'gpu', '-p', 'no:cacheprovider'] + sys.argv[1:]);"
            "from sample_efficient_gpt_b200 import ops; from sample_efficient_gpt_b200.ops import gemm as G;"
            "assert ops.ext().DEBUG_BOUNDS; torch.cuda.synchronize(); st = G.status(); print('FINAL-STATUS', st); sys.exit(int(rc) or (1 if st else 0))")
    r = subprocess.run([sys.executable, "-c", code, *files], capture_output=True, text=True, timeout=1500, env=_env(), cwd=ROOT)
    assert r.returncode == 0 and "FINAL-STATUS 0" in r.stdout, (r.stdout[-3000:], r.stderr[-2000:])
