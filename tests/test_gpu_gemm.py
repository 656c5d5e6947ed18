"""tcgen05 GEMM against an fp32 matmul of the same bf16 operands; ordered from one tile upwards.

Every case first checks the kernel's status word: a bounded wait that gave up is reported there instead of hanging.
"""

import pytest
import torch

from sample_efficient_gpt_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _g():
    from sample_efficient_gpt_b200.ops import gemm as G

    assert ops.has_kernel("gemm"), f"extension not built: {ops.ext_error()!r}"
    return G


@pytest.fixture(autouse=True, params=[1, 0], ids=["pair", "single"])
def gemm_impl(request):
    """Every case runs on the CTA-pair kernel and on the one-CTA-per-tile kernel."""
    G = _g()
    prev = G.DEFAULT_IMPL
    G.DEFAULT_IMPL = request.param
    yield request.param
    G.DEFAULT_IMPL = prev


def _check(d, want, name, tol=2e-2):
    G = _g()
    torch.cuda.synchronize()
    st = G.status()
    assert st == 0, f"{name}: kernel status {st} (a bounded wait gave up)"
    err = (d.float() - want).abs().max().item()
    scale = want.abs().max().item() + 1e-6
    assert err <= tol * scale, f"{name}: max err {err} vs scale {scale}"


def _rand(*shape):
    return (torch.randn(*shape, device=DEV) * 0.5).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 128, 256), (128, 256, 128), (256, 512, 512), (200, 136, 72), (1000, 1152, 1152),
                                   (24, 40, 64), (300, 1944, 200), (1300, 776, 1152)])
def test_nt(M, N, K):
    G = _g()
    torch.manual_seed(0)
    a, b = _rand(M, K), _rand(N, K)
    _check(G.mm_nt(a, b), a.float() @ b.float().t(), f"nt {M}x{N}x{K}")


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 320, 192), (520, 1152, 384)])
def test_nn_and_tn(M, N, K):
    G = _g()
    torch.manual_seed(1)
    a, w = _rand(M, K), _rand(K, N)
    _check(G.mm_nn(a, w), a.float() @ w.float(), f"nn {M}x{N}x{K}")
    at, bt = _rand(K, M), _rand(K, N)
    _check(G.mm_tn(at, bt), at.float().t() @ bt.float(), f"tn {M}x{N}x{K}")


def test_epilogue_batch_f32_and_strides():
    G = _g()
    torch.manual_seed(2)
    a, b = _rand(3, 256, 192), _rand(3, 384, 192)
    c = _rand(3, 256, 384)
    want = 0.5 * torch.bmm(a.float(), b.float().mT) - 1.5 * c.float()
    _check(G.gemm(a, b, c=c, alpha=0.5, beta=-1.5), want, "batched alpha/beta")
    cf = torch.randn(256, 384, device=DEV)
    d = G.gemm(a[0], b[0], c=cf, out=cf.clone(), out_f32=True, alpha=1.0, beta=1.0)
    _check(d, a[0].float() @ b[0].float().t() + cf, "fp32 accumulate", tol=1e-3)
    big = _rand(300, 512)
    view = big[:, 128:320]  # row stride 512, offset 128: still 16-byte aligned
    _check(G.mm_nt(view, b[1]), view.float() @ b[1].float().t(), "strided A")


def test_symmetric():
    G = _g()
    torch.manual_seed(3)
    x = _rand(2, 384, 640)
    a = G.gemm(x, x, symmetric=True)
    _check(a, torch.bmm(x.float(), x.float().mT), "x x^T symmetric")
    assert torch.allclose(a.float(), a.float().mT, atol=0.05, rtol=0.02)
    bb = G.gemm(a, a, c=a, alpha=0.3, beta=-0.7, symmetric=True)
    _check(bb, 0.3 * torch.bmm(a.float(), a.float()) - 0.7 * a.float(), "b A + c A A")


def test_newton_schulz_on_gemm_matches_library_path():
    from sample_efficient_gpt_b200.optim.newton_schulz import POLAR_EXPRESS_COEFFS
    from sample_efficient_gpt_b200.ops.newton_schulz import newton_schulz

    torch.manual_seed(4)
    for shape in [(4, 256, 512), (3, 512, 256), (1152, 1152), (5, 18, 256), (2, 256, 20)]:
        Gm = torch.randn(*shape, device=DEV)
        X = newton_schulz(Gm, 1e-7, POLAR_EXPRESS_COEFFS)
        Xb = Gm.to(torch.bfloat16)
        tr = Xb.size(-2) > Xb.size(-1)
        Y = Xb.mT if tr else Xb
        Y = Y / (Y.norm(dim=(-2, -1), keepdim=True) + 1e-7)
        for a, b, c in POLAR_EXPRESS_COEFFS:
            A = (Y.float() @ Y.float().mT).to(torch.bfloat16)
            B = (b * A.float() + c * (A.float() @ A.float())).to(torch.bfloat16)
            Y = (a * Y.float() + B.float() @ Y.float()).to(torch.bfloat16)
        Y = Y.mT if tr else Y
        _check(X, Y.float(), f"NS {shape}", tol=6e-2)
        s = torch.linalg.svdvals(X.float().reshape(-1, *X.shape[-2:])[0])
        assert s.max() < 1.3 and s.median() > 0.5


def test_large_shapes_and_speed():
    G = _g()
    torch.manual_seed(5)
    a, w = _rand(8192, 1152), _rand(6144, 1152)
    _check(G.mm_nt(a, w), a.float() @ w.float().t(), "8192x6144x1152")
    dy = _rand(8192, 3072)
    x = _rand(8192, 1152)
    _check(G.mm_tn(dy, x, out_f32=True), dy.float().t() @ x.float(), "wgrad 3072x1152x8192", tol=1e-2)


def test_pair_store_reduce_and_split_contraction():
    """The pair kernel's TMA epilogue (bf16 / fp32 store, accumulation into the output as a TMA reduce-add) with tiles that
    several pairs compute together (long contractions, few tiles) and with whole tiles per pair, on ragged shapes."""
    G = _g()
    torch.manual_seed(6)
    for (M, N, K) in [(1944, 1152, 4096), (200, 72, 1024), (1152, 1152, 8192), (256, 256, 16384)]:
        dy, x = _rand(K, M), _rand(K, N)
        want = dy.float().t() @ x.float()
        for sk in (True, False):
            _check(G.mm_tn(dy, x, out_f32=True, impl=1, split_k=sk), want, f"tn fp32 store split_k={sk} {M}x{N}x{K}", tol=1e-2)
            base = torch.randn(M, N, device=DEV)
            out = base.clone()
            G.gemm(dy, x, a_mn=True, b_mn=True, c=out, out=out, out_f32=True, beta=1.0, impl=1, split_k=sk)
            _check(out, want + base, f"tn fp32 accumulate split_k={sk} {M}x{N}x{K}", tol=1e-2)
        first = G.mm_tn(dy, x, out_f32=True, impl=1)
        again = G.mm_tn(dy, x, out_f32=True, impl=1)
        assert torch.equal(first, again), "the parts are summed in a fixed order: two runs must agree bit for bit"
    a, w = _rand(520, 328), _rand(328, 1000)
    o = torch.full((520, 1024), 7.0, device=DEV, dtype=torch.bfloat16)
    G.gemm(a, w, b_mn=True, out=o[:, :1000], impl=1)  # strided output: columns past N stay untouched
    _check(o[:, :1000], a.float() @ w.float(), "nn strided out")
    assert (o[:, 1000:] == 7.0).all()
    # generic epilogue (addend, bf16) on a long contraction that is cut between pairs
    a, b, c = _rand(256, 8192), _rand(300, 8192), _rand(256, 300)
    _check(G.gemm(a, b, c=c, alpha=0.5, beta=2.0, impl=1), 0.5 * (a.float() @ b.float().t()) + 2.0 * c.float(), "nt addend, cut contraction")


@pytest.mark.parametrize("M,F,K", [(512, 128, 64), (1000, 384, 1152), (4096, 3072, 1152), (77, 256, 200)])
def test_gemm_swiglu_epilogue(M, F, K, gemm_impl):
    """Up projection with the SwiGLU activation in the GEMM's epilogue: u against the fp32 product, f against the fp32
    statement of silu(gate) * up on the rounded u, and both bit-identical to GEMM + element-wise kernel."""
    if gemm_impl == 0:
        pytest.skip("the fused epilogue exists on the CTA-pair kernel only")
    G = _g()
    torch.manual_seed(M + F)
    x = (torch.randn(M, K, device=DEV) * 0.7).to(torch.bfloat16)
    w = (torch.randn(2 * F, K, device=DEV) * (1.5 / K**0.5)).to(torch.bfloat16)
    u, f = ops.ext().gemm_swiglu(x, w)
    torch.cuda.synchronize()
    assert G.status() == 0
    u_ref = x.float() @ w.float().T
    assert (u.float() - u_ref).abs().max().item() <= 2e-2 * u_ref.abs().max().item()
    ur = u.float()
    f_ref = torch.nn.functional.silu(ur[:, :F]) * ur[:, F:]
    assert (f.float() - f_ref).abs().max().item() <= 1e-2 * f_ref.abs().max().item() + 1e-3
    u2 = G.gemm(x, w, impl=1, split_k=False)  # same summation order as the fused launch: whole tiles
    f2 = ops.swiglu_fwd(u2)
    assert torch.equal(u, u2) and torch.equal(f, f2)


@pytest.mark.parametrize("M,F,K", [(512, 256, 64), (1000, 512, 1152), (4096, 3072, 1152), (77, 256, 200)])
def test_gemm_swiglu_backward_epilogue(M, F, K, gemm_impl):
    """Data gradient of the down projection with the SwiGLU backward in the GEMM's epilogue, against the fp32 statement and
    bit for bit against GEMM + element-wise kernel."""
    if gemm_impl == 0:
        pytest.skip("the fused epilogue exists on the CTA-pair kernel only")
    G = _g()
    torch.manual_seed(M + F + 1)
    dy = (torch.randn(M, K, device=DEV) * 0.5).to(torch.bfloat16)
    w = (torch.randn(K, F, device=DEV) * (1.5 / K**0.5)).to(torch.bfloat16)
    u = torch.randn(M, 2 * F, device=DEV).to(torch.bfloat16)
    du = ops.ext().gemm_swiglu_bwd(dy, w, u)
    torch.cuda.synchronize()
    assert G.status() == 0
    df = (dy.float() @ w.float()).to(torch.bfloat16).float()
    a, b = u.float()[:, :F], u.float()[:, F:]
    s = torch.sigmoid(a)
    want = torch.cat([df * b * (s + a * s * (1 - s)), df * a * s], dim=1)
    assert (du.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-3
    df2 = G.gemm(dy, w, b_mn=True, impl=1, split_k=False)  # same summation order as the fused launch: whole tiles
    assert torch.equal(du, ops.swiglu_bwd(df2, u))


@pytest.mark.parametrize("n_extra", [1, 3, 7])
@pytest.mark.parametrize("with_c", [True, False])
def test_gemm_extra_destinations(n_extra, with_c, gemm_impl):
    """Every output tile is stored to all further destinations as well (on several GPUs these are the peers' buffers: the
    all-gather of the sharded Newton-Schulz result); here they are local buffers, ragged shape, with and without addend,
    and once with a destination that is not 16-byte aligned (falls back to the register-store epilogue)."""
    G = _g()
    torch.manual_seed(n_extra)
    nb, M, N, K = 3, 328, 712, 264
    a = (torch.randn(nb, M, K, device=DEV) * 0.5).to(torch.bfloat16)
    b = (torch.randn(nb, N, K, device=DEV) * 0.1).to(torch.bfloat16)
    c = torch.randn(nb, M, N, device=DEV).to(torch.bfloat16) if with_c else None
    want = a.float() @ b.float().transpose(1, 2) + (0.5 * c.float() if with_c else 0.0)
    for misalign in (False, True):
        out = torch.empty(nb, M, N, device=DEV, dtype=torch.bfloat16)
        pool = torch.full((n_extra, nb * M * N + 8), 7.0, device=DEV, dtype=torch.bfloat16)
        off = 4 if misalign else 0  # 8 bytes off a 16-byte boundary
        extras = [pool[i, off : off + nb * M * N].view(nb, M, N) for i in range(n_extra)]
        if misalign:
            assert extras[0].data_ptr() % 16 == 8
        G.gemm(a, b, c=c, out=out, beta=0.5 if with_c else 0.0, extra_dst=[e.data_ptr() for e in extras])
        _check(out, want, f"out extra={n_extra} misalign={misalign}")
        for i, e in enumerate(extras):
            assert torch.equal(e, out), f"destination {i} differs from the main output"
            assert bool((pool[i, :off] == 7.0).all()) and bool((pool[i, off + nb * M * N :] == 7.0).all()), "stores outside the destination"
