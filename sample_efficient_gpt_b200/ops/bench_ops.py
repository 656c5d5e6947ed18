"""Microbenchmarks of the hot ops on one GPU, timed with CUDA events after warm-up (L2 flushed between iterations).

  python -m sample_efficient_gpt_b200.ops.bench_ops --op gemm --m 8192 --n 1920 --k 1152 [--kind nt|nn|tn] [--batch B]
  python -m sample_efficient_gpt_b200.ops.bench_ops --op ns --rows 1152 --cols 3072 --batch 30
  python -m sample_efficient_gpt_b200.ops.bench_ops --op attention --seq 2048        (B 8, 18q/6kv heads of 64, fwd+bwd)
  python -m sample_efficient_gpt_b200.ops.bench_ops --op linear_ce                    ([32768,1152] x [49152,1152])
  python -m sample_efficient_gpt_b200.ops.bench_ops --op elementwise
Each line reports milliseconds, achieved TFLOP/s or GB/s, and the library call it replaces where there is one.
"""

from __future__ import annotations

import argparse
import json

import torch

from sample_efficient_gpt_b200 import ops

_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")  # 2x the 126 MB L2
    _FLUSH.zero_()


def timeit(fn, iters: int = 10, warmup: int = 3, flush: bool = True) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def rnd(*shape, scale=0.5):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def bench_gemm(a):
    from sample_efficient_gpt_b200.ops import gemm as G

    bs = (a.batch,) if a.batch > 1 else ()
    M, N, K = a.m, a.n, a.k
    if a.kind == "nt":
        x, w = rnd(*bs, M, K), rnd(*bs, N, K)
        ours, lib = (lambda: G.mm_nt(x, w)), (lambda: x @ w.mT)
    elif a.kind == "nn":
        x, w = rnd(*bs, M, K), rnd(*bs, K, N)
        ours, lib = (lambda: G.mm_nn(x, w)), (lambda: x @ w)
    else:
        x, w = rnd(*bs, K, M), rnd(*bs, K, N)
        ours, lib = (lambda: G.mm_tn(x, w)), (lambda: x.mT @ w)
    fl = 2.0 * M * N * K * max(a.batch, 1) / 1e9
    t_o, t_l = timeit(ours, a.iters), timeit(lib, a.iters)
    print(json.dumps({"op": f"gemm_{a.kind}", "shape": [a.batch, M, N, K], "ours_ms": t_o, "ours_tflops": fl / t_o,
                      "cublas_ms": t_l, "cublas_tflops": fl / t_l, "status": G.status()}))


def bench_ns(a):
    from sample_efficient_gpt_b200.optim.newton_schulz import POLAR_EXPRESS_COEFFS
    from sample_efficient_gpt_b200.ops.newton_schulz import ns_iterations

    X = rnd(a.batch, a.rows, a.cols, scale=0.01)
    Y = torch.empty_like(X)
    r, c = min(a.rows, a.cols), max(a.rows, a.cols)
    fl = a.batch * 7 * (4.0 * r * r * c + 2.0 * r**3) / 1e9
    ours = lambda: ns_iterations(X, Y, POLAR_EXPRESS_COEFFS)  # noqa: E731

    def lib():
        Z = X.mT if a.rows > a.cols else X
        for aa, bb, cc in POLAR_EXPRESS_COEFFS:
            A = Z @ Z.mT
            B = torch.baddbmm(A, A, A, beta=bb, alpha=cc)
            Z = torch.baddbmm(Z, B, Z, beta=aa)

    t_o, t_l = timeit(ours, a.iters), timeit(lib, a.iters)
    print(json.dumps({"op": "newton_schulz", "shape": [a.batch, a.rows, a.cols], "ours_ms": t_o, "ours_tflops_full_equiv": fl / t_o,
                      "cublas_ms": t_l, "cublas_tflops": fl / t_l}))


def bench_attention(a):
    B, H, Hkv, hd, S = 8, 18, 6, 64, a.seq
    q, k, v = rnd(B, S, H, hd, scale=1.0), rnd(B, S, Hkv, hd, scale=1.0), rnd(B, S, Hkv, hd, scale=1.0)
    do = rnd(B, S, H, hd, scale=1.0)
    fl_f = 4.0 * B * H * S * S * hd / 2 / 1e9
    state = {}

    def fwd():
        state["o"], state["ctx"] = ops.attention_fwd(q, k, v, True, 0)

    def bwd():
        ops.attention_bwd(do, q, k, v, state["o"], state["ctx"], True, 0)

    t_f = timeit(fwd, a.iters)
    fwd()
    t_b = timeit(lambda: (fwd(), bwd()), a.iters) - t_f
    out = {"op": "attention", "seq": S, "library_fwd_ms": t_f, "library_fwd_tflops": fl_f / t_f, "library_bwd_ms": t_b,
           "library_bwd_tflops": 2.5 * fl_f / t_b}
    if ops.has_kernel("fa_fwd"):
        from sample_efficient_gpt_b200.ops import gemm as G

        t_n = timeit(lambda: ops.attention_fwd(q, k, v, True, 0, for_backward=False), a.iters)
        out.update({"native_fwd_ms": t_n, "native_fwd_tflops": fl_f / t_n, "status": G.status()})
    print(json.dumps(out))


def bench_linear_ce(a):
    from sample_efficient_gpt_b200.ops.cross_entropy import linear_ce_fwd_bwd

    T, d, V = 32768, 1152, 49152
    h = rnd(T, d, scale=1.0)
    w = rnd(V, d, scale=d**-0.5)
    tg = torch.randint(0, V, (T,), device="cuda")
    dw = torch.zeros(V, d, device="cuda")
    ours = lambda: linear_ce_fwd_bwd(h, w, tg, 1e-6, -100, 1.0 / T, 1.0, dw_out=dw)  # noqa: E731

    def lib():
        hh, ww = h.detach().requires_grad_(True), w.detach().requires_grad_(True)
        logits = hh @ ww.t()
        torch.nn.functional.cross_entropy(logits.float(), tg).backward()

    fl = 3 * 2.0 * T * d * V / 1e9
    t_o, t_l = timeit(ours, a.iters), timeit(lib, max(2, a.iters // 2))
    print(json.dumps({"op": "linear_ce_fwd_bwd", "ours_ms": t_o, "ours_tflops": fl / t_o, "materialised_logits_ms": t_l}))


def bench_elementwise(a):
    T, d, F = 32768, 1152, 3072
    res, delta, gain = torch.randn(T, d, device="cuda"), rnd(T, d), torch.ones(d, device="cuda")
    x, y, rstd, _ = ops.add_rmsnorm_fwd(res, delta, gain, 1.0, 1e-5, torch.bfloat16, True)
    u, df = rnd(T, 2 * F), rnd(T, F)
    rows = [
        ("add_rmsnorm_fwd", lambda: ops.add_rmsnorm_fwd(res, delta, gain, 1.0, 1e-5, torch.bfloat16, True), T * d * (4 + 2 + 4 + 2)),
        ("add_rmsnorm_bwd", lambda: ops.add_rmsnorm_bwd(y, res, x, gain, rstd, 1.0, torch.bfloat16), T * d * (2 + 4 + 4 + 4 + 2)),
        ("swiglu_fwd", lambda: ops.swiglu_fwd(u), T * F * 6),
        ("swiglu_bwd", lambda: ops.swiglu_bwd(df, u), T * F * 10),
    ]
    for name, fn, nbytes in rows:
        t = timeit(fn, a.iters)
        print(json.dumps({"op": name, "ms": t, "gb_per_s": nbytes / t / 1e6}))


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--op", required=True, choices=["gemm", "ns", "attention", "linear_ce", "elementwise"])
    p.add_argument("--m", type=int, default=8192)
    p.add_argument("--n", type=int, default=1920)
    p.add_argument("--k", type=int, default=1152)
    p.add_argument("--kind", default="nt", choices=["nt", "nn", "tn"])
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--rows", type=int, default=1152)
    p.add_argument("--cols", type=int, default=3072)
    p.add_argument("--seq", type=int, default=2048)
    p.add_argument("--iters", type=int, default=10)
    a = p.parse_args()
    {"gemm": bench_gemm, "ns": bench_ns, "attention": bench_attention, "linear_ce": bench_linear_ce, "elementwise": bench_elementwise}[a.op](a)


if __name__ == "__main__":
    main()
