"""Microbenchmarks of the hot ops on one GPU, timed with CUDA events after warm-up (L2 flushed between iterations).

  python -m sample_efficient_gpt_b200.ops.bench_ops --op gemm --m 8192 --n 1920 --k 1152 [--kind nt|nn|tn] [--batch B]
  python -m sample_efficient_gpt_b200.ops.bench_ops --op ns --rows 1152 --cols 3072 --batch 30
  python -m sample_efficient_gpt_b200.ops.bench_ops --op attention --seq 2048        (B 8, 18q/6kv heads of 64, fwd+bwd)
  python -m sample_efficient_gpt_b200.ops.bench_ops --op linear_ce                    ([32768,1152] x [49152,1152])
  python -m sample_efficient_gpt_b200.ops.bench_ops --op elementwise                  (norms, SwiGLU, qkv post-processing, gate, AdamW, EMA)
  python -m sample_efficient_gpt_b200.ops.bench_ops --op decode                       (generation: eager vs CUDA-graph decode step)
  python -m sample_efficient_gpt_b200.ops.bench_ops --op muon --layers 30                 (one NorMuonCWD step on the block matrices)
  python -m sample_efficient_gpt_b200.ops.bench_ops --op moe                          (router, dispatch, combine, router backward)
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


def time_sustained(fn, seconds: float = 1.0) -> float:
    """Milliseconds per call when the call runs back to back for about ``seconds`` (the power cap, not the burst clock,
    then sets the rate - the state a kernel meets inside a training step)."""
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        fn()
    e1.record()
    torch.cuda.synchronize()
    n = max(20, int(seconds * 1e3 / max(e0.elapsed_time(e1) / 20, 1e-3)))
    for _ in range(n // 4):  # bring the chip to its steady power state first
        fn()
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


def rnd(*shape, scale=0.5):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _bench_gemm_one(kind, M, N, K, batch, iters, split_k, label="", sustained=False):
    from sample_efficient_gpt_b200.ops import gemm as G

    bs = (batch,) if batch > 1 else ()
    f32 = kind == "tn"  # weight gradients are produced in fp32
    if kind == "nt":
        x, w = rnd(*bs, M, K), rnd(*bs, N, K)
        ours, lib = (lambda impl: G.mm_nt(x, w, impl=impl, split_k=split_k)), (lambda: x @ w.mT)
    elif kind == "nn":
        x, w = rnd(*bs, M, K), rnd(*bs, K, N)
        ours, lib = (lambda impl: G.mm_nn(x, w, impl=impl, split_k=split_k)), (lambda: x @ w)
    else:
        x, w = rnd(*bs, K, M), rnd(*bs, K, N)
        out = torch.empty(*bs, M, N, device="cuda", dtype=torch.float32)
        ours = lambda impl: G.mm_tn(x, w, out=out, out_f32=True, impl=impl, split_k=split_k)  # noqa: E731
        lib = (lambda: torch.bmm(x.mT, w, out_dtype=torch.float32, out=out)) if bs else (lambda: torch.mm(x.mT, w, out_dtype=torch.float32, out=out))
    fl = 2.0 * M * N * K * max(batch, 1) / 1e9
    if sustained:
        t_p, t_l = time_sustained(lambda: ours(1)), time_sustained(lib)
        print(json.dumps({"op": f"gemm_{kind}", "label": label, "mode": "sustained", "shape": [batch, M, N, K], "pair_ms": round(t_p, 4),
                          "pair_tflops": round(fl / t_p, 1), "cublas_ms": round(t_l, 4), "cublas_tflops": round(fl / t_l, 1),
                          "status": G.status()}), flush=True)
        return
    t_p, t_s, t_l = timeit(lambda: ours(1), iters), timeit(lambda: ours(0), iters), timeit(lib, iters)
    print(json.dumps({"op": f"gemm_{kind}", "label": label, "shape": [batch, M, N, K], "out": "fp32" if f32 else "bf16",
                      "pair_ms": round(t_p, 4), "pair_tflops": round(fl / t_p, 1), "single_ms": round(t_s, 4),
                      "single_tflops": round(fl / t_s, 1), "cublas_ms": round(t_l, 4), "cublas_tflops": round(fl / t_l, 1),
                      "split_k": split_k, "status": G.status()}), flush=True)


def bench_gemm(a):
    sk = not a.no_split_k
    if a.shapes == "block":  # IMU-1 430M projections at T tokens: y = x W^T, dx = dy W, dW = dy^T x
        T = a.m
        for name, n_out, n_in in [("qkv+gate", 1944, 1152), ("out", 1152, 1152), ("up", 6144, 1152), ("down", 1152, 3072)]:
            _bench_gemm_one("nt", T, n_out, n_in, 1, a.iters, sk, name + " fwd", a.sustained)
            _bench_gemm_one("nn", T, n_in, n_out, 1, a.iters, sk, name + " dgrad", a.sustained)
            _bench_gemm_one("tn", n_out, n_in, T, 1, a.iters, sk, name + " wgrad", a.sustained)
        return
    _bench_gemm_one(a.kind, a.m, a.n, a.k, a.batch, a.iters, sk, "", a.sustained)


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

    import os

    prev = os.environ.get("SEGPT_ATTN_IMPL")
    os.environ["SEGPT_ATTN_IMPL"] = "library"  # the dispatch's default is the native pair
    try:
        t_f = timeit(fwd, a.iters)
        fwd()
        t_b = timeit(lambda: (fwd(), bwd()), a.iters) - t_f
    finally:
        if prev is None:
            del os.environ["SEGPT_ATTN_IMPL"]
        else:
            os.environ["SEGPT_ATTN_IMPL"] = prev
    out = {"op": "attention", "seq": S, "library_fwd_ms": t_f, "library_fwd_tflops": fl_f / t_f, "library_bwd_ms": t_b,
           "library_bwd_tflops": 2.5 * fl_f / t_b}
    if ops.has_kernel("fa_fwd"):
        from sample_efficient_gpt_b200.ops import gemm as G

        t_n = timeit(lambda: ops.attention_fwd(q, k, v, True, 0, for_backward=False), a.iters)
        out.update({"native_fwd_ms": t_n, "native_fwd_tflops": fl_f / t_n})
        print(json.dumps(out), flush=True)
        if ops.has_kernel("fa_bwd"):
            o_n, lse_n = ops.ext().fa_fwd(q, k, v, True)
            t_nb = timeit(lambda: ops.ext().fa_bwd(do, q, k, v, o_n, lse_n, True), a.iters)
            out.update({"native_bwd_ms": t_nb, "native_bwd_tflops": 2.5 * fl_f / t_nb})
            # per-stage cycles of the CTA with the longest walk (slot meanings: csrc/attn_fwd.cu, csrc/attn_bwd.cu)
            pf = torch.zeros(16, dtype=torch.int64, device="cuda")
            pb = torch.zeros(16, dtype=torch.int64, device="cuda")
            ops.ext().fa_fwd(q, k, v, True, pf)
            ops.ext().fa_bwd(do, q, k, v, o_n, lse_n, True, pb)
            out["fwd_stage_cycles"], out["bwd_stage_cycles"] = pf.tolist(), pb.tolist()
        out["status"] = G.status()
    print(json.dumps(out))


def bench_linear_ce(a):
    from sample_efficient_gpt_b200.ops.cross_entropy import linear_ce_fwd_bwd

    T, d, V = a.tokens, 1152, 49152
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
    t_o = timeit(ours, a.iters)
    if a.ours_only:  # profiling runs: no library or materialised-logits comparison (6 GB of fp32 logits)
        print(json.dumps({"op": "linear_ce_fwd_bwd", "tokens": T, "ours_ms": t_o, "ours_tflops": fl / t_o}))
        return
    ops._DISABLED.add("ce_gemm")  # same chunking and CE kernel, library GEMMs
    try:
        t_c = timeit(ours, a.iters)
    finally:
        ops._DISABLED.discard("ce_gemm")
    t_l = timeit(lib, max(2, a.iters // 2))
    print(json.dumps({"op": "linear_ce_fwd_bwd", "ours_ms": t_o, "ours_tflops": fl / t_o, "with_library_gemms_ms": t_c,
                      "with_library_gemms_tflops": fl / t_c, "materialised_logits_ms": t_l}))


def bench_muon(a):
    """One NorMuonCWD step on the IMU-1 block matrices of ``--layers`` layers (momentum, Newton-Schulz, tail)."""
    from sample_efficient_gpt_b200.optim import NorMuonCWD

    shapes = [(1920, 1152), (1152, 1152), (6144, 1152), (1152, 3072)]
    ps = [torch.nn.Parameter(torch.randn(r, c, device="cuda") * 0.02) for _ in range(a.layers) for (r, c) in shapes]
    for p_ in ps:
        p_.grad = torch.randn_like(p_) * 1e-3
    opt = NorMuonCWD(ps, lr=0.02, momentum=0.95, weight_decay=0.1)
    t = timeit(lambda: opt.step(), a.iters, flush=False)
    print(json.dumps({"op": "normuon_cwd_step", "layers": a.layers, "matrices": len(ps), "ms": t}))


def measured_hbm_gbs() -> tuple[float, str]:
    """Copy bandwidth measured on this pool (MEASURED_PEAKS.json at the repository root), else the stated fallback."""
    from pathlib import Path

    f = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "of measured"
    return 6650.0, "of fallback"


def report(rows, iters):
    peak, label = measured_hbm_gbs()
    for name, fn, nbytes in rows:
        t = timeit(fn, iters)
        gbs = nbytes / t / 1e6
        print(json.dumps({"op": name, "ms": round(t, 4), "gb_per_s": round(gbs, 1), "mbytes": round(nbytes / 1e6, 1), "frac_hbm": round(gbs / peak, 3),
                          "frac_of": label}))


def bench_elementwise(a):
    """Memory-bound kernels at the IMU-1 training shapes (T = 16 x 2048 tokens); bytes are the algorithmic minimum."""
    T, d, F, H, Hkv, hd, B, S = 32768, 1152, 3072, 18, 6, 64, 16, 2048
    res, delta, gain = torch.randn(T, d, device="cuda"), rnd(T, d), torch.ones(d, device="cuda")
    x, y, rstd, _ = ops.add_rmsnorm_fwd(res, delta, gain, 1.0, 1e-5, torch.bfloat16, True)
    u, df = rnd(T, 2 * F), rnd(T, F)
    from sample_efficient_gpt_b200.models.rope import RotaryPositionalEmbedding

    rope = RotaryPositionalEmbedding(10000.0, hd, S, device="cuda")
    qkv = rnd(T, (H + 2 * Hkv) * hd)
    one = torch.ones(1, device="cuda")
    v1 = ops.qkv_post_fwd(qkv, None, rope.cos, rope.sin, one, one, one * 0.5, one, B, S, H, Hkv, hd, True)[2].clone()
    q, k, v = ops.qkv_post_fwd(qkv, v1, rope.cos, rope.sin, one, one, one * 0.5, one, B, S, H, Hkv, hd, True)
    dq, dk, dv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
    o, z, dg = rnd(T, H, hd), rnd(T, H), rnd(T, H * hd)
    nq, nkv = T * H * hd, T * Hkv * hd
    # flat parameter sets for the multi-tensor optimizer kernels (about the AdamW share of IMU-1: 2 x 49152 x 1152)
    ps = [torch.randn(49152, 1152, device="cuda") for _ in range(2)]
    gs, ms, vs = ([torch.randn_like(p) * 1e-3 for p in ps] for _ in range(3))
    vs = [t.abs() for t in vs]
    sh = [p.bfloat16() for p in ps]
    ema = [p.clone() for p in ps]
    npar = sum(p.numel() for p in ps)
    rows = [
        ("add_rmsnorm_fwd", lambda: ops.add_rmsnorm_fwd(res, delta, gain, 1.0, 1e-5, torch.bfloat16, True), T * d * (4 + 2 + 4 + 2)),
        ("add_rmsnorm_bwd", lambda: ops.add_rmsnorm_bwd(y, res, x, gain, rstd, 1.0, torch.bfloat16), T * d * (2 + 4 + 4 + 4 + 2)),
        ("swiglu_fwd", lambda: ops.swiglu_fwd(u), T * F * 6),
        ("swiglu_bwd", lambda: ops.swiglu_bwd(df, u), T * F * 10),
        ("qkv_post_fwd", lambda: ops.qkv_post_fwd(qkv, v1, rope.cos, rope.sin, one, one, one * 0.5, one, B, S, H, Hkv, hd, True),
         2 * ((nq + 2 * nkv) * 2 + nkv)),
        ("qkv_post_bwd", lambda: ops.qkv_post_bwd(dq, dk, dv, qkv, v1, rope.cos, rope.sin, one, one, one * 0.5, one, B, S, H, Hkv, hd, True),
         2 * ((nq + 2 * nkv) * 3 + 2 * nkv)),
        ("gate_fwd", lambda: ops.gate_fwd(o, z), 2 * (2 * nq + T * H)),
        ("gate_bwd", lambda: ops.gate_bwd(dg, o, z), 2 * (3 * nq + 2 * T * H)),
        ("fused_adamw", lambda: ops.fused_adamw(ps, gs, ms, vs, sh, 1e-3, 0.1, 0.9, 0.95, 1e-8, 1e-3), npar * (4 * 4 + 3 * 4 + 2)),
        ("fused_ema", lambda: ops.fused_ema(ema, ps, 0.999), npar * 12),
    ]
    report(rows, a.iters)


def bench_moe(a):
    """Routing and exchange kernels of the MoE block at the IMU-1 MoE shapes on one GPU (T = 8 x 2048 tokens, 16 experts,
    top-2, capacity 1.25): with one rank the peer stores/loads go to local memory, so the figures are HBM fractions."""
    from sample_efficient_gpt_b200.ops import moe as M

    T, d, E, k = 16384, 1152, 16, 2
    x, wr = rnd(T, d), torch.randn(E, d, device="cuda") * 0.1
    cap = M.capacity(T, k, E, 1.25)
    probs, idx, w, slot, totals = M.route(x, wr, k, cap)
    ex = M.PeerExchange(E, None, "cuda")
    xb, _ = ex.dispatch("x", x, idx, slot, totals, None, cap)
    yb = ex.expert_output("y", tuple(xb.shape), torch.bfloat16, "cuda")[0]
    yb.copy_(xb)
    kept = int((slot >= 0).sum())
    dw, aux = torch.randn(T, k, device="cuda"), torch.rand(E, device="cuda")
    rows = [
        ("moe_route (+scan +slots)", lambda: M.route(x, wr, k, cap), T * d * 2 + T * E * 4 + T * k * 12),
        ("moe_push (dispatch)", lambda: ex.dispatch("x", x, idx, slot, totals, None, cap), T * d * 2 + E * cap * d * 2),
        ("moe_push (scaled, backward)", lambda: ex.dispatch("x", x, idx, slot, totals, w, cap), T * d * 2 + E * cap * d * 2),
        ("moe_pull (combine)", lambda: ex.collect("y", yb, idx, slot, w, cap, torch.bfloat16), kept * d * 2 + T * d * 2),
        ("moe_pull (+dots, backward)", lambda: ex.collect("y", yb, idx, slot, None, cap, torch.float32, dot_buf=yb, g=x), 2 * kept * d * 2 + T * d * 2 + T * d * 4),
        ("moe_route_bwd", lambda: M.route_bwd(probs, idx, dw, aux), T * E * 8 + T * k * 8),
    ]
    report(rows, a.iters)


def bench_decode(a):
    """Tokens per second of the one-token decode step of IMU-1 430M (random init, bf16), eager KV-cache decode against the
    CUDA-graph replay of the same step; the prompt is 128 tokens, 128 tokens are generated."""
    import time

    from sample_efficient_gpt_b200.evals.generation import ChatEngine, SamplingParams
    from sample_efficient_gpt_b200.models import build_model
    from sample_efficient_gpt_b200.utils.config_tools import load_cfg

    cfg = load_cfg("imu1_base.yaml", "stable")
    model = build_model(cfg.model).cuda().eval()

    class Tok:
        eos_token_id = None
        chat_template = None

        def get_vocab(self):
            return {}

    for batch in (1, 8):
        prompts = [[(7 * i + j) % 1000 + 10 for j in range(128)] for i in range(batch)]
        row = {"op": "decode", "batch": batch, "new_tokens": 128}
        for name, graphs in (("eager", False), ("cuda_graph", True)):
            eng = ChatEngine(model, Tok(), "cuda", max_model_len=512, cuda_graphs=graphs, cast_weights=True)
            p = SamplingParams(max_tokens=128, temperature=0.0)
            eng.generate_ids([list(x) for x in prompts], p)  # warm-up (and graph capture)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            eng.generate_ids([list(x) for x in prompts], p)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            row[f"{name}_ms_per_token"] = dt / 128 * 1e3
            row[f"{name}_tokens_per_s"] = batch * 128 / dt
        print(json.dumps(row))


def bench_swiglu_gemm(a):
    """The feed-forward's two fused launches against GEMM + element-wise kernel: up projection with SwiGLU in the epilogue,
    and the down projection's data gradient with the SwiGLU backward in the epilogue (IMU-1 shapes: d 1152, F 3072)."""
    from sample_efficient_gpt_b200.ops import gemm as G

    T, d, F = a.tokens, a.k, a.cols
    x, dy = rnd(T, d), rnd(T, d)
    w_up, w_down = rnd(2 * F, d, scale=0.03), rnd(d, F, scale=0.03)
    u = rnd(T, 2 * F, scale=1.0)
    df = G.gemm(dy, w_down, b_mn=True)
    ext = ops.ext()
    t = (lambda fn: time_sustained(fn)) if a.sustained else (lambda fn: timeit(fn, a.iters))
    rows = [
        ("up projection + swiglu, fused", lambda: ext.gemm_swiglu(x, w_up), 2.0 * T * 2 * F * d),
    ]
    if not a.ours_only:
        rows += [("up projection (GEMM alone)", lambda: G.gemm(x, w_up), 2.0 * T * 2 * F * d),
                 ("swiglu_fwd kernel", lambda: ops.swiglu_fwd(u), 0.0)]
    rows.append(("down dgrad + swiglu backward, fused", lambda: ext.gemm_swiglu_bwd(dy, w_down, u), 2.0 * T * F * d))
    if not a.ours_only:
        rows += [("down dgrad (GEMM alone)", lambda: G.gemm(dy, w_down, b_mn=True), 2.0 * T * F * d),
                 ("swiglu_bwd kernel", lambda: ops.swiglu_bwd(df, u), 0.0)]
    for name, fn, flops in rows:
        ms = t(fn)
        print(json.dumps({"op": name, "tokens": T, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1) if flops else None,
                          "mode": "sustained" if a.sustained else "flushed single calls"}))
    torch.cuda.synchronize()
    assert G.status() == 0


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--op", required=True, choices=["gemm", "ns", "attention", "linear_ce", "elementwise", "moe", "decode", "muon", "swiglu_gemm"])
    p.add_argument("--layers", type=int, default=30, help="muon: layers whose four block matrices are stepped")
    p.add_argument("--m", type=int, default=8192)
    p.add_argument("--n", type=int, default=1920)
    p.add_argument("--k", type=int, default=1152)
    p.add_argument("--kind", default="nt", choices=["nt", "nn", "tn"])
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--rows", type=int, default=1152)
    p.add_argument("--cols", type=int, default=3072)
    p.add_argument("--seq", type=int, default=2048)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--tokens", type=int, default=32768, help="linear_ce / swiglu_gemm: rows of the hidden-state matrix")
    p.add_argument("--ours-only", action="store_true", help="linear_ce / muon: skip the comparison arms (profiling runs)")
    p.add_argument("--sustained", action="store_true", help="gemm: time about a second of back-to-back calls (power-capped rate) instead of flushed single calls")
    p.add_argument("--no-split-k", action="store_true", help="gemm: whole tiles only, no tile is cut along the contraction")
    p.add_argument("--shapes", default="", help="gemm: 'block' runs the IMU-1 block shapes (forward, data gradient, weight gradient)")
    a = p.parse_args()
    {"gemm": bench_gemm, "ns": bench_ns, "attention": bench_attention, "linear_ce": bench_linear_ce, "elementwise": bench_elementwise, "moe": bench_moe, "decode": bench_decode, "muon": bench_muon, "swiglu_gemm": bench_swiglu_gemm}[a.op](a)


if __name__ == "__main__":
    main()
