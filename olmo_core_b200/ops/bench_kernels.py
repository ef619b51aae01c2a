"""
Micro-benchmarks of the sm_100a kernels against their library counterparts.

``python -m olmo_core_b200.ops.bench_kernels <case> [--iters N] [--profile]`` with ``case`` one of ``gemm``, ``mlp`` (gated
MLP with the activation in the GEMM epilogues), ``fp8``, ``mx``, ``grouped``, ``attention``, ``norm``, ``norm_rope``,
``swiglu``, ``ce``, ``adamw``, ``router``.

Each case is timed with CUDA events on the launching stream after warm-up, with a buffer larger than L2 rewritten
between iterations, and printed as one JSON line per case: milliseconds, achieved TFLOP/s or GB/s, and the same
figure for the library kernel (cuBLAS through ``torch.matmul``, cuDNN / flash attention through
``scaled_dot_product_attention``, ``torch.nn.functional.rms_norm``). ``--peaks FILE`` names a JSON file with
``bf16_tflops`` / ``hbm_gbs`` entries; when given, fractions of those peaks are added.

``--profile`` launches every kernel of the case exactly once with no timing loop, which is the form to run under a
profiler restricted to a few launches of one kernel.
"""

from __future__ import annotations

import argparse
import json
import math
from typing import Callable, Dict, Optional

import torch

_flush: Optional[torch.Tensor] = None


def _flush_l2() -> None:
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_ms(fn: Callable[[], None], iters: int, warmup: int = 3) -> float:
    """Median device time of ``fn`` over ``iters`` runs, L2 flushed before each."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        _flush_l2()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def _emit(row: Dict, peaks: Optional[Dict]) -> None:
    if peaks:
        if "tflops" in row and peaks.get("bf16_tflops"):
            row["frac_of_measured_bf16"] = round(row["tflops"] / float(peaks["bf16_tflops"]), 3)
        if "gbs" in row and peaks.get("hbm_gbs"):
            row["frac_of_measured_hbm"] = round(row["gbs"] / float(peaks["hbm_gbs"]), 3)
    print(json.dumps(row), flush=True)


def bench_gemm(args, peaks) -> None:
    from .gemm import gemm

    # the projections of a 7B layer at 8192 tokens: QKV/out (4096x4096) and the MLP (11008x4096), all three passes
    shapes = [(8192, 4096, 4096), (8192, 11008, 4096), (8192, 4096, 11008)]
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        g = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        dw = torch.zeros(N, K, device="cuda", dtype=torch.float32)
        cases = {
            "fwd_nt": (lambda: gemm(a, w, trans_b=True), lambda: torch.matmul(a, w.t())),
            "dgrad_nn": (lambda: gemm(g, w, trans_b=False), lambda: torch.matmul(g, w)),
            "wgrad_tn_f32acc": (lambda: gemm(g, a, trans_a=True, trans_b=False, out=dw, accumulate=True),
                                lambda: torch.matmul(g.t(), a)),
        }
        for name, (ours, library) in cases.items():
            if args.profile:
                ours()
                continue
            flops = 2.0 * M * N * K
            t_ours, t_lib = time_ms(ours, args.iters), time_ms(library, args.iters)
            _emit({"kernel": "gemm_" + name, "M": M, "N": N, "K": K, "ms": round(t_ours, 4),
                   "tflops": round(flops / t_ours / 1e9, 1), "library_ms": round(t_lib, 4),
                   "library_tflops": round(flops / t_lib / 1e9, 1)}, peaks)
    torch.cuda.synchronize()


def bench_attention(args, peaks) -> None:
    from .attention import attention

    B, T, H, D = 2, 4096, 32, 128
    q, k, v = (torch.randn(B, T, H, D, device="cuda", dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    do = torch.randn(B, T, H, D, device="cuda", dtype=torch.bfloat16)
    if args.profile:
        attention(q, k, v).backward(do)
        torch.cuda.synchronize()
        return
    fwd_flops = 4.0 * B * H * T * T * D / 2  # causal: half of the score matrix
    bwd_flops = 2.5 * fwd_flops

    def sdpa():
        return torch.nn.functional.scaled_dot_product_attention(
            q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), is_causal=True).permute(0, 2, 1, 3)

    for name, fn in (("ours", lambda: attention(q, k, v)), ("library_sdpa", sdpa)):
        with torch.no_grad():
            t_f = time_ms(fn, args.iters)
        out = fn()
        t_b = time_ms(lambda: torch.autograd.grad(out, (q, k, v), do, retain_graph=True), args.iters)
        _emit({"kernel": "attention_causal_" + name, "B": B, "T": T, "H": H, "D": D, "fwd_ms": round(t_f, 4),
               "fwd_tflops": round(fwd_flops / t_f / 1e9, 1), "bwd_ms": round(t_b, 4),
               "bwd_tflops": round(bwd_flops / t_b / 1e9, 1)}, None)
    for window, docs in ((1024, False), (0, True)):
        cu = torch.tensor([0, 1000, 2500, 4096, 4096 + 3000, 2 * 4096], device="cuda", dtype=torch.int32) if docs else None
        kw = dict(window_size=window or None, cu_seqlens=cu)
        with torch.no_grad():
            t_f = time_ms(lambda: attention(q, k, v, **kw), args.iters)
        out = attention(q, k, v, **kw)
        t_b = time_ms(lambda: torch.autograd.grad(out, (q, k, v), do, retain_graph=True), args.iters)
        _emit({"kernel": "attention_ours_" + ("documents" if docs else f"window{window}"), "fwd_ms": round(t_f, 4),
               "bwd_ms": round(t_b, 4)}, None)


def bench_norm(args, peaks) -> None:
    from .elementwise import rms_norm as rmsnorm

    rows, cols = 8192, 4096
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(cols, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    if args.profile:
        rmsnorm(x, w, 1e-6).backward(g)
        torch.cuda.synchronize()
        return
    nbytes = 2.0 * rows * cols * 2
    for name, fn in (("ours", lambda: rmsnorm(x, w, 1e-6)),
                     ("library", lambda: torch.nn.functional.rms_norm(x, (cols,), w, 1e-6))):
        with torch.no_grad():
            t_f = time_ms(fn, args.iters)
        out = fn()
        t_b = time_ms(lambda: torch.autograd.grad(out, (x, w), g, retain_graph=True), args.iters)
        _emit({"kernel": "rmsnorm_" + name, "rows": rows, "cols": cols, "fwd_ms": round(t_f, 4),
               "gbs": round(nbytes / t_f / 1e6, 1), "bwd_ms": round(t_b, 4),
               "bwd_gbs": round(1.5 * nbytes / t_b / 1e6, 1)}, peaks)
    # The backward numbers above include the host's launch gaps between the four launches of an autograd call. The
    # kernels alone, through the C entry points with every buffer allocated once (with and without the residual):
    from . import _lib

    L, st = _lib.lib(), _lib.stream_ptr()
    res = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    y, dx = torch.empty_like(g), torch.empty_like(g)
    rstd = torch.empty(rows, device="cuda", dtype=torch.float32)
    partial = torch.empty(L.ocb_norm_bwd_partials(), cols, device="cuda", dtype=torch.float32)
    xd, wd = x.detach(), w.detach()
    bf = _lib.dt(xd)

    def fwd(r):
        _lib.check(L.ocb_rmsnorm_fwd(xd.data_ptr(), wd.data_ptr(), _lib.ptr(r), y.data_ptr(), rstd.data_ptr(), rows, cols,
                                     cols, cols, cols, cols if r is not None else 0, 1e-6, bf, bf, st), "ocb_rmsnorm_fwd")

    def bwd():
        _lib.check(L.ocb_rmsnorm_bwd(g.data_ptr(), xd.data_ptr(), wd.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                     partial.data_ptr(), rows, cols, cols, cols, cols, cols, bf, bf, st), "ocb_rmsnorm_bwd")

    t0, t1, t2 = time_ms(lambda: fwd(None), args.iters), time_ms(lambda: fwd(res), args.iters), time_ms(bwd, args.iters)
    _emit({"kernel": "rmsnorm_kernels_only", "rows": rows, "cols": cols, "fwd_ms": round(t0, 4),
           "gbs": round(nbytes / t0 / 1e6, 1), "fwd_residual_ms": round(t1, 4),
           "fwd_residual_gbs": round(1.5 * nbytes / t1 / 1e6, 1), "bwd_ms": round(t2, 4),
           "bwd_gbs": round(1.5 * nbytes / t2 / 1e6, 1), "note": "bwd includes clearing the partial rows"}, peaks)


def bench_mlp(args, peaks) -> None:
    """Gated MLP of a 7B layer: fused up-projection (a | b and silu(a) * b in one epilogue) and fused backward through it."""
    from . import _lib
    from .elementwise import swiglu
    from .gemm import gemm

    M, H, K = 8192, 11008, 4096
    L = _lib.lib()
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w13 = torch.randn(2 * H, K, device="cuda", dtype=torch.bfloat16) * 0.02
    w2 = torch.randn(K, H, device="cuda", dtype=torch.bfloat16) * 0.02
    dy = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    ab = torch.empty(M, 2 * H, device="cuda", dtype=torch.bfloat16)
    dab = torch.empty_like(ab)
    h = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    st = _lib.status_buffer(torch.device("cuda")).data_ptr()

    def fused_fwd():
        _lib.check(L.ocb_gemm_swiglu_fwd(x.data_ptr(), w13.data_ptr(), ab.data_ptr(), h.data_ptr(), M, H, K, K, K, 2 * H, H,
                                         st, _lib.stream_ptr()), "ocb_gemm_swiglu_fwd")

    def fused_bwd():
        _lib.check(L.ocb_gemm_swiglu_bwd(dy.data_ptr(), w2.data_ptr(), ab.data_ptr(), dab.data_ptr(), None, M, H, K, K, H,
                                         2 * H, 2 * H, H, st, _lib.stream_ptr()), "ocb_gemm_swiglu_bwd")

    a_ = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    b_ = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    dh = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)

    def unfused_fwd():
        gemm(x, w13[:H], trans_b=True, out=a_)
        gemm(x, w13[H:], trans_b=True, out=b_)
        with torch.no_grad():
            swiglu(a_, b_)

    a_g, b_g = a_.clone().requires_grad_(True), b_.clone().requires_grad_(True)
    h_g = swiglu(a_g, b_g)

    def unfused_bwd():
        gemm(dy, w2, trans_b=False, out=dh)
        torch.autograd.grad(h_g, (a_g, b_g), dh, retain_graph=True)

    if args.profile:
        fused_fwd()
        fused_bwd()
        torch.cuda.synchronize()
        return
    for name, fn, flops in (("mlp_up_fused_swiglu", fused_fwd, 2.0 * M * 2 * H * K),
                            ("mlp_up_two_gemms_plus_swiglu_kernel", unfused_fwd, 2.0 * M * 2 * H * K),
                            ("mlp_down_dgrad_fused_swiglu_bwd", fused_bwd, 2.0 * M * H * K),
                            ("mlp_down_dgrad_plus_swiglu_bwd_kernel", unfused_bwd, 2.0 * M * H * K)):
        t = time_ms(fn, args.iters)
        _emit({"kernel": name, "M": M, "H": H, "K": K, "ms": round(t, 4), "tflops": round(flops / t / 1e9, 1)}, peaks)
    _lib.check_device_status()


def bench_fp8(args, peaks) -> None:
    from .fp8 import gemm_fp8, quantize_colwise_transposed, quantize_rowwise

    M, N, K = 8192, 4096, 4096
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    aq, asc = quantize_rowwise(a)
    wq, wsc = quantize_rowwise(w)
    if args.profile:
        quantize_rowwise(a)
        quantize_colwise_transposed(a)
        gemm_fp8(aq, asc, wq, wsc)
        torch.cuda.synchronize()
        return
    t = time_ms(lambda: gemm_fp8(aq, asc, wq, wsc), args.iters)
    _emit({"kernel": "gemm_e4m3_rowwise", "M": M, "N": N, "K": K, "ms": round(t, 4),
           "tflops": round(2.0 * M * N * K / t / 1e9, 1)}, None)
    for name, fn in (("quantize_e4m3_rowwise", lambda: quantize_rowwise(a)),
                     ("quantize_e4m3_colwise_transposed", lambda: quantize_colwise_transposed(a))):
        t = time_ms(fn, args.iters)
        _emit({"kernel": name, "rows": M, "cols": K, "ms": round(t, 4), "gbs": round(M * K * 3.0 / t / 1e6, 1)}, peaks)


def bench_mx(args, peaks) -> None:
    """Block-scaled (MX) e4m3 GEMM on the 7B layer shapes, its two quantisers, and a whole linear layer fwd+bwd next to bf16."""
    from .gemm import linear
    from .mx import gemm_mx, mx_linear, quantize_mx_colwise_transposed, quantize_mx_rowwise

    M = 8192
    a = torch.randn(M, 4096, device="cuda", dtype=torch.bfloat16)
    if args.profile:
        w = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
        aq, asf = quantize_mx_rowwise(a)
        wq, wsf = quantize_mx_rowwise(w)
        quantize_mx_colwise_transposed(a)
        gemm_mx(aq, asf, wq, wsf)
        torch.cuda.synchronize()
        return
    for N, K in ((4096, 4096), (22016, 4096), (4096, 11008)):
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        xq, xsf = quantize_mx_rowwise(x)
        wq, wsf = quantize_mx_rowwise(w)
        t = time_ms(lambda: gemm_mx(xq, xsf, wq, wsf), args.iters)
        tl = time_ms(lambda: torch.matmul(x, w.t()), args.iters)
        _emit({"kernel": "gemm_mx_e4m3", "M": M, "N": N, "K": K, "ms": round(t, 4), "tflops": round(2.0 * M * N * K / t / 1e9, 1),
               "cublas_bf16_ms": round(tl, 4)}, None)
    for name, fn in (("quantize_mx_rowwise", lambda: quantize_mx_rowwise(a)),
                     ("quantize_mx_colwise_transposed", lambda: quantize_mx_colwise_transposed(a))):
        t = time_ms(fn, args.iters)
        _emit({"kernel": name, "rows": M, "cols": 4096, "ms": round(t, 4), "gbs": round(M * 4096 * 3.0 / t / 1e6, 1)}, peaks)
    for N, K in ((4096, 4096), (11008, 4096)):
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)

        def run(fn):
            x.grad = w.grad = None
            fn(x, w).backward(dy)

        t_mx = time_ms(lambda: run(mx_linear), args.iters)
        t_bf = time_ms(lambda: run(linear), args.iters)
        _emit({"kernel": "linear_fwd_bwd", "M": M, "N": N, "K": K, "mx_ms": round(t_mx, 4), "bf16_ms": round(t_bf, 4),
               "speedup": round(t_bf / t_mx, 3)}, None)


def bench_grouped(args, peaks) -> None:
    """Expert MLP shapes of OLMoE-1B-7B: 64 experts, d_model 2048, hidden 1024, 32768 x 8 routed rows."""
    from .gemm import grouped_gemm, grouped_gemm_wgrad

    E, D, Hh, R = 64, 2048, 1024, 32768 * 8
    x = torch.randn(R, D, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E * Hh, D, device="cuda", dtype=torch.bfloat16) * 0.02
    counts = torch.full((E,), R // E, dtype=torch.int32, device="cuda")
    offsets = torch.cat([torch.zeros(1, dtype=torch.int32, device="cuda"), counts.cumsum(0).to(torch.int32)])
    g = torch.randn(R, Hh, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(E * Hh, D, device="cuda", dtype=torch.float32)
    if args.profile:
        grouped_gemm(x, w, offsets, trans_b=True)
        grouped_gemm_wgrad(g, x, offsets, dw, accumulate=True)
        torch.cuda.synchronize()
        return
    flops = 2.0 * R * Hh * D
    t = time_ms(lambda: grouped_gemm(x, w, offsets, trans_b=True), args.iters)
    _emit({"kernel": "grouped_gemm_rows", "experts": E, "rows": R, "N": Hh, "K": D, "ms": round(t, 4),
           "tflops": round(flops / t / 1e9, 1)}, peaks)
    t = time_ms(lambda: grouped_gemm_wgrad(g, x, offsets, dw, accumulate=True), args.iters)
    _emit({"kernel": "grouped_gemm_wgrad_f32acc", "experts": E, "rows": R, "M": Hh, "N": D, "ms": round(t, 4),
           "tflops": round(flops / t / 1e9, 1)}, peaks)


def bench_norm_rope(args, peaks) -> None:
    from .elementwise import norm_rope

    B, S, H, D = 2, 4096, 32, 128
    x = torch.randn(B, S, H * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(H * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    pos = torch.arange(S, device="cuda", dtype=torch.float32)[:, None]
    inv = 1.0 / (500000 ** (torch.arange(0, D, 2, device="cuda", dtype=torch.float32) / D))
    ang = torch.cat([pos * inv, pos * inv], dim=-1)
    sin, cos = ang.sin().contiguous(), ang.cos().contiguous()
    g = torch.randn_like(x)
    if args.profile:
        norm_rope(x, w, sin, cos, H).backward(g)
        torch.cuda.synchronize()
        return
    nbytes = 2.0 * x.numel() * 2
    with torch.no_grad():
        t_f = time_ms(lambda: norm_rope(x, w, sin, cos, H), args.iters)
    out = norm_rope(x, w, sin, cos, H)
    t_b = time_ms(lambda: torch.autograd.grad(out, (x, w), g, retain_graph=True), args.iters)
    _emit({"kernel": "qk_norm_rope", "tokens": B * S, "width": H * D, "fwd_ms": round(t_f, 4), "gbs": round(nbytes / t_f / 1e6, 1),
           "bwd_ms": round(t_b, 4), "bwd_gbs": round(1.5 * nbytes / t_b / 1e6, 1)}, peaks)
    # kernels alone (no autograd, no allocation; the backward call includes clearing the partial rows)
    from . import _lib

    L, st = _lib.lib(), _lib.stream_ptr()
    rows, cols = B * S, H * D
    xd, wd = x.detach().view(rows, cols), w.detach()
    y, dx, g2 = torch.empty_like(xd), torch.empty_like(xd), g.view(rows, cols)
    rstd = torch.empty(rows, device="cuda", dtype=torch.float32)
    partial = torch.empty(L.ocb_norm_bwd_partials(), cols, device="cuda", dtype=torch.float32)
    bf = _lib.dt(xd)

    def fwd():
        _lib.check(L.ocb_norm_rope_fwd(xd.data_ptr(), wd.data_ptr(), y.data_ptr(), rstd.data_ptr(), sin.data_ptr(),
                                       cos.data_ptr(), None, rows, H, D, S, 0, 1, cols, cols, 1e-6, bf, bf, st),
                   "ocb_norm_rope_fwd")

    def bwd():
        _lib.check(L.ocb_norm_rope_bwd(g2.data_ptr(), xd.data_ptr(), wd.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                       partial.data_ptr(), sin.data_ptr(), cos.data_ptr(), None, rows, H, D, S, 0, 1, cols,
                                       cols, cols, bf, bf, st), "ocb_norm_rope_bwd")

    t0, t1 = time_ms(fwd, args.iters), time_ms(bwd, args.iters)
    _emit({"kernel": "qk_norm_rope_kernels_only", "tokens": rows, "width": cols, "fwd_ms": round(t0, 4),
           "gbs": round(nbytes / t0 / 1e6, 1), "bwd_ms": round(t1, 4), "bwd_gbs": round(1.5 * nbytes / t1 / 1e6, 1)}, peaks)


def bench_swiglu(args, peaks) -> None:
    from .elementwise import swiglu

    rows, cols = 8192, 11008
    a = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    if args.profile:
        swiglu(a, b).backward(g)
        torch.cuda.synchronize()
        return
    n = rows * cols * 2.0
    with torch.no_grad():
        t_f = time_ms(lambda: swiglu(a, b), args.iters)
    out = swiglu(a, b)
    t_b = time_ms(lambda: torch.autograd.grad(out, (a, b), g, retain_graph=True), args.iters)
    _emit({"kernel": "swiglu_standalone", "rows": rows, "cols": cols, "fwd_ms": round(t_f, 4), "gbs": round(3 * n / t_f / 1e6, 1),
           "bwd_ms": round(t_b, 4), "bwd_gbs": round(5 * n / t_b / 1e6, 1)}, peaks)


def bench_ce(args, peaks) -> None:
    """LM head + loss of the 7B model on one 8192-token micro-batch (vocabulary 100352)."""
    from .loss import fused_linear_cross_entropy

    T, V, D = 8192, 100352, 4096
    h = torch.randn(T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(V, D, device="cuda", dtype=torch.bfloat16) * 0.02).requires_grad_(True)
    labels = torch.randint(0, V, (T,), device="cuda")

    def step():
        ce, z = fused_linear_cross_entropy(h, w, labels, z_loss_multiplier=1e-5)
        (ce + z).backward()
        h.grad = None
        w.grad = None

    if args.profile:
        step()
        torch.cuda.synchronize()
        return
    t = time_ms(step, max(3, args.iters // 2))
    _emit({"kernel": "fused_linear_cross_entropy_fwd_bwd", "tokens": T, "vocab": V, "d_model": D, "ms": round(t, 4),
           "tflops": round(3 * 2.0 * T * V * D / t / 1e9, 1)}, peaks)


def bench_adamw(args, peaks) -> None:
    from .optim import adamw_step_, sumsq

    n = 202_391_552  # one 7B block
    p, m, v, g = (torch.randn(n, device="cuda") * 0.01 for _ in range(4))
    v.abs_()
    lowp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    step = torch.ones((), device="cuda")

    def run():
        adamw_step_(p, m, v, g, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, step=step, lowp=lowp)

    if args.profile:
        run()
        sumsq(g)
        torch.cuda.synchronize()
        return
    t = time_ms(run, args.iters)
    _emit({"kernel": "adamw_fp32_master_bf16_copy", "numel": n, "ms": round(t, 4), "gbs": round(n * 30.0 / t / 1e6, 1)}, peaks)
    t = time_ms(lambda: sumsq(g), args.iters)
    _emit({"kernel": "sum_of_squares", "numel": n, "ms": round(t, 4), "gbs": round(n * 4.0 / t / 1e6, 1)}, peaks)


def bench_router(args, peaks) -> None:
    from ..nn.moe.router import _FusedSoftmaxTopK
    from .moe import indices_and_bins

    N, E, k = 32768, 64, 8
    logits = torch.randn(N, E, device="cuda", dtype=torch.bfloat16)
    if args.profile:
        _, _, ids, _ = _FusedSoftmaxTopK.apply(logits, k)
        indices_and_bins(ids, E)
        torch.cuda.synchronize()
        return
    with torch.no_grad():
        t = time_ms(lambda: _FusedSoftmaxTopK.apply(logits, k), args.iters)
        _emit({"kernel": "router_softmax_topk", "tokens": N, "experts": E, "top_k": k, "ms": round(t, 4),
               "gbs": round((N * E * 6.0 + N * k * 8.0) / t / 1e6, 1)}, peaks)
        ids = _FusedSoftmaxTopK.apply(logits, k)[2]
        t = time_ms(lambda: indices_and_bins(ids, E), args.iters)
        _emit({"kernel": "routing_counting_sort", "copies": N * k, "ms": round(t, 4)}, None)
        t = time_ms(lambda: torch.sort(ids.reshape(-1), stable=True), args.iters)
        _emit({"kernel": "routing_torch_sort_library", "copies": N * k, "ms": round(t, 4)}, None)


CASES = {"gemm": bench_gemm, "mlp": bench_mlp, "fp8": bench_fp8, "mx": bench_mx, "grouped": bench_grouped, "attention": bench_attention,
         "norm": bench_norm, "norm_rope": bench_norm_rope, "swiglu": bench_swiglu, "ce": bench_ce, "adamw": bench_adamw,
         "router": bench_router}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--peaks", default=None)
    args = ap.parse_args(argv)
    peaks = json.load(open(args.peaks)) if args.peaks else None
    torch.manual_seed(0)
    CASES[args.case](args, peaks)
    assert math.isfinite(torch.cuda.memory_allocated())


if __name__ == "__main__":
    main()
