"""
Micro-benchmarks of the sm_100a kernels against their library counterparts.

``python -m olmo_core_b200.ops.bench_kernels <gemm|attention|norm> [--iters N] [--profile]``

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


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=["gemm", "attention", "norm"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--peaks", default=None)
    args = ap.parse_args(argv)
    peaks = json.load(open(args.peaks)) if args.peaks else None
    torch.manual_seed(0)
    {"gemm": bench_gemm, "attention": bench_attention, "norm": bench_norm}[args.case](args, peaks)
    assert math.isfinite(torch.cuda.memory_allocated())


if __name__ == "__main__":
    main()
