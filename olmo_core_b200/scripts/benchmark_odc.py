"""
Memory and time of :class:`olmo_core_b200.nn.output_discard_checkpoint.OutputDiscardCheckpoint` against plain autograd and against
``torch.utils.checkpoint`` (the role of src/scripts/benchmark_odc.py)::

    python -m olmo_core_b200.scripts.benchmark_odc [--d-model 2048 --d-ff 8192 --batch 2 --seq 2048 --n-layers 4]

Output-discard checkpointing frees a region's (large) output right after its consumer has used it and recomputes it in
the backward pass; what it saves only shows when several such regions are stacked, because the freed output of layer
``i`` is memory that layers ``i+1 ..`` can use. Each case therefore runs a stack of ``--n-layers`` "up-projection ->
activation -> down-projection" layers three ways and prints peak memory and forward+backward time (CUDA events).
"""

from __future__ import annotations

import argparse
import json

import torch
import torch.nn as nn


class _Layer(nn.Module):
    def __init__(self, d: int, f: int, mode: str):
        super().__init__()
        self.up = nn.Linear(d, f, bias=False)
        self.down = nn.Linear(f, d, bias=False)
        self.mode = mode

    def forward(self, x):
        if self.mode == "odc":
            from ..nn.output_discard_checkpoint import OutputDiscardCheckpoint

            odc = OutputDiscardCheckpoint()
            h = odc.checkpoint(lambda t: torch.nn.functional.silu(self.up(t)), x)  # the fat [tokens, d_ff] tensor
            y = self.down(h)
            odc.discard_output_and_register_recompute(y)  # h's memory is free from here until the backward pass
            return x + y
        if self.mode == "checkpoint":
            from torch.utils.checkpoint import checkpoint

            h = checkpoint(lambda t: torch.nn.functional.silu(self.up(t)), x, use_reentrant=False)
            return x + self.down(h)
        return x + self.down(torch.nn.functional.silu(self.up(x)))


def run(mode: str, a) -> dict:
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    torch.manual_seed(0)
    model = nn.Sequential(*[_Layer(a.d_model, a.d_ff, mode) for _ in range(a.n_layers)]).to(dev, torch.bfloat16)
    x = torch.randn(a.batch * a.seq, a.d_model, device=dev, dtype=torch.bfloat16, requires_grad=True)
    times = []
    for it in range(a.iters + 2):
        if dev.type == "cuda":
            torch.cuda.reset_peak_memory_stats()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        model(x).float().pow(2).mean().backward()
        if dev.type == "cuda":
            stop.record()
            torch.cuda.synchronize()
            if it >= 2:
                times.append(start.elapsed_time(stop))
        model.zero_grad(set_to_none=True)
        x.grad = None
    peak = torch.cuda.max_memory_allocated() / 2**20 if dev.type == "cuda" else float("nan")
    times.sort()
    return {"mode": mode, "peak_mib": round(peak, 1), "ms": round(times[len(times) // 2], 3) if times else None}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--d-ff", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--n-layers", type=int, default=4)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args(argv)
    for mode in ("baseline", "checkpoint", "odc"):
        print(json.dumps(run(mode, a)), flush=True)


if __name__ == "__main__":
    main()
