"""
Trainer helpers: RNG state capture/restore and the batched cross-rank reduction of metrics
(role of src/olmo_core/train/utils.py:30-348).

Metrics are recorded per step as device tensors; every ``metrics_collect_interval`` steps they are stacked,
moved once to the bookkeeping device and reduced with ONE sum all-reduce and ONE max all-reduce for the whole
window, so logging costs two small collectives per window rather than one per metric per step.
"""

from __future__ import annotations

import random
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..config import Config
from ..distributed.utils import get_reduce_divide_factor, get_world_size, is_distributed
from .common import ReduceType

__all__ = ["EnvRngStates", "LibRngState", "move_metrics", "reduce_metrics", "check_metrics_consistent",
           "get_metrics_reduce_type_by_step", "get_metric_world_sizes_by_step"]


@dataclass
class LibRngState:
    """One library's generator state with the library version it was taken under."""

    version: Tuple[int, int]
    state: Any


@dataclass
class EnvRngStates(Config):
    """Snapshot of the Python / NumPy / torch (CPU and CUDA) generators."""

    python: Any = None
    numpy: Any = None
    torch: Any = None
    cuda: Any = None

    @classmethod
    def current_state(cls) -> "EnvRngStates":
        return cls(
            python=random.getstate(),
            numpy=np.random.get_state(),
            torch=torch.random.get_rng_state(),
            cuda=torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
        )

    def restore(self) -> bool:
        """Restore what can be restored; returns False if some generator could not be restored."""
        ok = True
        try:
            random.setstate(self.python)
            np.random.set_state(self.numpy)
            torch.random.set_rng_state(self.torch)
        except Exception:
            ok = False
        if self.cuda is not None:
            if torch.cuda.is_available():
                try:
                    torch.cuda.set_rng_state(self.cuda)
                except Exception:
                    ok = False
            else:
                ok = False
        return ok

    def as_dict(self, **kwargs) -> Dict[str, Any]:  # type: ignore[override]
        return dict(python=self.python, numpy=self.numpy, torch=self.torch, cuda=self.cuda)

    @classmethod
    def from_dict(cls, data: Dict[str, Any], overrides=None) -> "EnvRngStates":  # type: ignore[override]
        return cls(**{k: data.get(k) for k in ("python", "numpy", "torch", "cuda")})


def move_metrics(source: Dict[int, Dict[str, torch.Tensor]], device: torch.device) -> Dict[int, Dict[str, torch.Tensor]]:
    """Move a window of metrics ``{step: {name: scalar tensor}}`` to ``device`` with a single stacked copy."""
    keys: List[Tuple[int, str]] = []
    vals: List[torch.Tensor] = []
    for step, metrics in source.items():
        for name, value in metrics.items():
            keys.append((step, name))
            vals.append(value.detach().float().reshape(()))
    out: Dict[int, Dict[str, torch.Tensor]] = {step: {} for step in source}
    if not vals:
        return out
    by_device: Dict[torch.device, List[int]] = {}
    for i, v in enumerate(vals):
        by_device.setdefault(v.device, []).append(i)
    moved: List[Optional[torch.Tensor]] = [None] * len(vals)
    for dev, idxs in by_device.items():
        stacked = torch.stack([vals[i] for i in idxs]).to(device, non_blocking=False)
        for j, i in enumerate(idxs):
            moved[i] = stacked[j]
    for (step, name), v in zip(keys, moved):
        out[step][name] = v  # type: ignore[assignment]
    return out


def check_metrics_consistent(metrics_reduce_type: Dict[str, Optional[ReduceType]],
                             process_group: Optional[dist.ProcessGroup] = None) -> bool:
    """True when every rank recorded the same set of metrics (then a dense reduction is valid)."""
    if not is_distributed() or get_world_size(process_group) == 1:
        return True
    names = sorted(metrics_reduce_type)
    gathered: List[Any] = [None] * get_world_size(process_group)
    dist.all_gather_object(gathered, names, group=process_group)
    return all(g == names for g in gathered)


def reduce_metrics(
    metrics: Dict[int, Dict[str, torch.Tensor]],
    metrics_reduce_type: Dict[str, Optional[ReduceType]],
    device: torch.device,
    process_group: Optional[dist.ProcessGroup] = None,
    metrics_consistent: bool = True,
) -> Dict[int, Dict[str, float]]:
    """
    Reduce a window of metrics across ranks. ``mean`` / ``sum`` / ``l2_norm`` go through one SUM all-reduce
    (l2 norms are squared first; sums are pre-divided by about sqrt(world) for fp range), ``max`` through one
    MAX all-reduce, metrics with reduce type ``None`` are taken from the local rank. A rank that lacks a
    metric contributes zero and does not count towards its mean. With ``metrics_consistent=False`` the ranks first
    exchange which metrics they know (one object gather), so that a metric recorded on some ranks only, e.g. the loss
    on the last pipeline stage, still reduces over buffers of one shape.
    """
    if not metrics_consistent and is_distributed():
        merged: Dict[str, Optional[ReduceType]] = {}
        for per_rank in _gather_reduce_types(metrics_reduce_type, process_group):
            merged.update(per_rank)
        metrics_reduce_type = merged
    steps = sorted(metrics)
    names = sorted({n for m in metrics.values() for n in m} | set(metrics_reduce_type))
    names = [n for n in names if any(n in metrics[s] for s in steps) or metrics_reduce_type.get(n) is not None]
    if not steps or not names:
        return {s: {} for s in steps}
    world = get_world_size(process_group) if is_distributed() else 1
    S, N = len(steps), len(names)
    vals = torch.zeros(S, N, dtype=torch.float32, device=device)
    present = torch.zeros(S, N, dtype=torch.float32, device=device)
    for i, s in enumerate(steps):
        for j, n in enumerate(names):
            v = metrics[s].get(n)
            if v is not None:
                vals[i, j] = v.to(device)
                present[i, j] = 1.0
    kinds = [metrics_reduce_type.get(n) for n in names]
    sum_cols = [j for j, k in enumerate(kinds) if k in (ReduceType.mean, ReduceType.sum, ReduceType.l2_norm)]
    max_cols = [j for j, k in enumerate(kinds) if k == ReduceType.max]
    l2_cols = [j for j, k in enumerate(kinds) if k == ReduceType.l2_norm]
    if world > 1:
        if sum_cols:
            f = get_reduce_divide_factor(world)
            buf = vals[:, sum_cols].clone()
            if l2_cols:
                rel = [sum_cols.index(j) for j in l2_cols]
                buf[:, rel] = buf[:, rel] ** 2
            packed = torch.cat([buf / f, present[:, sum_cols]], dim=1)
            dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=process_group)
            total, count = packed[:, : len(sum_cols)] * f, packed[:, len(sum_cols):]
            for c, j in enumerate(sum_cols):
                if kinds[j] == ReduceType.mean:
                    vals[:, j] = total[:, c] / count[:, c].clamp(min=1.0)
                elif kinds[j] == ReduceType.l2_norm:
                    vals[:, j] = total[:, c].sqrt()
                else:
                    vals[:, j] = total[:, c]
                present[:, j] = (count[:, c] > 0).float()
        if max_cols:
            buf = torch.where(present[:, max_cols] > 0, vals[:, max_cols], torch.full_like(vals[:, max_cols], float("-inf")))
            dist.all_reduce(buf, op=dist.ReduceOp.MAX, group=process_group)
            vals[:, max_cols] = buf
            present[:, max_cols] = torch.isfinite(buf).float()
    host_vals, host_present = vals.cpu(), present.cpu()
    out: Dict[int, Dict[str, float]] = {}
    for i, s in enumerate(steps):
        out[s] = {n: float(host_vals[i, j]) for j, n in enumerate(names) if host_present[i, j] > 0}
    return out


def _gather_reduce_types(metrics_reduce_type, process_group) -> List[Dict[str, Optional[ReduceType]]]:
    if not is_distributed():
        return [metrics_reduce_type]
    gathered: List[Any] = [None] * get_world_size(process_group)
    dist.all_gather_object(gathered, metrics_reduce_type, group=process_group)
    return gathered


def get_metrics_reduce_type_by_step(metrics: Dict[int, Dict[str, torch.Tensor]],
                                    metrics_reduce_type: Dict[str, Optional[ReduceType]],
                                    process_group: Optional[dist.ProcessGroup] = None) -> Dict[int, Dict[str, Optional[ReduceType]]]:
    """For every step, the reduce type of every metric that ANY rank recorded (ranks may record different metrics)."""
    merged: Dict[str, Optional[ReduceType]] = {}
    for per_rank in _gather_reduce_types(metrics_reduce_type, process_group):
        merged.update(per_rank)
    return {step: dict(merged) for step in metrics}


def get_metric_world_sizes_by_step(metrics: Dict[int, Dict[str, torch.Tensor]],
                                   metrics_reduce_type: Dict[str, Optional[ReduceType]],
                                   process_group: Optional[dist.ProcessGroup] = None) -> Dict[int, Dict[str, int]]:
    """For every step, how many ranks recorded each metric (the divisor of a mean over the ranks that have it)."""
    counts: Dict[str, int] = {}
    for per_rank in _gather_reduce_types(metrics_reduce_type, process_group):
        for name in per_rank:
            counts[name] = counts.get(name, 0) + 1
    return {step: dict(counts) for step in metrics}
