"""
Helpers of the composable data API (role of src/olmo_core/data/composable/utils.py:79-310): a module-wide default seed,
sample-size arithmetic for ratio-based mixing and the chunk-preserving global shuffle.
"""

from __future__ import annotations

import warnings
from typing import Optional, Sequence, TypeVar, Union

import numpy as np
import torch

from ...exceptions import OLMoConfigurationError
from ..utils import get_rng

__all__ = ["SEED_NOT_SET", "resolve_seed", "set_composable_seed", "reset_composable_seed", "calculate_sample_sizes",
           "build_global_indices", "format_token_count", "format_fname_from_fields", "as_ndarray", "as_tensor"]


class _NotSetInt(int):
    """Sentinel type: "use the module-wide seed stream" (an ``int`` so that it type-checks as a seed)."""


SEED_NOT_SET = _NotSetInt()
_seed_stream: Optional[np.random.Generator] = None
S = TypeVar("S", int, None, Optional[int])


def resolve_seed(default: S) -> S:
    """An explicit seed (or ``None``) is returned as is; the sentinel draws the next seed of the module-wide stream."""
    if default is not SEED_NOT_SET:
        return default
    if _seed_stream is None:
        return 0  # type: ignore[return-value]
    return int(_seed_stream.integers(0, 2**31 - 1))  # type: ignore[return-value]


def set_composable_seed(seed: int) -> None:
    """Start the module-wide seed stream: every source built without an explicit seed then gets its own, reproducibly."""
    global _seed_stream
    _seed_stream = get_rng(seed)


def reset_composable_seed() -> None:
    global _seed_stream
    _seed_stream = None


def format_fname_from_fields(prefix: str, **fields) -> str:
    parts = [prefix] + [f"{k}{v}" for k, v in sorted(fields.items()) if v is not None]
    return "_".join(parts)


def format_token_count(n: int) -> str:
    for limit, unit in ((1e12, "T"), (1e9, "B"), (1e6, "M"), (1e3, "K")):
        if n >= limit:
            return f"{n / limit:.1f}{unit}"
    return str(n)


def as_ndarray(array: Union[Sequence[int], Sequence[bool], np.ndarray, torch.Tensor]) -> np.ndarray:
    if isinstance(array, np.ndarray):
        return array
    if isinstance(array, torch.Tensor):
        return array.numpy()
    return np.asarray(array)


def as_tensor(array: Union[Sequence[int], Sequence[bool], np.ndarray, torch.Tensor]) -> torch.Tensor:
    if isinstance(array, torch.Tensor):
        return array
    if isinstance(array, np.ndarray):
        if array.dtype in (np.uint16, np.uint32):
            array = array.astype(np.int64)
        elif array.dtype == np.uint64:
            array = array.astype(np.int64)
        return torch.from_numpy(np.ascontiguousarray(array))
    return torch.as_tensor(array)


def calculate_sample_sizes(source_sizes: Sequence[int], target_ratios: Sequence[float],
                           max_repetition_factors: Sequence[float], target_size: Optional[int] = None,
                           labels: Optional[Sequence[str]] = None, unit: str = "tokens") -> np.ndarray:
    """
    How many items to take from each source so that the mix has the target ratios.

    With ``target_size=None`` the mix is as large as the ratios allow: each source may be repeated up to its
    ``max_repetition_factor`` and the whole mix is scaled down until no source is over-drawn. With a ``target_size`` the
    same computation must reach that size exactly, otherwise an error names the source that limits it.
    """
    sizes = np.asarray(source_sizes, dtype=np.float64)
    ratios = np.asarray(target_ratios, dtype=np.float64)
    max_rep = np.asarray(max_repetition_factors, dtype=np.float64)
    if not (len(sizes) == len(ratios) == len(max_rep)) or (labels is not None and len(labels) != len(sizes)):
        raise ValueError("source sizes, ratios, repetition factors and labels must have the same length")
    if not (ratios > 0).all():
        raise ValueError(f"All ratios must be positive! Got {list(target_ratios)}")
    if not (max_rep >= 1.0).all():
        raise ValueError(f"All max repetition factors must be at least 1.0! Got {list(max_repetition_factors)}")
    if not (sizes > 0).all():
        raise ValueError(f"All source sizes must be positive! Got {list(source_sizes)}")

    def name(i: int) -> str:
        return f"'{labels[i]}'" if labels is not None else str(i)

    if not np.isclose(ratios.sum(), 1.0):
        normalized = ratios / ratios.sum()
        lines = "\n".join(f" ❯ Source {name(i)}: target ratio adjusted from {target_ratios[i]} to {normalized[i]}"
                          for i in range(len(ratios)))
        warnings.warn(f"Target mixing ratios don't sum to 1. They will be normalized as follows:\n{lines}", UserWarning)
        ratios = normalized

    strict = target_size is not None
    goal = float(target_size) if strict else float(sizes.sum())
    ideal = goal * ratios  # what each source would contribute if it were large enough
    needed_rep = np.maximum(ideal / sizes, 1.0)
    available = sizes * np.minimum(max_rep, needed_rep)
    shrink = min(1.0, float((available / ideal).min()))  # scale the whole mix so that the scarcest source suffices
    actual = ideal * shrink
    result = actual.astype(np.uint64)
    assert (result <= available).all()
    if strict and not np.isclose(goal, actual.sum()):
        worst = int(np.argmax(needed_rep - max_rep))
        raise OLMoConfigurationError(
            f"Unable to meet target size of {int(goal):,d} {unit} with the given source ratios and max repetition "
            f"factors. The best we can do is {int(actual.sum()):,d} {unit}. The source with the biggest discrepancy "
            f"between its required sample size (~{int(ideal[worst]):,d} {unit}, {100 * ratios[worst]:.1f}% of mix) and "
            f"the size it can provide after accounting for the max repetition factor ({int(sizes[worst]):,d} x "
            f"{max_rep[worst]:.2f} ~= {int(sizes[worst] * max_rep[worst]):,d} {unit}) is the source {name(worst)}. "
            f"Consider either decreasing the target size of the mix to {int(actual.sum()):,d} {unit} or increasing the "
            f"max repetition factor for that source to {needed_rep[worst]:.2f}.")
    return result


def build_global_indices(total_instances: int, *, sequence_length: int, max_sequence_length: int, seed: Optional[int],
                         dtype=np.uint32) -> np.ndarray:
    """
    Shuffled instance order that is stable under a change of ``sequence_length`` with ``max_sequence_length`` fixed:
    instances are permuted in groups of ``max_sequence_length // sequence_length`` neighbours, so the same text is seen
    in the same order whichever way it is cut.
    """
    if total_instances >= np.iinfo(dtype).max:
        raise ValueError("too many instances for the index dtype")
    if max_sequence_length % sequence_length != 0:
        raise ValueError("max_sequence_length must be a multiple of sequence_length")
    group = max_sequence_length // sequence_length
    if total_instances % group != 0:
        raise ValueError("the number of instances must be a multiple of max_sequence_length // sequence_length")
    order = np.arange(total_instances // group, dtype=dtype)
    if seed is not None:
        get_rng(seed).shuffle(order)
    if group == 1:
        return order
    return (order[:, None] * group + np.arange(group, dtype=dtype)[None, :]).reshape(-1)


def path_map(func, paths, *, max_workers: Optional[int] = None, method: str = "threads"):
    """
    ``[func(p) for p in paths]`` computed by a pool of threads or processes, results in the order of ``paths``
    (src/olmo_core/data/composable/utils.py:41-90). ``max_workers=0`` runs in the calling thread.
    """
    import concurrent.futures

    paths = list(paths)
    if max_workers == 0 or len(paths) <= 1:
        return [func(p) for p in paths]
    if method == "threads":
        pool_cls = concurrent.futures.ThreadPoolExecutor
    elif method == "processes":
        pool_cls = concurrent.futures.ProcessPoolExecutor
    else:
        raise ValueError(method)
    with pool_cls(max_workers=max_workers) as pool:
        return list(pool.map(func, paths))
