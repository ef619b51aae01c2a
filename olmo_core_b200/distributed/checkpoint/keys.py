"""
Key-level utilities on nested state dicts: renaming parameters, pruning keys that a checkpoint lacks and
merging partial state dicts (behaviour of src/olmo_core/distributed/checkpoint/__init__.py:760-1057).

A *flat key* addresses a leaf of a nested dict with ``.``-joined path components, e.g. ``optim.state.w.exp_avg``
is ``sd["optim"]["state.w.exp_avg"]`` or ``sd["optim"]["state"]["w"]["exp_avg"]`` -- both nestings occur, so the
lookups here try every split of the key.
"""

from __future__ import annotations

import logging
from typing import Any, Dict, Iterator, List, Optional, Set, Tuple

from torch.distributed.checkpoint.metadata import Metadata

log = logging.getLogger(__name__)

__all__ = ["swap_param_keys", "prune_state_dict", "merge_state_dicts", "iter_flat_keys", "get_key", "set_key", "pop_key"]


def iter_flat_keys(state_dict: Dict[str, Any], prefix: str = "") -> Iterator[str]:
    for k, v in state_dict.items():
        full = f"{prefix}{k}"
        if isinstance(v, dict):
            yield from iter_flat_keys(v, f"{full}.")
        else:
            yield full


def _locate(state_dict: Dict[str, Any], key: str) -> Optional[Tuple[Dict[str, Any], str]]:
    """The (containing dict, leaf key) of flat ``key``; tries the longest leading component first."""
    if key in state_dict and not isinstance(state_dict[key], dict):
        return state_dict, key
    parts = key.split(".")
    for i in range(len(parts) - 1, 0, -1):
        head, tail = ".".join(parts[:i]), ".".join(parts[i:])
        child = state_dict.get(head)
        if isinstance(child, dict):
            found = _locate(child, tail)
            if found is not None:
                return found
    return None


def get_key(state_dict: Dict[str, Any], key: str, *, pop: bool = False) -> Any:
    found = _locate(state_dict, key)
    if found is None:
        raise KeyError(key)
    container, leaf = found
    return container.pop(leaf) if pop else container[leaf]


def pop_key(state_dict: Dict[str, Any], key: str) -> Any:
    return get_key(state_dict, key, pop=True)


def set_key(state_dict: Dict[str, Any], key: str, value: Any) -> None:
    """Set flat ``key``; descends into existing sub-dicts as far as they match, then stores the remainder flat."""
    parts = key.split(".")
    container = state_dict
    i = 0
    while i < len(parts) - 1:
        # longest existing sub-dict that prefixes the remaining path
        for j in range(len(parts) - 1, i, -1):
            head = ".".join(parts[i:j])
            if isinstance(container.get(head), dict):
                container = container[head]
                i = j
                break
        else:
            break
    container[".".join(parts[i:])] = value


def swap_param_keys(state_dict: Dict[str, Any], key_mapping: Dict[str, str], metadata: Optional[Metadata] = None,
                    reverse: bool = False, quiet: bool = False) -> None:
    """
    Rename parameters in place in a ``{"model": ..., "optim": ...}`` state dict. ``key_mapping`` maps current
    names to checkpoint names; with ``reverse=True`` the renaming is undone. When ``metadata`` is given, a
    parameter is only renamed if the checkpoint really has the new name.
    """
    mapping = {v: k for k, v in key_mapping.items()} if reverse else dict(key_mapping)
    known = set(metadata.state_dict_metadata.keys()) if metadata is not None else None
    flat = list(iter_flat_keys(state_dict))
    for old, new in mapping.items():
        if known is not None and f"model.{new}" not in known:
            continue
        for full in flat:
            # model.<old>, optim.state.<old>.<field>, optim.param_groups.<old>.<field>
            for prefix in ("model.", "optim.state.", "optim.param_groups."):
                if not full.startswith(prefix):
                    continue
                rest = full[len(prefix):]
                if rest == old or rest.startswith(old + "."):
                    renamed = f"{prefix}{new}{rest[len(old):]}"
                    if not quiet:
                        log.info(f"Renaming state dict key '{full}' -> '{renamed}'")
                    set_key(state_dict, renamed, pop_key(state_dict, full))


def prune_state_dict(state_dict: Dict[str, Any], allowed_keys: Set[str]) -> Set[str]:
    """Remove every leaf whose flat key is not in ``allowed_keys``; returns the removed keys."""
    pruned: Set[str] = set()
    for full in list(iter_flat_keys(state_dict)):
        if full not in allowed_keys:
            pop_key(state_dict, full)
            pruned.add(full)
    return pruned


def merge_state_dicts(lhs: Dict[str, Any], rhs: Dict[str, Any]) -> None:
    """Merge ``rhs`` into ``lhs`` in place; nested dicts are merged recursively, leaves of ``rhs`` win."""
    for k, v in rhs.items():
        if isinstance(v, dict) and isinstance(lhs.get(k), dict):
            merge_state_dicts(lhs[k], v)
        else:
            lhs[k] = v
