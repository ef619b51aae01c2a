"""
Show what differs between the configs of two Weights & Biases runs (the role of src/scripts/compare_wandb_configs.py)::

    python -m olmo_core_b200.scripts.compare_wandb_configs entity/project/run_a https://wandb.ai/entity/project/runs/run_b

Both configs are flattened to dotted keys; keys present on one side only and keys whose values differ are listed.
Two local JSON files (as written by the config-saver callback) work as well, which needs no network.
"""

from __future__ import annotations

import argparse
import json
import os
import re
from typing import Any, Dict, Tuple

_URL = re.compile(r"^https?://wandb\.ai/([^/]+)/([^/]+)/runs/([^/?#]+)")
_PATH = re.compile(r"^[^/]+/[^/]+/[^/]+$")


def run_path(spec: str) -> str:
    """``entity/project/run`` from a run path or a run URL."""
    spec = spec.strip().rstrip("/")
    m = _URL.match(spec)
    if m:
        return "/".join(m.groups())
    if _PATH.match(spec):
        return spec
    raise ValueError(f"'{spec}' is neither 'entity/project/run' nor a wandb run URL")


def flatten(d: Any, prefix: str = "") -> Dict[str, Any]:
    if isinstance(d, dict):
        out: Dict[str, Any] = {}
        for k, v in d.items():
            out.update(flatten(v, f"{prefix}{k}."))
        return out
    if isinstance(d, (list, tuple)) and any(isinstance(x, (dict, list)) for x in d):
        out = {}
        for i, v in enumerate(d):
            out.update(flatten(v, f"{prefix}{i}."))
        return out
    return {prefix[:-1]: d}


def load(spec: str) -> Dict[str, Any]:
    if os.path.isfile(spec):
        with open(spec) as f:
            return flatten(json.load(f))
    import wandb

    return flatten(wandb.Api().run(run_path(spec)).config)


def diff(left: Dict[str, Any], right: Dict[str, Any]) -> Tuple[list, list, list]:
    only_left = sorted(set(left) - set(right))
    only_right = sorted(set(right) - set(left))
    changed = sorted(k for k in set(left) & set(right) if left[k] != right[k])
    return only_left, only_right, changed


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("left")
    ap.add_argument("right")
    a = ap.parse_args(argv)
    left, right = load(a.left), load(a.right)
    only_left, only_right, changed = diff(left, right)
    for title, keys, fmt in (("only in left", only_left, lambda k: f"  {k} = {left[k]!r}"),
                             ("only in right", only_right, lambda k: f"  {k} = {right[k]!r}"),
                             ("different", changed, lambda k: f"  {k}: {left[k]!r} -> {right[k]!r}")):
        print(f"{title} ({len(keys)}):")
        for k in keys:
            print(fmt(k))


if __name__ == "__main__":
    main()
