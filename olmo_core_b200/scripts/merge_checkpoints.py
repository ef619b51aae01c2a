"""
Average the model weights of several checkpoints of one run ("model soup"; role of src/scripts/merge_core_checkpoints.py)::

    python -m olmo_core_b200.scripts.merge_checkpoints OUT_DIR CKPT_A CKPT_B [CKPT_C ...] [--weights 0.5 0.25 0.25]

Every input is unsharded key by key (no model is built, so this runs on a CPU box for any model size); the result is a
distributed checkpoint of the same layout with ``model`` entries only, loadable with ``Trainer.load_checkpoint(...,
load_optim_state=False, load_trainer_state=False)``.
"""

import argparse
from typing import Dict, List, Optional

import torch

from ..distributed.checkpoint import get_checkpoint_metadata, load_keys, save_state_dict
from ..io import join_path, normalize_path
from ..utils import prepare_cli_environment


def merge(out_dir: str, checkpoints: List[str], weights: Optional[List[float]] = None, overwrite: bool = False) -> None:
    if weights is None:
        weights = [1.0 / len(checkpoints)] * len(checkpoints)
    if len(weights) != len(checkpoints) or abs(sum(weights) - 1.0) > 1e-6:
        raise ValueError("one weight per checkpoint, summing to 1")
    dirs = [d if d.rstrip("/").endswith("model_and_optim") else join_path(normalize_path(d), "model_and_optim")
            for d in checkpoints]
    keys = sorted(k for k in get_checkpoint_metadata(dirs[0]).state_dict_metadata if k.startswith("model."))
    merged: Dict[str, torch.Tensor] = {}
    for key in keys:
        total = None
        for d, w in zip(dirs, weights):
            (t,) = load_keys(d, [key])
            total = t.float() * w if total is None else total + t.float() * w
            dtype = t.dtype
        merged[key[len("model."):]] = total.to(dtype)
    save_state_dict(join_path(normalize_path(out_dir), "model_and_optim"), {"model": merged}, save_overwrite=overwrite)


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("out_dir")
    p.add_argument("checkpoints", nargs="+")
    p.add_argument("--weights", type=float, nargs="*", default=None)
    p.add_argument("--overwrite", action="store_true")
    args = p.parse_args(argv)
    prepare_cli_environment()
    merge(args.out_dir, args.checkpoints, args.weights, args.overwrite)
    print(f"merged {len(args.checkpoints)} checkpoints into {args.out_dir}")


if __name__ == "__main__":
    main()
