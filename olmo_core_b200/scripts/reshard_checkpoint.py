"""
Rewrite a sharded checkpoint with another number of shards (the role of src/scripts/reshard_core_checkpoint.py)::

    python -m olmo_core_b200.scripts.reshard_checkpoint /runs/r/step1000/model_and_optim /tmp/resharded --ranks 4 \
        [--skip-optimizer-state]

A checkpoint written by N ranks holds N files per save (``__<rank>_<i>.distcp``); loading it on a very different
world size still works but reads every file from every rank. This tool spawns ``--ranks`` CPU (gloo) processes, each
of which loads its dim-0 slice of every tensor straight from the source files and writes it back, so the result has
exactly ``--ranks`` shards per tensor and the same keys. No model object is needed: the tensors' names, shapes and
dtypes come from the checkpoint's metadata. Entries that are not tensors (optimizer hyper-parameters, step counters
saved as objects) are copied by rank 0.
"""

from __future__ import annotations

import argparse
import logging
import os
from typing import Any, Dict

import torch
import torch.distributed as dist

log = logging.getLogger(__name__)


def _worker(src: str, dst: str, skip_optim: bool) -> None:
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata
    from torch.distributed.device_mesh import DeviceMesh
    from torch.distributed.tensor import DTensor, Shard

    from ..distributed.checkpoint import get_checkpoint_metadata, load_state_dict, save_state_dict

    rank, ws = dist.get_rank(), dist.get_world_size()
    meta = get_checkpoint_metadata(src)
    mesh = DeviceMesh("cpu", list(range(ws)))
    state: Dict[str, Any] = {}
    n_tensors = n_objects = 0
    for key, info in meta.state_dict_metadata.items():
        if skip_optim and key.startswith("optim."):
            continue
        if isinstance(info, TensorStorageMetadata):
            shape, dtype = tuple(info.size), info.properties.dtype
            n_tensors += 1
            if len(shape) >= 1 and shape[0] >= ws:
                rows = -(-shape[0] // ws)  # torch.chunk's split: the last ranks may hold fewer rows, or none
                mine = max(0, min(rows, shape[0] - rank * rows))
                local = torch.empty((mine,) + shape[1:], dtype=dtype)
                stride = torch.empty(shape, device="meta").stride()
                state[key] = DTensor.from_local(local, mesh, [Shard(0)], run_check=False, shape=torch.Size(shape), stride=stride)
            else:
                state[key] = torch.empty(shape, dtype=dtype)  # scalars and tiny tensors stay whole (written once)
        else:
            n_objects += 1
            state[key] = None  # filled in by the loader
    load_state_dict(src, state)
    save_state_dict(dst, state, save_overwrite=True)
    if rank == 0:
        log.info(f"rewrote {n_tensors} tensors and {n_objects} other entries of '{src}' as {ws} shards under '{dst}'")


def reshard(src: str, dst: str, ranks: int, skip_optimizer_state: bool = False) -> None:
    from ..testing import run_distributed_test

    if ranks == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    run_distributed_test(_worker, world_size=ranks, backend="gloo", func_args=(src, dst, skip_optimizer_state))


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("input", help="checkpoint directory (the one that holds .metadata)")
    ap.add_argument("output")
    ap.add_argument("--ranks", type=int, required=True, help="number of shards per tensor in the output")
    ap.add_argument("--skip-optimizer-state", action="store_true")
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    reshard(a.input, a.output, a.ranks, a.skip_optimizer_state)


if __name__ == "__main__":
    main()
