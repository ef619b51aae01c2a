"""
Launcher for multi-process tests (src/olmo_core/testing/distributed.py:111-147): CPU tests of multi-rank logic run as
``gloo`` ranks forked from the test process; multi-GPU ones use the ``cuda:nccl,cpu:gloo`` backend with one spawned
process per device.
"""

from __future__ import annotations

import datetime
import logging
import os
import socket
import sys
import traceback
from typing import Any, Callable, Dict, Optional, Tuple

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

__all__ = ["run_distributed_test"]


def _free_port(host: str) -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((host, 0))
        return s.getsockname()[1]


def _worker(rank: int, world_size: int, backend: str, log_from_all_ranks: bool, func: Callable, func_args, func_kwargs,
            addr: str, port: int) -> None:
    # A forked child inherits an OpenMP pool whose worker threads do not exist in it; entering a parallel
    # region would wait for them forever. One thread per rank also keeps N ranks from oversubscribing the host.
    torch.set_num_threads(1)
    os.environ.update(
        RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world_size), LOCAL_WORLD_SIZE=str(world_size),
        FS_LOCAL_RANK=str(rank), NUM_NODES="1", MASTER_ADDR=addr, MASTER_PORT=str(port),
    )
    logging.basicConfig(level=logging.INFO if (log_from_all_ranks or rank == 0) else logging.WARNING,
                        format=f"[rank {rank}] %(levelname)s %(name)s: %(message)s", force=True)
    if "nccl" in backend:
        torch.cuda.set_device(rank)
    dist.init_process_group(backend=backend, init_method=f"tcp://{addr}:{port}", world_size=world_size, rank=rank,
                            timeout=datetime.timedelta(seconds=120))
    try:
        func(*(func_args or ()), **(func_kwargs or {}))
    except BaseException:
        traceback.print_exc()
        sys.stderr.flush()
        raise
    finally:
        from ..distributed.parallel import reset_world_mesh

        reset_world_mesh()
        dist.destroy_process_group()


def run_distributed_test(
    func: Callable,
    world_size: int = 2,
    log_from_all_ranks: bool = False,
    backend: str = "gloo",
    start_method: Optional[str] = None,
    func_args: Optional[Tuple[Any, ...]] = None,
    func_kwargs: Optional[Dict[str, Any]] = None,
    primary_addr: str = "127.0.0.1",
    primary_port: Optional[int] = None,
) -> None:
    """Run ``func(*func_args, **func_kwargs)`` on ``world_size`` ranks with an initialised default process group."""
    if start_method is None:
        start_method = "fork" if backend == "gloo" else "spawn"
    port = primary_port or _free_port(primary_addr)
    mp.start_processes(
        _worker,
        args=(world_size, backend, log_from_all_ranks, func, func_args, func_kwargs, primary_addr, port),
        nprocs=world_size,
        start_method=start_method,
    )
