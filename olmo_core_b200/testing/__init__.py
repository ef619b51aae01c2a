"""
Helpers for the test-suite: pytest marks and parametrisations for devices / backends and a launcher for
multi-process tests (API of src/olmo_core/testing/__init__.py, src/olmo_core/testing/distributed.py:111-150).

CPU tests of multi-rank logic run as ``gloo`` ranks forked from the test process; GPU tests carry the ``gpu``
mark and multi-GPU ones use the ``cuda:nccl,cpu:gloo`` backend with one spawned process per device.
"""

from __future__ import annotations

import datetime
import logging
import os
import socket
import sys
import traceback
from typing import Any, Callable, Dict, Optional, Tuple

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

log = logging.getLogger(__name__)

__all__ = [
    "BACKENDS",
    "DEVICES",
    "INIT_DEVICES",
    "LOW_PRECISION_DTYPES",
    "GPU_MARKS",
    "MULTI_GPU_MARKS",
    "has_cuda",
    "has_multiple_gpus",
    "requires_gpu",
    "requires_multi_gpu",
    "run_distributed_test",
    "FLASH_2_MARKS", "FLASH_3_MARKS", "FLASH_4_MARKS", "GROUPED_GEMM_MARKS", "TE_MARKS",
    "has_flash_attn_2", "has_flash_attn_3", "has_flash_attn_4", "has_grouped_gemm", "has_torchao", "has_quack",
    "requires_flash_attn_2", "requires_flash_attn_3", "requires_flash_attn_4", "requires_grouped_gemm", "requires_fla",
    "requires_quack", "requires_dion", "requires_te", "requires_compute_capability",
]

has_cuda = torch.cuda.is_available()
has_multiple_gpus = has_cuda and torch.cuda.device_count() > 1

GPU_MARKS = (pytest.mark.gpu, pytest.mark.skipif(not has_cuda, reason="Requires a GPU"))
MULTI_GPU_MARKS = (pytest.mark.gpu, pytest.mark.skipif(not has_multiple_gpus, reason="Requires multiple GPUs"))


def _apply(marks, func):
    for mark in marks:
        func = mark(func)
    return func


def requires_gpu(func):
    return _apply(GPU_MARKS, func)


has_mps = bool(getattr(torch.backends, "mps", None)) and torch.backends.mps.is_available()
MPS_MARKS = (pytest.mark.skipif(not has_mps, reason="Requires MPS"),)


def requires_mps(func):
    return _apply(MPS_MARKS, func)


def requires_multi_gpu(func):
    return _apply(MULTI_GPU_MARKS, func)


def _kernels_available() -> bool:
    if not has_cuda:
        return False
    from ..ops.attention import has_flash_kernel

    return has_flash_kernel()


# The capabilities that the reference gates on optional wheels are built in here: each probe answers whether this
# package's own kernel for that role can run on the current machine.
has_flash_attn_2 = has_flash_attn_3 = has_flash_attn_4 = _kernels_available()
has_grouped_gemm = has_cuda
has_torchao = has_cuda  # float8 training uses this package's own GEMMs
has_quack = has_cuda  # fused RMSNorm / cross-entropy kernels are built in
has_te = False

FLASH_2_MARKS = FLASH_3_MARKS = FLASH_4_MARKS = (
    pytest.mark.gpu, pytest.mark.skipif(not has_flash_attn_2, reason="Requires the flash-attention kernels (B200)"))
GROUPED_GEMM_MARKS = GPU_MARKS
TE_MARKS = (pytest.mark.gpu, pytest.mark.skipif(True, reason="Transformer Engine is not used by this framework"))


def requires_flash_attn_2(func):
    return _apply(FLASH_2_MARKS, func)


requires_flash_attn_3 = requires_flash_attn_4 = requires_flash_attn_2


def requires_grouped_gemm(func):
    return _apply(GROUPED_GEMM_MARKS, func)


def requires_fla(func):  # the gated delta rule is built in and runs everywhere
    return func


def requires_quack(func):
    return _apply(GPU_MARKS, func)


def requires_dion(func):  # the Dion optimizer is built in
    return func


def requires_te(func):
    return _apply(TE_MARKS, func)


def requires_compute_capability(min_cc: int):
    """``min_cc`` as major * 10 + minor, e.g. 100 for sm_100."""
    def decorator(func):
        ok = has_cuda and (lambda c: c[0] * 10 + c[1])(torch.cuda.get_device_capability()) >= min_cc
        return _apply((pytest.mark.gpu, pytest.mark.skipif(not ok, reason=f"Requires compute capability >= {min_cc}")), func)

    return decorator


INIT_DEVICES = [
    pytest.param(torch.device("meta"), id="device=meta"),
    pytest.param(torch.device("cpu"), id="device=CPU"),
    pytest.param(torch.device("cuda"), id="device=CUDA", marks=GPU_MARKS),
]
DEVICES = [
    pytest.param(torch.device("cpu"), id="device=CPU"),
    pytest.param(torch.device("cuda"), id="device=CUDA", marks=GPU_MARKS),
]
BACKENDS = [
    pytest.param("gloo", id="backend=GLOO"),
    pytest.param("cuda:nccl,cpu:gloo", id="backend=NCCL", marks=MULTI_GPU_MARKS),
]
LOW_PRECISION_DTYPES = [
    pytest.param(torch.float16, id="dtype=float16"),
    pytest.param(torch.bfloat16, id="dtype=bfloat16", marks=GPU_MARKS),
]


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
