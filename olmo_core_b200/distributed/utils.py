"""
Process-group bootstrap, rank helpers and small host-side collectives.

``torch.distributed`` is the control plane: NCCL for CUDA tensors (over NVLink 5 / NVSwitch inside one
box) and Gloo for CPU-side bookkeeping, i.e. backend string ``"cpu:gloo,cuda:nccl"``. The fused
compute+collective kernels use peer memory directly (see ``olmo_core_b200.parallel``) and only rely on
this module for rendezvous. Function names follow src/olmo_core/distributed/utils.py:72-587.
"""

from __future__ import annotations

import logging
import os
import socket
from datetime import timedelta
from typing import Any, Callable, Generator, List, Optional, TypeVar, Union

import torch
import torch.distributed as dist

from ..config import StrEnum
from ..exceptions import OLMoEnvironmentError

try:
    from torch.distributed.tensor import DTensor, distribute_tensor
except ImportError:  # pragma: no cover
    DTensor = None  # type: ignore
    distribute_tensor = None  # type: ignore

log = logging.getLogger(__name__)
T = TypeVar("T")

OLMO_SHARED_FS_ENV_VAR = "OLMO_SHARED_FS"
OLMO_FS_LOCAL_RANK_ENV_VAR = "FS_LOCAL_RANK"
OLMO_LOCAL_RANK_ENV_VAR = "LOCAL_RANK"
OLMO_NUM_NODES_ENV_VAR = "NUM_NODES"
OLMO_LOCAL_WORLD_SIZE_ENV_VAR = "LOCAL_WORLD_SIZE"

__all__ = [
    "init_distributed",
    "validate_env_vars",
    "is_distributed",
    "barrier",
    "get_rank",
    "get_global_rank",
    "get_local_rank",
    "get_fs_local_rank",
    "get_world_size",
    "get_local_world_size",
    "get_num_nodes",
    "get_node_hostname",
    "synchronize_value",
    "synchronize_flag",
    "all_reduce_value",
    "broadcast_object",
    "all_gather",
    "all_gather_object",
    "get_mesh_coordinates",
    "backend_supports_cuda",
    "backend_supports_cpu",
    "get_reduce_divide_factor",
    "get_local_tensor",
    "get_full_tensor",
    "distribute_like",
    "do_n_at_a_time",
    "hide_from_torch",
    "unhide_from_torch",
]


def _find_free_local_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _bootstrap_single_process_env() -> None:
    """Fill in the rendezvous variables so a plain ``python script.py`` run is a world of one."""
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault(OLMO_LOCAL_WORLD_SIZE_ENV_VAR, "1")
    os.environ.setdefault(OLMO_NUM_NODES_ENV_VAR, "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(_find_free_local_port()))


def init_distributed(
    backend: str = "nccl",
    timeout: timedelta = timedelta(minutes=30),
    shared_filesystem: Optional[bool] = None,
    **kwargs,
) -> None:
    """
    Initialise the default process group. Binds this process to ``cuda:LOCAL_RANK`` *before* creating
    the group when the backend drives CUDA devices.
    """
    if "RANK" not in os.environ or "WORLD_SIZE" not in os.environ:
        if "init_method" not in kwargs:
            _bootstrap_single_process_env()
    # Keeps NCCL from holding references to tensors on side streams; ordering is managed explicitly.
    os.environ.setdefault("TORCH_NCCL_AVOID_RECORD_STREAMS", "1")
    os.environ.setdefault("TORCH_DIST_INIT_BARRIER", "1")
    if shared_filesystem is not None:
        os.environ[OLMO_SHARED_FS_ENV_VAR] = "1" if shared_filesystem else "0"
    if backend_supports_cuda(backend) and torch.cuda.is_available():
        local_rank = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(local_rank % max(torch.cuda.device_count(), 1))
        device_id = torch.device("cuda", torch.cuda.current_device())
        try:
            dist.init_process_group(backend, timeout=timeout, device_id=device_id, **kwargs)
        except TypeError:
            dist.init_process_group(backend, timeout=timeout, **kwargs)
    else:
        if "nccl" in backend and not torch.cuda.is_available():
            backend = "gloo"
        dist.init_process_group(backend, timeout=timeout, **kwargs)
    validate_env_vars()
    msg = (
        f"Global rank {get_rank()} = local rank {get_local_rank()} = file system local rank {get_fs_local_rank()}"
    )
    log.info(msg)


def validate_env_vars() -> None:
    if not is_distributed():
        return
    missing = [v for v in (OLMO_NUM_NODES_ENV_VAR,) if v not in os.environ]
    if missing and "LOCAL_WORLD_SIZE" not in os.environ:
        raise OLMoEnvironmentError(
            f"Missing env vars {missing} (and LOCAL_WORLD_SIZE); launch with torchrun or set them explicitly."
        )


def get_node_hostname() -> str:
    return os.environ.get("NODE_HOSTNAME", socket.gethostname())


def is_distributed() -> bool:
    return dist.is_available() and dist.is_initialized()


def barrier(group: Optional[dist.ProcessGroup] = None) -> None:
    if is_distributed():
        dist.barrier(group)


def get_rank(group: Optional[dist.ProcessGroup] = None) -> int:
    if is_distributed():
        return dist.get_rank(group)
    return int(os.environ.get("RANK", 0)) if group is None else 0


def get_global_rank(group_rank: int, group: Optional[dist.ProcessGroup] = None) -> int:
    if group is None or not is_distributed():
        return group_rank
    return dist.get_global_rank(group, group_rank)


def get_local_rank() -> int:
    if OLMO_LOCAL_RANK_ENV_VAR in os.environ:
        return int(os.environ[OLMO_LOCAL_RANK_ENV_VAR])
    if is_distributed():
        raise OLMoEnvironmentError(f"'{OLMO_LOCAL_RANK_ENV_VAR}' must be set in a distributed run")
    return 0


def get_fs_local_rank(group: Optional[dist.ProcessGroup] = None) -> int:
    """
    Rank with respect to the file system: the global (group) rank when all ranks share one file system
    (``OLMO_SHARED_FS=1``), the explicit ``FS_LOCAL_RANK`` when given, else the node-local rank.
    """
    if os.environ.get(OLMO_SHARED_FS_ENV_VAR, "0") in ("1", "true", "True"):
        return int(os.environ.get(OLMO_FS_LOCAL_RANK_ENV_VAR, get_rank(group)))
    if OLMO_FS_LOCAL_RANK_ENV_VAR in os.environ:
        return int(os.environ[OLMO_FS_LOCAL_RANK_ENV_VAR])
    return get_local_rank()


def get_world_size(group: Optional[dist.ProcessGroup] = None) -> int:
    if is_distributed():
        return dist.get_world_size(group)
    return int(os.environ.get("WORLD_SIZE", 1)) if group is None else 1


def get_local_world_size() -> int:
    if OLMO_LOCAL_WORLD_SIZE_ENV_VAR in os.environ:
        return int(os.environ[OLMO_LOCAL_WORLD_SIZE_ENV_VAR])
    if is_distributed():
        raise OLMoEnvironmentError(f"'{OLMO_LOCAL_WORLD_SIZE_ENV_VAR}' must be set in a distributed run")
    return 1


def get_num_nodes() -> int:
    if OLMO_NUM_NODES_ENV_VAR in os.environ:
        return int(os.environ[OLMO_NUM_NODES_ENV_VAR])
    if is_distributed():
        return max(1, get_world_size() // get_local_world_size())
    return 1


def _default_device() -> torch.device:
    if is_distributed() and backend_supports_cuda() and torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


V = TypeVar("V", bool, int, float)


def synchronize_value(value: V, device: Optional[torch.device] = None, src: int = 0,
                      group: Optional[dist.ProcessGroup] = None) -> V:
    """Broadcast a scalar from ``src`` (a rank of ``group``) to every rank."""
    if not is_distributed() or get_world_size(group) == 1:
        return value
    device = device or _default_device()
    t = torch.tensor(value, device=device)
    dist.broadcast(t, get_global_rank(src, group), group=group)
    return t.item()  # type: ignore[return-value]


def synchronize_flag(flag: bool, device: Optional[torch.device] = None, group: Optional[dist.ProcessGroup] = None) -> bool:
    return bool(synchronize_value(flag, device, group=group))


def all_reduce_value(value: V, device: Optional[torch.device] = None, op=dist.ReduceOp.SUM,
                     group: Optional[dist.ProcessGroup] = None) -> V:
    if not is_distributed() or get_world_size(group) == 1:
        return value
    device = device or _default_device()
    t = torch.tensor(value, device=device)
    dist.all_reduce(t, op=op, group=group)
    return t.item()  # type: ignore[return-value]


def broadcast_object(obj: T, src: int = 0, group: Optional[dist.ProcessGroup] = None) -> T:
    if not is_distributed() or get_world_size(group) == 1:
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=get_global_rank(src, group), group=group)
    return box[0]


def all_gather(tensor: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> List[torch.Tensor]:
    """All-gather tensors whose shapes may differ across ranks (shapes are exchanged first)."""
    if not is_distributed() or get_world_size(group) == 1:
        return [tensor]
    shapes = all_gather_object(tuple(tensor.shape), group=group)
    outs = [torch.empty(s, dtype=tensor.dtype, device=tensor.device) for s in shapes]
    dist.all_gather(outs, tensor.contiguous(), group=group)
    return outs


def all_gather_object(obj: T, group: Optional[dist.ProcessGroup] = None) -> List[T]:
    if not is_distributed() or get_world_size(group) == 1:
        return [obj]
    out: List[Any] = [None] * get_world_size(group)
    dist.all_gather_object(out, obj, group=group)
    return out


def get_mesh_coordinates(mesh, rank: Optional[int] = None) -> Optional[List[int]]:
    rank = get_rank() if rank is None else rank
    where = (mesh.mesh == rank).nonzero()
    if where.size(0) == 0:
        return None
    return where[0].tolist()


def backend_supports_cuda(backend: Optional[str] = None) -> bool:
    if backend is None:
        if not is_distributed():
            return False
        backend = dist.get_backend()
    return "nccl" in backend


def backend_supports_cpu(backend: Optional[str] = None) -> bool:
    if backend is None:
        if not is_distributed():
            return True
        backend = dist.get_backend()
    return "gloo" in backend or "mpi" in backend


def get_reduce_divide_factor(world_size: int) -> float:
    """Power of two near sqrt(world): divide by it before a SUM all-reduce and by world/it after."""
    factor = 1
    while world_size % factor == 0 and world_size / factor > factor:
        factor *= 2
    return float(factor)


def get_local_tensor(x: torch.Tensor) -> torch.Tensor:
    if DTensor is not None and isinstance(x, DTensor):
        return x.to_local()
    return x


def get_full_tensor(x: torch.Tensor) -> torch.Tensor:
    if DTensor is not None and isinstance(x, DTensor):
        return x.full_tensor()
    return x


def distribute_like(source: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Give plain tensor ``target`` the same DTensor placement as ``source`` (no-op for plain sources)."""
    if DTensor is None or not isinstance(source, DTensor):
        return get_full_tensor(target)
    if isinstance(target, DTensor):
        if target.device_mesh == source.device_mesh and target.placements == source.placements:
            return target
        return target.redistribute(source.device_mesh, source.placements)
    return distribute_tensor(target, source.device_mesh, source.placements)


def do_n_at_a_time(f: Callable[[], T], *, n: Optional[int] = None, process_group: Optional[dist.ProcessGroup] = None,
                   world_size: Optional[int] = None, local_rank: Optional[int] = None) -> T:
    """Run ``f`` on at most ``n`` ranks at a time (throttles bursts of uploads), with barriers in between."""
    world_size = world_size if world_size is not None else get_world_size(process_group)
    local_rank = local_rank if local_rank is not None else get_rank(process_group)
    if n is None or n >= world_size:
        return f()
    result: Optional[T] = None
    done = False
    for turn in range((world_size + n - 1) // n):
        if local_rank // n == turn:
            result = f()
            done = True
        barrier(process_group)
    assert done
    return result  # type: ignore[return-value]


class _HiddenTensor:
    """Wrapper that keeps a tensor out of ``module.to()``, ``state_dict()`` and FSDP-style wrappers."""

    def __init__(self, x: torch.Tensor):
        self.x = x

    @property
    def device(self) -> torch.device:
        return self.x.device

    def to(self, *args, **kwargs) -> "_HiddenTensor":
        return _HiddenTensor(self.x.to(*args, **kwargs))


def hide_from_torch(x: torch.Tensor) -> _HiddenTensor:
    return _HiddenTensor(x)


def unhide_from_torch(x: Union[torch.Tensor, _HiddenTensor]) -> torch.Tensor:
    return x.x if isinstance(x, _HiddenTensor) else x
