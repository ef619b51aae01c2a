"""
World-mesh construction and sub-mesh lookup for every parallelism strategy
(API of src/olmo_core/distributed/parallel/__init__.py:22-609).

Dimension order, outermost first: ``pp`` -> (``dp_replicate``, ``dp_shard``) or ``dp`` (-> ``ep``) ->
``cp`` -> ``tp``. Tensor parallel ranks are therefore neighbours, which on an NVSwitch box does not
matter for bandwidth (every peer is one hop away) but keeps rank numbering identical to the reference
so checkpoints and data order match.
"""

from __future__ import annotations

import logging
from typing import Dict, List, Optional, Tuple

from torch.distributed import ProcessGroup
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

from ...config import StrEnum
from ...exceptions import OLMoConfigurationError
from ...utils import get_default_device
from ..utils import get_world_size
from .context_parallel import ContextParallelConfig
from .data_parallel import DataParallelConfig, DataParallelType, DPMeshDimName
from .expert_parallel import ExpertParallelConfig
from .pipeline_parallel import (
    PipelineParallelConfig,
    PipelineSchedule,
    PipelineScheduleType,
    PipelineSplitStyle,
)
from .tensor_parallel import TensorParallelConfig

__all__ = [
    "build_world_mesh",
    "get_world_mesh",
    "reset_world_mesh",
    "build_expert_parallel_mesh",
    "MeshDimName",
    "get_dp_model_mesh",
    "get_dp_mesh",
    "get_tp_mesh",
    "get_cp_mesh",
    "get_pp_mesh",
    "get_pp_stage_mesh",
    "get_ep_mesh",
    "get_dp_shard_mesh",
    "get_dp_replicate_mesh",
    "get_dp_process_group",
    "get_device_mesh_info",
    "flatten_mesh",
    "DataParallelType",
    "DataParallelConfig",
    "DPMeshDimName",
    "TensorParallelConfig",
    "ContextParallelConfig",
    "ExpertParallelConfig",
    "PipelineParallelConfig",
    "PipelineScheduleType",
    "PipelineSplitStyle",
    "PipelineSchedule",
]

log = logging.getLogger(__name__)


class MeshDimName(StrEnum):
    dp = "dp"
    dp_replicate = DPMeshDimName.replicate.value
    dp_shard = DPMeshDimName.shard.value
    ep = "ep"
    ep_replicate = "ep_replicate"
    ep_shard = "ep_shard"
    dp_ep = "dp_ep"
    dp_cp = "dp_cp"
    tp = "tp"
    cp = "cp"
    pp = "pp"


_WORLD_MESH: Optional[DeviceMesh] = None
_FLATTENED: Dict[Tuple[int, Tuple[str, ...]], DeviceMesh] = {}


def get_world_mesh() -> Optional[DeviceMesh]:
    return _WORLD_MESH


def reset_world_mesh() -> None:
    """Forget the global mesh (tests build several meshes in one process)."""
    global _WORLD_MESH
    _WORLD_MESH = None
    _FLATTENED.clear()


def _take(world: int, degree: int, what: str) -> int:
    if degree < 1 or world % degree != 0:
        raise OLMoConfigurationError(f"{what}.degree ({degree}) must be at least 1 and divide the remaining world size ({world})")
    return world // degree


def build_world_mesh(
    *,
    dp: Optional[DataParallelConfig] = None,
    tp: Optional[TensorParallelConfig] = None,
    cp: Optional[ContextParallelConfig] = None,
    pp: Optional[PipelineParallelConfig] = None,
    ep: Optional[ExpertParallelConfig] = None,
    device_type: Optional[str] = None,
) -> DeviceMesh:
    """Build the global mesh once per process from the parallelism configs."""
    global _WORLD_MESH
    if _WORLD_MESH is not None:
        raise RuntimeError("world mesh already exists! You can only call 'build_world_mesh' once!")
    device_type = device_type or get_default_device().type
    remaining = get_world_size()

    if dp is None:
        if any(c is not None for c in (tp, cp, pp, ep)):
            raise OLMoConfigurationError(
                "Data parallel config is required in addition to expert/tensor/context/pipeline parallel configs"
            )
        _WORLD_MESH = init_device_mesh(device_type, (remaining,), mesh_dim_names=(MeshDimName.dp.value,))
        return _WORLD_MESH

    if pp is not None:
        remaining = _take(remaining, pp.degree, "PipelineParallelConfig")
    if cp is not None:
        remaining = _take(remaining, cp.degree, "ContextParallelConfig")
    if tp is not None:
        remaining = _take(remaining, tp.degree, "TensorParallelConfig")
    if ep is not None:
        if tp is not None:
            raise OLMoConfigurationError("expert parallelism is mutually exclusive with tensor parallelism")
        if dp.name != DataParallelType.hsdp:
            raise OLMoConfigurationError("expert parallelism can currently only be used with HSDP data parallelism")

    dims: List[Tuple[str, int]] = []
    if pp is not None:
        dims.append((MeshDimName.pp.value, pp.degree))
    if dp.name == DataParallelType.hsdp:
        replicas, shards = dp.get_replicate_and_shard_degree(remaining)
        if ep is not None and ep.degree >= 0 and ep.degree != shards:
            raise OLMoConfigurationError("expert parallelism + HSDP requires the same sharding degree")
        dims += [(MeshDimName.dp_replicate.value, replicas), (MeshDimName.dp_shard.value, shards)]
    else:
        dims.append((MeshDimName.dp.value, remaining))
    if cp is not None:
        dims.append((MeshDimName.cp.value, cp.degree))
    if tp is not None:
        dims.append((MeshDimName.tp.value, tp.degree))

    mesh = init_device_mesh(device_type, tuple(d for _, d in dims), mesh_dim_names=tuple(n for n, _ in dims))
    log.info(f"Built {get_device_mesh_info(mesh)}")
    _WORLD_MESH = mesh
    get_dp_process_group(mesh)  # create the data-parallel group eagerly, on every rank
    return mesh


def get_device_mesh_info(device_mesh: DeviceMesh) -> str:
    names = device_mesh.mesh_dim_names
    shape = " x ".join(
        f"{n}={device_mesh.size(i)}" if names else str(device_mesh.size(i))
        for i, n in enumerate(names or range(device_mesh.ndim))
    )
    return f"{device_mesh.ndim}D device mesh ({shape})"


def build_expert_parallel_mesh(ep_config: ExpertParallelConfig, device_type: Optional[str] = None) -> DeviceMesh:
    """Stand-alone (``ep_replicate``, ``ep_shard``) mesh for MoE layers outside of a world mesh."""
    device_type = device_type or get_default_device().type
    world = get_world_size()
    degree = world if ep_config.degree < 0 else ep_config.degree
    if degree < 1 or world % degree != 0:
        raise OLMoConfigurationError(f"ExpertParallelConfig.degree ({degree}) must divide the world size ({world})")
    return init_device_mesh(
        device_type, (world // degree, degree), mesh_dim_names=(MeshDimName.ep_replicate.value, MeshDimName.ep_shard.value)
    )


def _names(device_mesh: DeviceMesh) -> Tuple[str, ...]:
    if device_mesh.mesh_dim_names is None:
        raise RuntimeError("could not determine a sub-mesh without dimension names")
    return tuple(device_mesh.mesh_dim_names)


def _flatten(device_mesh: DeviceMesh, dims: Tuple[str, ...], name: str) -> DeviceMesh:
    """1-D mesh spanning ``dims`` of ``device_mesh`` (cached: flattening creates a process group)."""
    key = (id(device_mesh), dims)
    if key not in _FLATTENED:
        _FLATTENED[key] = device_mesh[dims]._flatten(mesh_dim_name=name)
    return _FLATTENED[key]


def flatten_mesh(device_mesh: DeviceMesh, name: Optional[str] = None) -> DeviceMesh:
    names = _names(device_mesh)
    return _flatten(device_mesh, names, name or "_".join(names))


def get_dp_model_mesh(device_mesh: DeviceMesh) -> DeviceMesh:
    """
    The mesh the model-parallel wrapper (sharded or replicated data parallelism) runs over. Context-
    parallel ranks hold full parameter replicas, so ``cp`` is folded into the adjacent data-parallel
    dimension; an ``ep`` dimension is folded in the same way.
    """
    names = _names(device_mesh)
    has = lambda n: n in names  # noqa: E731
    if has(MeshDimName.dp_replicate.value) and has(MeshDimName.dp_shard.value):
        if has(MeshDimName.cp.value):
            shard = _flatten(device_mesh, (MeshDimName.dp_shard.value, MeshDimName.cp.value), MeshDimName.dp_cp.value)
            # 2-D (replicate, shard x cp) view assembled from the parent mesh
            return _compose_2d(device_mesh, MeshDimName.dp_replicate.value, shard)
        return device_mesh[MeshDimName.dp_replicate.value, MeshDimName.dp_shard.value]
    if has(MeshDimName.dp.value):
        extra = tuple(n for n in (MeshDimName.ep.value, MeshDimName.cp.value) if has(n))
        if extra:
            return _flatten(device_mesh, (MeshDimName.dp.value,) + extra, "dp_" + "_".join(extra))
        return device_mesh[MeshDimName.dp.value]
    if has(MeshDimName.ep_replicate.value) and has(MeshDimName.ep_shard.value):
        return _flatten(device_mesh, (MeshDimName.ep_replicate.value, MeshDimName.ep_shard.value), MeshDimName.dp.value)
    raise RuntimeError(f"could not determine the data-parallel model sub-mesh from dims {names}")


class _Composed2D:
    """Minimal 2-D mesh view (replicate group x flattened shard group) used with HSDP + CP."""

    def __init__(self, replicate: DeviceMesh, shard: DeviceMesh):
        self.replicate, self.shard = replicate, shard
        self.mesh_dim_names = (MeshDimName.dp_replicate.value, MeshDimName.dp_cp.value)
        self.ndim = 2

    def __getitem__(self, name: str) -> DeviceMesh:
        return self.replicate if name == MeshDimName.dp_replicate.value else self.shard

    def size(self, dim: Optional[int] = None) -> int:
        sizes = (self.replicate.size(), self.shard.size())
        return sizes[0] * sizes[1] if dim is None else sizes[dim]

    def get_group(self, dim):
        return (self.replicate if dim in (0, MeshDimName.dp_replicate.value) else self.shard).get_group()


def _compose_2d(device_mesh: DeviceMesh, replicate_dim: str, shard: DeviceMesh):
    return _Composed2D(device_mesh[replicate_dim], shard)


def get_dp_mesh(device_mesh: DeviceMesh) -> DeviceMesh:
    """
    1-D mesh over the ranks that receive *different data* (what a data loader needs). Unlike
    :func:`get_dp_model_mesh` this leaves out ``cp``: context-parallel ranks share a batch.
    """
    names = _names(device_mesh)
    dp_dims = tuple(
        n
        for n in (MeshDimName.dp_replicate.value, MeshDimName.dp_shard.value, MeshDimName.dp.value, MeshDimName.ep.value,
                  MeshDimName.ep_replicate.value, MeshDimName.ep_shard.value)
        if n in names
    )
    if not dp_dims:
        raise RuntimeError(f"could not determine the data-parallel sub-mesh from dims {names}")
    if len(dp_dims) == 1:
        return device_mesh[dp_dims[0]]
    return _flatten(device_mesh, dp_dims, MeshDimName.dp.value)


def get_dp_process_group(device_mesh: DeviceMesh) -> ProcessGroup:
    return get_dp_mesh(device_mesh).get_group()


def _get_1d(device_mesh: DeviceMesh, name: str, what: str) -> DeviceMesh:
    names = _names(device_mesh)
    if name not in names:
        raise RuntimeError(f"could not determine the {what} sub-mesh: no '{name}' dimension in {names}")
    return device_mesh[name]


def get_dp_shard_mesh(device_mesh: DeviceMesh) -> DeviceMesh:
    names = _names(device_mesh)
    if MeshDimName.dp_shard.value in names:
        return device_mesh[MeshDimName.dp_shard.value]
    return get_dp_mesh(device_mesh)


def get_dp_replicate_mesh(device_mesh: DeviceMesh) -> DeviceMesh:
    return _get_1d(device_mesh, MeshDimName.dp_replicate.value, "data-parallel replicate")


def get_ep_mesh(device_mesh: DeviceMesh) -> DeviceMesh:
    names = _names(device_mesh)
    for cand in (MeshDimName.ep.value, MeshDimName.ep_shard.value, MeshDimName.dp_shard.value):
        if cand in names:
            return device_mesh[cand]
    raise RuntimeError(f"could not determine the expert-parallel sub-mesh from dims {names}")


def get_tp_mesh(device_mesh: DeviceMesh) -> DeviceMesh:
    return _get_1d(device_mesh, MeshDimName.tp.value, "tensor-parallel")


def get_cp_mesh(device_mesh: DeviceMesh) -> DeviceMesh:
    return _get_1d(device_mesh, MeshDimName.cp.value, "context-parallel")


def get_pp_mesh(device_mesh: DeviceMesh) -> DeviceMesh:
    return _get_1d(device_mesh, MeshDimName.pp.value, "pipeline-parallel")


def get_pp_stage_mesh(device_mesh: DeviceMesh, pp_mesh: Optional[DeviceMesh] = None) -> DeviceMesh:
    """Everything but the ``pp`` dimension: the ranks that jointly hold one pipeline stage."""
    names = _names(device_mesh)
    rest = tuple(n for n in names if n != MeshDimName.pp.value)
    if not rest:
        raise RuntimeError("the mesh has no non-pipeline dimensions")
    return device_mesh[rest] if len(rest) > 1 else device_mesh[rest[0]]
