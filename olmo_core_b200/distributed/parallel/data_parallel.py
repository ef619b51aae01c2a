"""Data-parallel configuration (FSDP / HSDP / DDP). API of src/olmo_core/distributed/parallel/data_parallel.py:12-81."""

from dataclasses import dataclass
from typing import Optional, Tuple

from ...config import Config, DType, StrEnum
from ...exceptions import OLMoConfigurationError
from ..utils import get_num_nodes

__all__ = ["DataParallelType", "DataParallelConfig", "DPMeshDimName"]


class DPMeshDimName(StrEnum):
    """Names of the two mesh dimensions of hybrid-sharded data parallelism."""

    replicate = "dp_replicate"
    shard = "dp_shard"


class DataParallelType(StrEnum):
    fsdp = "fsdp"
    hsdp = "hsdp"
    ddp = "ddp"


def _divides(value: int, world: int, what: str) -> int:
    if value < 1 or world % value != 0:
        raise OLMoConfigurationError(f"data parallel world size ({world}) must be divisible by '{what}' ({value})")
    return value


@dataclass
class DataParallelConfig(Config):
    """
    ``name`` selects sharded (fsdp), hybrid (hsdp: shard inside a group, replicate across groups) or
    replicated (ddp) data parallelism. ``param_dtype`` is the compute dtype of the gathered parameters,
    ``reduce_dtype`` the dtype gradients are reduced in.
    """

    name: DataParallelType
    param_dtype: Optional[DType] = None
    reduce_dtype: DType = DType.float32
    num_replicas: Optional[int] = None
    shard_degree: Optional[int] = None

    def get_replicate_and_shard_degree(self, dp_world_size: int) -> Tuple[int, int]:
        """(replicas, shard degree); by default one replica per node."""
        replicas, shards = self.num_replicas, self.shard_degree
        if replicas is None and shards is None:
            nodes = get_num_nodes()
            return nodes, dp_world_size // nodes
        if replicas is not None and shards is not None:
            _divides(replicas, dp_world_size, "num_replicas")
            _divides(shards, dp_world_size, "shard_degree")
            if replicas * shards != dp_world_size:
                raise OLMoConfigurationError(
                    f"num_replicas ({replicas}) x shard_degree ({shards}) != data parallel world size ({dp_world_size})"
                )
            return replicas, shards
        if replicas is not None:
            return _divides(replicas, dp_world_size, "num_replicas"), dp_world_size // replicas
        assert shards is not None
        return dp_world_size // _divides(shards, dp_world_size, "shard_degree"), shards
