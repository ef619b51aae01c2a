"""
Configuration of the transformer train module and its parallelism strategies
(API of src/olmo_core/train/train_module/transformer/config.py:43-386).
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from ....config import Config, DType
from ....distributed.parallel import (
    ContextParallelConfig,
    DataParallelConfig,
    ExpertParallelConfig,
    PipelineParallelConfig,
    PipelineSplitStyle,
    TensorParallelConfig,
)
from ....doc_utils import beta_feature
from ....exceptions import OLMoConfigurationError
from ....float8 import Float8Config
from ....nn.attention.ring import (
    RingAttentionLoadBalancerType,
    RingContextParallelStyle,
    UlyssesContextParallelStyle,
)
from ....nn.transformer.config import (
    TransformerActivationCheckpointingMode,
    TransformerDataParallelWrappingStrategy,
)
from ....optim import OptimConfig
from ....optim.scheduler import Scheduler
from ..config import TrainModuleConfig

__all__ = [
    "TransformerTrainModuleConfig",
    "TransformerPipelineTrainModuleConfig",
    "TransformerDataParallelConfig",
    "TransformerDataParallelWrappingStrategy",
    "TransformerTensorParallelConfig",
    "TransformerContextParallelConfig",
    "TransformerExpertParallelConfig",
    "TransformerPipelineParallelConfig",
    "TransformerActivationCheckpointingConfig",
    "TransformerActivationCheckpointingMode",
]


@dataclass
class TransformerPipelineParallelConfig(PipelineParallelConfig):
    """Pipeline config that also knows how to cut a transformer into stages."""

    split_points: Optional[List[int]] = None

    def get_split_points(self, n_layers: int) -> List[int]:
        """Block indices at which a new stage starts (embeddings go with the first, LM head with the last stage)."""
        if self.split_points is not None:
            return list(self.split_points)
        num_stages = self.degree * (1 if self.schedule.is_single_stage else 2)
        if num_stages > n_layers:
            raise OLMoConfigurationError(f"cannot split {n_layers} layers into {num_stages} pipeline stages")
        per_stage = n_layers / num_stages
        return [round(i * per_stage) for i in range(1, num_stages)]

    def split_model(self, model: nn.Module, *, pp_mesh, device: torch.device) -> Tuple[List[Any], List[nn.Module]]:
        """Copy the (meta-device) model once per local stage, delete what the stage does not own, wrap in PipelineStage."""
        from torch.distributed.pipelining import PipelineStage

        n_layers = len(model.blocks)
        bounds = [0] + self.get_split_points(n_layers) + [n_layers]
        num_stages = len(bounds) - 1
        pp_rank = pp_mesh.get_local_rank()
        stages, parts = [], []
        for stage_id in self.stage_ids_this_rank(pp_rank, num_stages):
            part = copy.deepcopy(model)
            lo, hi = bounds[stage_id], bounds[stage_id + 1]
            for key in list(part.blocks.keys()):
                if not lo <= int(key) < hi:
                    del part.blocks[key]
            if stage_id != 0:
                part.embeddings = None
                part.embedding_norm = None
            if stage_id != num_stages - 1:
                part.lm_head = None
            if getattr(part, "tie_word_embeddings", False):
                raise OLMoConfigurationError("tied word embeddings are not supported with pipeline parallelism")
            part.apply_pp(pp_mesh)
            stages.append(PipelineStage(part, stage_id, num_stages, device, group=pp_mesh.get_group()))
            parts.append(part)
        return stages, parts


@dataclass
class TransformerDataParallelConfig(DataParallelConfig):
    wrapping_strategy: TransformerDataParallelWrappingStrategy = TransformerDataParallelWrappingStrategy.full
    prefetch_factor: int = 0


@dataclass
class TransformerTensorParallelConfig(TensorParallelConfig):
    pass


@dataclass
class TransformerContextParallelConfig(ContextParallelConfig):
    ring: Optional[RingContextParallelStyle] = None
    uly: Optional[UlyssesContextParallelStyle] = None

    def __post_init__(self):
        if self.ring is not None and self.uly is not None:
            raise NotImplementedError("Only one of ring or ulysses can be specified.")
        if self.ring is None and self.uly is None:
            raise OLMoConfigurationError("One of ring or uly must be specified")

    @classmethod
    def zig_zag(cls, degree: int, head_stride: int = 1) -> "TransformerContextParallelConfig":
        return cls(degree=degree, ring=RingContextParallelStyle(load_balancer=RingAttentionLoadBalancerType.zig_zag, head_stride=head_stride))

    @classmethod
    def llama3(cls, degree: int, head_stride: int = 1) -> "TransformerContextParallelConfig":
        return cls(degree=degree, ring=RingContextParallelStyle(load_balancer=RingAttentionLoadBalancerType.llama3, head_stride=head_stride))

    @classmethod
    def ulysses(cls, degree: int) -> "TransformerContextParallelConfig":
        return cls(degree=degree, uly=UlyssesContextParallelStyle())


@dataclass
class TransformerExpertParallelConfig(ExpertParallelConfig):
    pass


@beta_feature
@dataclass
class TransformerActivationCheckpointingConfig(Config):
    mode: TransformerActivationCheckpointingMode = TransformerActivationCheckpointingMode.full
    block_interval: Optional[int] = None
    modules: Optional[List[str]] = None
    activation_memory_budget: Optional[float] = None
    determinism_check: str = "default"

    def __post_init__(self):
        if self.mode == TransformerActivationCheckpointingMode.selected_blocks and self.block_interval is None:
            raise OLMoConfigurationError("'block_interval' is required for 'selected_blocks' activation checkpointing")
        if self.mode == TransformerActivationCheckpointingMode.selected_modules and self.modules is None:
            raise OLMoConfigurationError("'modules' is required for 'selected_modules' activation checkpointing")

    def as_kwargs(self) -> Dict[str, Any]:
        return dict(mode=self.mode, block_interval=self.block_interval, modules=self.modules,
                    activation_memory_budget=self.activation_memory_budget)


@dataclass
class TransformerTrainModuleConfig(TrainModuleConfig):
    rank_microbatch_size: int
    """Micro-batch size per rank, in tokens."""
    max_sequence_length: int
    optim: OptimConfig
    max_grad_norm: Optional[float] = None
    scheduler: Optional[Scheduler] = None
    compile_model: bool = False
    float8_config: Optional[Float8Config] = None
    pp_config: Optional[TransformerPipelineParallelConfig] = None
    dp_config: Optional[TransformerDataParallelConfig] = None
    tp_config: Optional[TransformerTensorParallelConfig] = None
    cp_config: Optional[TransformerContextParallelConfig] = None
    ep_config: Optional[TransformerExpertParallelConfig] = None
    ac_config: Optional[TransformerActivationCheckpointingConfig] = None
    z_loss_multiplier: Optional[float] = None
    state_dict_save_opts: Optional[Dict[str, Any]] = None
    state_dict_load_opts: Optional[Dict[str, Any]] = None
    load_key_mapping: Optional[Dict[str, str]] = None
    autocast_precision: Optional[DType] = None
    label_ignore_index: int = -100

    def build(self, model, device: Optional[torch.device] = None):
        from .pipeline_train_module import TransformerPipelineTrainModule
        from .train_module import TransformerTrainModule

        kwargs = self.as_dict(exclude_none=True, recurse=False)
        if (ap := kwargs.pop("autocast_precision", None)) is not None:
            kwargs["autocast_precision"] = DType(ap).as_pt()
        cls = TransformerPipelineTrainModule if self.pp_config is not None else TransformerTrainModule
        return cls(model=model, device=device, **kwargs)


@dataclass
class TransformerPipelineTrainModuleConfig(TransformerTrainModuleConfig):
    """Older name of a :class:`TransformerTrainModuleConfig` whose ``pp_config`` is set
    (src/olmo_core/train/train_module/transformer/config.py:379-386)."""

    def __post_init__(self):
        if self.pp_config is None:
            raise OLMoConfigurationError("'pp_config' is required")
