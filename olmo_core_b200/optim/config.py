"""
Optimizer configuration base (API of src/olmo_core/optim/config.py:43-399): parameter groups from
``fnmatch`` patterns over fully-qualified parameter names, ``initial_lr`` bookkeeping for schedulers and
fields that survive ``load_state_dict``.
"""

from __future__ import annotations

import logging
from abc import ABCMeta, abstractmethod
from collections import OrderedDict
from dataclasses import dataclass
from fnmatch import fnmatch
from typing import Any, Dict, Generic, Iterable, List, Optional, Set, Tuple, Type, TypeVar, Union

import torch
import torch.nn as nn

from ..config import Config, Registrable
from ..exceptions import OLMoConfigurationError
from ..utils import get_default_device, move_to_device

__all__ = ["OptimConfig", "OptimGroupOverride", "MatrixAwareOptimConfig", "INITIAL_LR_FIELD", "LR_FIELD"]

log = logging.getLogger(__name__)

LR_FIELD = "lr"
INITIAL_LR_FIELD = "initial_lr"

Opt = TypeVar("Opt", bound=torch.optim.Optimizer)


@dataclass
class OptimGroupOverride(Config):
    params: List[str]
    """Fully-qualified parameter names or wildcards."""
    opts: Dict[str, Any]
    """Options set on the resulting param group."""


@dataclass
class OptimConfig(Config, Registrable, Generic[Opt], metaclass=ABCMeta):
    group_overrides: Optional[List[OptimGroupOverride]] = None
    compile: bool = False
    fixed_fields: Tuple[str, ...] = (INITIAL_LR_FIELD,)

    @property
    def device(self) -> torch.device:
        return get_default_device()

    def build_groups(self, model: nn.Module, strict: bool = True) -> List[Dict[str, Any]]:
        """Param groups: one per override (in order), then one for everything not matched."""
        trainable: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        frozen: Set[str] = set()
        for n, p in model.named_parameters():
            (trainable.__setitem__(n, p) if p.requires_grad else frozen.add(n))
        groups: List[Dict[str, Any]] = []
        taken: Set[str] = set()
        for g_idx, go in enumerate(self.group_overrides or []):
            names: List[str] = []
            for pattern in go.params:
                matched = [n for n in trainable if fnmatch(n, pattern)]
                if not matched:
                    if any(fnmatch(n, pattern) for n in frozen):
                        log.warning(f"optim group {g_idx} override pattern '{pattern}' matches a frozen parameter and will be ignored")
                    else:
                        msg = f"optim group {g_idx} override pattern '{pattern}' does not match any parameters"
                        if strict:
                            raise OLMoConfigurationError(msg)
                        log.warning(msg)
                names.extend(matched)
            taken.update(names)
            if names:
                groups.append({"params": [trainable[n] for n in names], "param_names": names, **go.opts})
        rest = [n for n in trainable if n not in taken]
        if rest:
            groups.append({"params": [trainable[n] for n in rest], "param_names": rest})
        for g in groups:
            g.pop("param_names")
        return groups

    @classmethod
    @abstractmethod
    def optimizer(cls) -> Type[Opt]:
        raise NotImplementedError

    def build(self, model: nn.Module, strict: bool = True) -> Opt:
        kwargs = self.as_dict()
        for k in ("group_overrides", "compile", "fixed_fields"):
            kwargs.pop(k)
        optim: torch.optim.Optimizer = self.optimizer()(self.build_groups(model, strict=strict), **kwargs)
        fixed_per_group: List[Dict[str, Any]] = [{} for _ in optim.param_groups]
        for fixed, group in zip(fixed_per_group, optim.param_groups):
            lr = group.get(LR_FIELD, getattr(self, LR_FIELD, None))
            if lr is not None:
                group[LR_FIELD] = move_to_device(torch.tensor(lr), self.device) if self.compile else lr
                group.setdefault(INITIAL_LR_FIELD, lr)
            for k in self.fixed_fields:
                if k in group:
                    fixed[k] = group[k]
        log.info(f"Building {self.optimizer().__name__} optimizer with {len(optim.param_groups)} param group(s)...")

        def reset_fixed_fields(opt: torch.optim.Optimizer) -> None:
            for fixed, group in zip(fixed_per_group, opt.param_groups):
                group.update(fixed)

        optim.register_load_state_dict_post_hook(reset_fixed_fields)
        runtime = getattr(model, "_sharding_runtime", None)
        if runtime is not None and hasattr(optim, "attach_runtime"):
            optim.attach_runtime(runtime)
        return optim  # type: ignore[return-value]


@dataclass
class MatrixAwareOptimConfig(OptimConfig[Opt], metaclass=ABCMeta):
    """
    Base for optimizers that treat matrices differently from embeddings, vectors and the LM head (Muon,
    Dion): parameters are categorised by role and each category gets its own group options.
    """

    embedding_lr: Optional[float] = None
    lm_head_lr: Optional[float] = None
    vector_lr: Optional[float] = None

    @staticmethod
    def categorize(model: nn.Module) -> Dict[str, List[str]]:
        cats: Dict[str, List[str]] = {"embed": [], "lm_head": [], "vector": [], "matrix": []}
        for n, p in model.named_parameters():
            if not p.requires_grad:
                continue
            if n.startswith("embeddings."):
                cats["embed"].append(n)
            elif n.startswith("lm_head.") and p.ndim >= 2:
                cats["lm_head"].append(n)
            elif p.ndim < 2:
                cats["vector"].append(n)
            else:
                cats["matrix"].append(n)
        return cats

    def categorize_parameters(self, model: nn.Module) -> Dict[str, List[str]]:
        """
        Parameter names by role: ``embed``, ``matrix`` (two-dimensional block parameters), ``vector`` (norm gains,
        biases, scales) and ``lm_head`` (src/olmo_core/optim/config.py:240-277).
        """
        return self.categorize(model)

    def default_group_overrides(self, model: nn.Module) -> List["OptimGroupOverride"]:
        """
        The split the matrix-aware optimizers use: matrices go to the matrix algorithm, everything else to AdamW
        (embeddings without weight decay).
        """
        cats = self.categorize_parameters(model)
        return [OptimGroupOverride(params=cats["matrix"], opts={}),
                OptimGroupOverride(params=cats["vector"], opts=dict(algorithm="adamw")),
                OptimGroupOverride(params=cats["embed"], opts=dict(algorithm="adamw", weight_decay=0.0)),
                OptimGroupOverride(params=cats["lm_head"], opts=dict(algorithm="adamw"))]

    def build_parallelism_config(self) -> Dict[str, Any]:
        """
        What the optimizer needs to know about the sharding of its parameters. The matrix-aware optimizers here gather
        a sharded matrix over the data-parallel group themselves (its group comes with the parameter's shard
        information), so there is no mesh to hand over; tensor parallelism is not supported by them.
        """
        from ..distributed.parallel import MeshDimName, get_world_mesh

        mesh = get_world_mesh()
        if mesh is not None and mesh.mesh_dim_names is not None and MeshDimName.tp in mesh.mesh_dim_names:
            raise NotImplementedError(f"Tensor parallelism is not supported for {type(self).__name__}")
        return {}

    def create_optimizer(self, model: nn.Module, strict: bool = True, **kwargs) -> Opt:
        """Build the optimizer (same as :meth:`build`; extra keyword arguments override config fields)."""
        self.build_parallelism_config()
        return self.replace(**kwargs).build(model, strict=strict) if kwargs else self.build(model, strict=strict)
