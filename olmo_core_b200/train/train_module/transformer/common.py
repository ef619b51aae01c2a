"""
``parallelize_model``: applies the configured parallelism / memory strategies to a transformer in the order
pipeline -> float8 -> context -> tensor -> expert -> activation checkpointing -> (compile) -> data parallel ->
weight initialisation (the order of src/olmo_core/train/train_module/transformer/common.py:34-158).
"""

from __future__ import annotations

import logging
from typing import Optional

import torch

from ....distributed.parallel import (
    DataParallelType,
    get_cp_mesh,
    get_dp_model_mesh,
    get_ep_mesh,
    get_tp_mesh,
)
from ....float8 import Float8Config
from ....nn.transformer import MoETransformer, Transformer

log = logging.getLogger(__name__)

__all__ = ["parallelize_model"]


def parallelize_model(
    model: Transformer,
    *,
    world_mesh=None,
    device: torch.device,
    max_sequence_length: int,
    rank_microbatch_size: int,
    compile_model: bool = False,
    float8_config: Optional[Float8Config] = None,
    dp_config=None,
    tp_config=None,
    cp_config=None,
    ep_config=None,
    ac_config=None,
    pp_enabled: bool = False,
    init_weights: bool = True,
) -> Transformer:
    if float8_config is not None and float8_config.enabled:
        model.apply_fp8(float8_config)
        log.info("Swapped linear layers to Float8 linear layers")
    if cp_config is not None:
        assert world_mesh is not None
        model.apply_cp(get_cp_mesh(world_mesh), ring=cp_config.ring, uly=cp_config.uly)
        log.info(f"Applied context parallelism (degree {cp_config.degree})")
    if tp_config is not None:
        assert world_mesh is not None
        tp_mesh = get_tp_mesh(world_mesh)
        model.apply_tp(tp_mesh, float8_enabled=float8_config is not None and float8_config.enabled)
        tp_config.maybe_enable_async_tp(tp_mesh)
        log.info(f"Applied {'async ' if tp_config.enable_async else ''}tensor parallelism (degree {tp_config.degree})")
    if ep_config is not None:
        assert world_mesh is not None
        if not isinstance(model, MoETransformer):
            raise ValueError("expert parallelism is only valid for MoE models")
        model.apply_ep(get_ep_mesh(world_mesh))
        log.info("Applied expert parallelism")
    if ac_config is not None:
        model.apply_activation_checkpointing(**ac_config.as_kwargs())
        log.info(f"Applied '{ac_config.mode}' activation checkpointing")
    if compile_model:
        model.apply_compile()
    if dp_config is None and tp_config is not None:
        # the parameter runtime also owns the tensor-parallel gradient bookkeeping (partial-gradient sums, global norm)
        dp_mesh = get_dp_model_mesh(world_mesh) if world_mesh is not None else None
        model.apply_ddp(dp_mesh=dp_mesh, param_dtype=None)
    if dp_config is not None:
        dp_mesh = get_dp_model_mesh(world_mesh) if world_mesh is not None else None
        param_dtype = dp_config.param_dtype.as_pt() if dp_config.param_dtype is not None else None
        if dp_config.name in (DataParallelType.fsdp, DataParallelType.hsdp):
            if isinstance(model, MoETransformer):
                model.prepare_experts_for_fsdp()
            model.apply_fsdp(dp_mesh=dp_mesh, param_dtype=param_dtype, reduce_dtype=dp_config.reduce_dtype.as_pt(),
                             pp_enabled=pp_enabled, prefetch_factor=getattr(dp_config, "prefetch_factor", 0),
                             wrapping_strategy=getattr(dp_config, "wrapping_strategy", "full"))
            log.info(f"Applied sharded data parallelism ({dp_config.name})")
        elif dp_config.name == DataParallelType.ddp:
            if isinstance(model, MoETransformer):
                model.prepare_experts_for_ddp()
            model.apply_ddp(dp_mesh=dp_mesh, param_dtype=param_dtype)
            log.info("Applied replicated data parallelism")
        else:
            raise NotImplementedError(dp_config.name)

    runtime = getattr(model, "_sharding_runtime", None)
    if runtime is not None:
        runtime.materialize(device)
        model._device = device
    if init_weights:
        log.info("Initializing model weights...")
        model.init_weights(max_seq_len=max_sequence_length, max_local_microbatch_size=rank_microbatch_size, device=device,
                           world_mesh=world_mesh)
        if runtime is not None:
            runtime.sync_lowp()
    return model
