"""
Sharded checkpoints: saving, loading, asynchronous saving, unsharding and partial loading of nested state
dictionaries (API of src/olmo_core/distributed/checkpoint/__init__.py:64-1057).

A checkpoint directory holds ``__{rank}_{i}.distcp`` data files and a pickled ``.metadata`` index (see
:mod:`.filesystem`). Nested state dicts are flattened with ``.`` separators, so a model parameter ``w`` is
stored under ``model.w`` and its AdamW moment under ``optim.state.w.exp_avg``; parameters are written as their
dim-0 shards, one per data-parallel rank, and can be loaded into any other world size or into an unsharded
model.

Models driven by the sharded-parameter runtime (:mod:`olmo_core_b200.parallel.fsdp`) keep their parameters
as rows of flat fp32 master buffers; :func:`model_state` / :func:`optim_state` present those rows as ``DTensor``
shards so that the generic ``torch.distributed.checkpoint`` planners lay the file out exactly as they would
for an FSDP2 model.
"""

from __future__ import annotations

import logging
import re
import tempfile
from concurrent.futures import Future
from dataclasses import dataclass
from enum import Enum
from pathlib import Path
from typing import Any, Dict, Generator, Iterable, List, Optional, Set, Tuple, Union

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dist_cp
import torch.nn as nn
from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner, DefaultSavePlanner
from torch.distributed.checkpoint.metadata import BytesStorageMetadata, Metadata, TensorStorageMetadata

from ...aliases import PathOrStr
from ...config import StrEnum
from ...exceptions import OLMoCheckpointError
from ...io import clear_directory, dir_is_empty, is_url, normalize_path
from ...utils import gc_cuda, wait_for
from ..utils import barrier, get_fs_local_rank, get_local_tensor, get_rank, is_distributed
from .filesystem import RemoteFileSystemReader, RemoteFileSystemWriter
from .keys import merge_state_dicts, prune_state_dict, swap_param_keys
from .unshard import (
    UnshardStrategy,
    UnshardStrategyType,
    get_checkpoint_metadata,
    load_keys,
    load_unsharded_keys,
    unshard_checkpoint,
)

log = logging.getLogger(__name__)

__all__ = [
    "save_state_dict",
    "async_save_state_dict",
    "load_state_dict",
    "save_model_and_optim_state",
    "async_save_model_and_optim_state",
    "load_model_and_optim_state",
    "unshard_checkpoint",
    "load_keys",
    "get_checkpoint_metadata",
    "UnshardStrategy",
    "UnshardStrategyType",
    "swap_param_keys",
    "prune_state_dict",
    "merge_state_dicts",
    "model_state",
    "optim_state",
    "load_model_state",
    "load_optim_state",
]


# ---------------------------------------------------------------------------------------------------------
# presenting a model / optimizer as a checkpointable state dict
# ---------------------------------------------------------------------------------------------------------
def _runtime_of(model: nn.Module):
    return getattr(model, "_sharding_runtime", None)


def _present(model: nn.Module, p: torch.Tensor, local: torch.Tensor) -> torch.Tensor:
    rt = _runtime_of(model)
    if rt is not None:
        slot = rt.slot_for(p)
        if slot is not None:
            return rt.sharded_tensor(slot, local)
    return local


def model_state(model: nn.Module) -> Dict[str, torch.Tensor]:
    """``{fqn: tensor}`` of parameters and persistent buffers; sharded parameters appear as ``DTensor`` shards."""
    out: Dict[str, torch.Tensor] = {n: _present(model, p, p.data) for n, p in model.named_parameters()}
    persistent = set(model.state_dict(keep_vars=True).keys())
    for n, b in model.named_buffers():
        if n in persistent:
            out.setdefault(n, b)
    return out


def _ensure_optim_state(model: nn.Module, optim: torch.optim.Optimizer) -> None:
    """Create the state tensors of ``optim`` (as a first ``step`` would) so that they can be loaded in place."""
    if hasattr(optim, "_init_flat_state") and _runtime_of(model) is not None:
        optim._init_flat_state()
        return
    if hasattr(optim, "init_state"):
        optim.init_state()
        return
    missing = [p for g in optim.param_groups for p in g["params"] if p.requires_grad and not optim.state.get(p)]
    if not missing:
        return
    # A zero-gradient step at lr 0 materialises every built-in optimizer's state without moving parameters.
    saved = [(g, {k: g[k] for k in ("lr", "weight_decay") if k in g}) for g in optim.param_groups]
    grads = [(p, p.grad) for p in missing]
    try:
        for g, _ in saved:
            g["lr"] = 0.0
            if "weight_decay" in g:
                g["weight_decay"] = 0.0
        for p in missing:
            p.grad = torch.zeros_like(p)
        optim.step()
    finally:
        for g, old in saved:
            g.update(old)
        for p, grad in grads:
            p.grad = grad
    for p in missing:
        st = optim.state.get(p, {})
        if torch.is_tensor(st.get("step")):
            st["step"].zero_()


def optim_state(model: nn.Module, optim: torch.optim.Optimizer, *, flatten: bool = True) -> Dict[str, Any]:
    """
    Optimizer state keyed by parameter name. Flattened (what trainer checkpoints use): ``state.<fqn>.<field>`` tensors
    and ``param_groups.<fqn>.<field>`` values. Unflattened (the default of the reference's stand-alone
    ``save_model_and_optim_state``): the same ``state.<fqn>.<field>`` tensors, and ``param_groups`` as a list with one
    dict per group whose ``params`` entry lists parameter names; on disk that list appears as
    ``optim.param_groups.<i>.<field>``.
    """
    name_of = {id(p): n for n, p in model.named_parameters()}
    out: Dict[str, Any] = {}
    if not flatten:
        groups = []
        for group in optim.param_groups:
            names = [name_of[id(p)] for p in group["params"] if id(p) in name_of]
            groups.append({"params": names, **{k: v for k, v in group.items() if k != "params"}})
            for p in group["params"]:
                n = name_of.get(id(p))
                if n is None:
                    continue
                for field, value in optim.state.get(p, {}).items():
                    if torch.is_tensor(value) and value.dim() > 0:
                        value = _present(model, p, value)
                    out[f"state.{n}.{field}"] = value
        out["param_groups"] = groups
        return out
    for group in optim.param_groups:
        for p in group["params"]:
            n = name_of.get(id(p))
            if n is None:
                continue
            for field, value in optim.state.get(p, {}).items():
                if torch.is_tensor(value) and value.dim() > 0:
                    value = _present(model, p, value)
                out[f"state.{n}.{field}"] = value
            for field, value in group.items():
                if field != "params":
                    out[f"param_groups.{n}.{field}"] = value
    return out


@torch.no_grad()
def load_model_state(model: nn.Module, state: Dict[str, torch.Tensor], *, strict: bool = True) -> None:
    """Copy ``state`` (as produced by :func:`model_state`, possibly loaded into in place) into ``model``."""
    params = dict(model.named_parameters())
    buffers = dict(model.named_buffers())
    for n, value in state.items():
        target = params.get(n)
        target = target.data if target is not None else buffers.get(n)
        if target is None:
            if strict:
                raise KeyError(f"unexpected key '{n}' in model state dict")
            continue
        src = get_local_tensor(value)
        if src.data_ptr() != target.data_ptr() or src.device != target.device:
            target.copy_(src)
    if strict:
        missing = set(params) - set(state)
        if missing:
            raise KeyError(f"model state dict is missing keys: {sorted(missing)}")
    rt = _runtime_of(model)
    if rt is not None and rt.materialized:
        rt.sync_lowp()


@torch.no_grad()
def load_optim_state(model: nn.Module, optim: torch.optim.Optimizer, state: Dict[str, Any]) -> None:
    _ensure_optim_state(model, optim)
    name_of = {id(p): n for n, p in model.named_parameters()}
    saved_groups = state.get("param_groups")
    if isinstance(saved_groups, list):  # unflattened layout: one dict per group, in the optimizer's group order
        if len(saved_groups) != len(optim.param_groups):
            raise ValueError(f"checkpoint has {len(saved_groups)} optimizer param groups, the optimizer has "
                             f"{len(optim.param_groups)}")
        for group, saved in zip(optim.param_groups, saved_groups):
            for field, value in saved.items():
                if field not in ("params", "initial_lr") and field in group:
                    group[field] = value
    for group in optim.param_groups:
        for p in group["params"]:
            n = name_of.get(id(p))
            if n is None:
                continue
            for field, cur in optim.state.get(p, {}).items():
                key = f"state.{n}.{field}"
                if key not in state:
                    continue
                new = state[key]
                if torch.is_tensor(cur):
                    src = get_local_tensor(new) if torch.is_tensor(new) else torch.as_tensor(new)
                    if src.data_ptr() != cur.data_ptr():
                        cur.copy_(src.to(cur.device))
                else:
                    optim.state[p][field] = new
            for field in list(group.keys()):
                key = f"param_groups.{n}.{field}"
                if field not in ("params", "initial_lr") and key in state:
                    group[field] = state[key]


# ---------------------------------------------------------------------------------------------------------
# saving and loading nested state dicts
# ---------------------------------------------------------------------------------------------------------
def _prepare_target_dir(dir: PathOrStr, process_group: Optional[dist.ProcessGroup], save_overwrite: bool) -> str:
    """Normalise ``dir`` and make sure it is empty (clearing it first when overwriting is allowed)."""
    dir = normalize_path(dir)
    if get_fs_local_rank(process_group) == 0 or is_url(dir):
        if get_rank(process_group) == 0 or not is_url(dir):
            if save_overwrite:
                clear_directory(dir)
            elif not dir_is_empty(dir):
                raise FileExistsError(f"checkpoint directory '{dir}' is not empty (pass save_overwrite=True to replace it)")
    barrier(process_group)
    if not is_url(dir):
        if get_fs_local_rank(process_group) == 0:
            Path(dir).mkdir(parents=True, exist_ok=True)
        # On a shared file system the directory may take a moment to appear on the other ranks.
        wait_for(lambda: Path(dir).exists(), f"directory '{dir}' to be created", timeout=30.0)
    barrier(process_group)
    return dir


def _save_planner() -> DefaultSavePlanner:
    return DefaultSavePlanner(dedup_save_to_lowest_rank=True)


@torch.no_grad()
def save_state_dict(
    dir: PathOrStr,
    state_dict: Dict[str, Any],
    process_group: Optional[dist.ProcessGroup] = None,
    save_overwrite: bool = False,
    thread_count: Optional[int] = None,
    process_count: Optional[int] = None,
    throttle_uploads: bool = False,
    enable_plan_caching: bool = False,
    _skip_prepare: bool = False,
) -> None:
    """
    Write an arbitrary nested state dict (tensors, ``DTensor`` shards, picklable leaves) to ``dir``. ``process_count``
    (a process pool in the reference) is served by the writer's thread pool: the files are written by threads that spend
    their time in ``write`` system calls, not in the interpreter. ``_skip_prepare``: the target directory was already
    checked / cleared by the caller.
    """
    del enable_plan_caching  # the plan is cheap to rebuild at these sizes; accepted for API compatibility
    thread_count = thread_count if thread_count is not None else process_count
    if not _skip_prepare:
        dir = _prepare_target_dir(dir, process_group, save_overwrite)
    writer = RemoteFileSystemWriter(dir, thread_count=thread_count, process_group=process_group,
                                    throttle_uploads=throttle_uploads, save_overwrite=save_overwrite)
    dist_cp.state_dict_saver.save(state_dict, storage_writer=writer, process_group=process_group,
                                  planner=_save_planner(), no_dist=not is_distributed())


@torch.no_grad()
def async_save_state_dict(
    dir: PathOrStr,
    state_dict: Dict[str, Any],
    process_group: Optional[dist.ProcessGroup] = None,
    save_overwrite: bool = False,
    thread_count: Optional[int] = None,
    process_count: Optional[int] = None,
    throttle_uploads: bool = False,
    enable_plan_caching: bool = False,
    _skip_prepare: bool = False,
) -> Future:
    """
    Like :func:`save_state_dict`, but returns once the state has been staged in host memory; the returned future
    completes when the files are written. In distributed runs ``process_group`` should be a group with a CPU
    (gloo) backend that is not used for anything else while the save is in flight.
    """
    del enable_plan_caching
    thread_count = thread_count if thread_count is not None else process_count
    if not _skip_prepare:
        dir = _prepare_target_dir(dir, process_group, save_overwrite)
    writer = RemoteFileSystemWriter(dir, thread_count=thread_count, process_group=process_group,
                                    throttle_uploads=throttle_uploads, save_overwrite=save_overwrite)
    if is_distributed():
        return dist_cp.state_dict_saver.async_save(state_dict, storage_writer=writer, process_group=process_group,
                                                   planner=_save_planner())
    # Single process: stage to host memory now, write on a worker thread.
    from concurrent.futures import ThreadPoolExecutor

    staged = _stage_to_host(state_dict)
    pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="ckpt-save")
    fut = pool.submit(dist_cp.state_dict_saver.save, staged, storage_writer=writer, planner=_save_planner(), no_dist=True)
    fut.add_done_callback(lambda _: pool.shutdown(wait=False))
    return fut


def _stage_to_host(obj: Any) -> Any:
    if torch.is_tensor(obj):
        t = get_local_tensor(obj).detach()
        return t.to("cpu", copy=True)
    if isinstance(obj, dict):
        return {k: _stage_to_host(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_stage_to_host(v) for v in obj)
    return obj


@torch.no_grad()
def load_state_dict(
    dir: PathOrStr,
    state_dict: Dict[str, Any],
    process_group: Optional[dist.ProcessGroup] = None,
    pre_download: bool = False,
    work_dir: Optional[PathOrStr] = None,
    thread_count: Optional[int] = None,
) -> None:
    """Load ``dir`` into ``state_dict`` in place (tensors are filled, other leaves replaced)."""
    dir = normalize_path(dir)
    reader = RemoteFileSystemReader(dir, thread_count=thread_count, pre_download=pre_download, work_dir=work_dir)
    _dcp_load(state_dict, dir, reader, process_group)


def _dcp_load(state_dict: Dict[str, Any], dir: str, reader: RemoteFileSystemReader,
              process_group: Optional[dist.ProcessGroup]) -> None:
    """``dist_cp.load`` with its failures (a ``BaseException`` subclass that wraps per-rank tracebacks) turned into one
    :class:`OLMoCheckpointError` that names the checkpoint and the first underlying cause."""
    from torch.distributed.checkpoint.api import CheckpointException

    try:
        dist_cp.state_dict_loader.load(state_dict, checkpoint_id=dir, storage_reader=reader, process_group=process_group,
                                       no_dist=not is_distributed())
    except CheckpointException as e:
        causes = [f"rank {r}: {type(x).__name__}: {x}" for r, x in sorted(getattr(e, "failures", {}).items())]
        raise OLMoCheckpointError(f"could not load checkpoint '{dir}': " + ("; ".join(causes) or str(e))) from e


def _model_optim_state(model: nn.Module, optim: Optional[torch.optim.Optimizer], *, for_load: bool = False,
                       flatten: bool = True) -> Dict[str, Any]:
    sd: Dict[str, Any] = {"model": model_state(model)}
    if optim is not None:
        if for_load:
            _ensure_optim_state(model, optim)
        sd["optim"] = optim_state(model, optim, flatten=flatten)
    return sd


UNFLATTENED_MARKER = "optim.param_groups.0.params"
"""Present in a checkpoint's metadata exactly when its optimizer state was written unflattened."""


@torch.no_grad()
def save_model_and_optim_state(
    dir: PathOrStr,
    model: nn.Module,
    optim: Optional[torch.optim.Optimizer] = None,
    *,
    process_group: Optional[dist.ProcessGroup] = None,
    save_overwrite: bool = False,
    flatten_optimizer_state: bool = False,
    thread_count: Optional[int] = None,
    process_count: Optional[int] = None,
    throttle_uploads: bool = False,
    enable_plan_caching: bool = False,
) -> None:
    """
    Save model (and optimizer) state under the keys ``model.*`` / ``optim.*``. The result can be loaded with any
    other sharding, world size or wrapping, and by the reference implementation.
    """
    save_state_dict(dir, _model_optim_state(model, optim, flatten=flatten_optimizer_state), process_group=process_group, save_overwrite=save_overwrite,
                    thread_count=thread_count, process_count=process_count, throttle_uploads=throttle_uploads,
                    enable_plan_caching=enable_plan_caching)


@torch.no_grad()
def async_save_model_and_optim_state(
    dir: PathOrStr,
    model: nn.Module,
    optim: Optional[torch.optim.Optimizer] = None,
    *,
    process_group: Optional[dist.ProcessGroup] = None,
    save_overwrite: bool = False,
    flatten_optimizer_state: bool = False,
    thread_count: Optional[int] = None,
    process_count: Optional[int] = None,
    throttle_uploads: bool = False,
    enable_plan_caching: bool = False,
) -> Future:
    return async_save_state_dict(dir, _model_optim_state(model, optim, flatten=flatten_optimizer_state), process_group=process_group,
                                 save_overwrite=save_overwrite, thread_count=thread_count, process_count=process_count,
                                 throttle_uploads=throttle_uploads, enable_plan_caching=enable_plan_caching)


@torch.no_grad()
def load_model_and_optim_state(
    dir: PathOrStr,
    model: nn.Module,
    optim: Optional[torch.optim.Optimizer] = None,
    *,
    process_group: Optional[dist.ProcessGroup] = None,
    key_mapping: Optional[Dict[str, str]] = None,
    pre_download: bool = False,
    work_dir: Optional[PathOrStr] = None,
    strict: bool = True,
    flatten_optimizer_state: bool = False,
    thread_count: Optional[int] = None,
) -> None:
    """
    Load a checkpoint written by :func:`save_model_and_optim_state` (here or by the reference) into ``model`` and
    ``optim``. ``key_mapping`` maps current parameter names to the names used in the checkpoint.
    """
    dir = normalize_path(dir)
    reader = RemoteFileSystemReader(dir, thread_count=thread_count, pre_download=pre_download, work_dir=work_dir)
    metadata = reader.read_metadata()
    # the layout on disk decides, whatever the caller asked for (both layouts are in use: see optim_state)
    on_disk_flat = UNFLATTENED_MARKER not in metadata.state_dict_metadata
    if optim is not None and on_disk_flat != flatten_optimizer_state and any(
            k.startswith("optim.") for k in metadata.state_dict_metadata):
        log.info(f"Checkpoint at '{dir}' holds {'a flattened' if on_disk_flat else 'an unflattened'} optimizer state; "
                 "loading it in that layout")
    sd = _model_optim_state(model, optim, for_load=True, flatten=on_disk_flat)
    if optim is not None and not on_disk_flat:
        # another optimizer class may have written other group fields: ask only for those that are on disk
        for i, group in enumerate(sd["optim"]["param_groups"]):
            for field in list(group.keys()):
                if f"optim.param_groups.{i}.{field}" not in metadata.state_dict_metadata:
                    del group[field]
    if key_mapping is not None:
        swap_param_keys(sd, key_mapping, metadata=metadata)
    if not strict:
        pruned = prune_state_dict(sd, set(metadata.state_dict_metadata.keys()))
        if pruned:
            log.warning(f"Checkpoint at '{dir}' is missing keys: {sorted(pruned)}")
    _dcp_load(sd, dir, reader, process_group)
    if key_mapping is not None:
        swap_param_keys(sd, key_mapping, reverse=True, quiet=True)
    load_model_state(model, sd["model"], strict=strict)
    if optim is not None:
        load_optim_state(model, optim, sd["optim"])
    gc_cuda()
