"""
Sharded-parameter runtime: the B200-first replacement for the reference's use of FSDP2 / DDP
(src/olmo_core/nn/transformer/model.py:859-968, src/olmo_core/train/train_module/transformer/common.py:119-136).

Layout (per data-parallel rank, sized for 180 GB of HBM3e):

* ``master`` / optimizer moments -- flat fp32 buffers holding only this rank's rows of every parameter
  (dim-0 sharding, the same ownership FSDP2 uses, so checkpoints present identical per-parameter shards);
* ``lowp`` -- one flat bf16 buffer with the *full* compute copy of every parameter, parameter-contiguous so
  each matrix is directly a GEMM operand. It stays resident: parameters are all-gathered once per optimizer
  step, not once per micro-batch per block (a 7B model's bf16 weights are 14.6 GB of 180 GB);
* ``main_grad`` -- one flat full-size gradient buffer (fp32 by default) that the wgrad GEMM epilogues
  accumulate into across micro-batches; it is reduce-scattered once per optimizer step.

Per optimizer step the communication is therefore one reduce-scatter and one all-gather of the model,
instead of the reference's per-micro-batch, per-block all-gathers and reduce-scatters. The mathematical
result is the same up to fp32 summation order: gradients are summed over micro-batches locally and then
averaged over ranks.

Parameters consumed by ops that know about the low-precision copy (dense projections, embeddings, RMSNorm
weights, expert weights) are sharded; all others (biases, router weights, nGPT scalers, ...) are kept
replicated in fp32 and their gradients all-reduced.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import optim as optim_ops

log = logging.getLogger(__name__)

__all__ = ["ShardedParamRuntime", "ShardInfo", "ParamSlot"]


@dataclass
class ShardInfo:
    full_shape: Tuple[int, ...]
    row_start: int
    sharded: bool


@dataclass
class ParamSlot:
    """Where one parameter lives inside the flat buffers."""

    name: str
    param: nn.Parameter
    full_shape: Tuple[int, ...]
    sharded: bool
    local_rows: int
    row_start: int
    master_offset: int  # offset (elements) into the flat master / moment / grad-shard buffers
    local_numel: int
    full_offset: int  # offset into the flat lowp / main_grad buffers (-1 for replicated fp32-only params)
    full_numel: int
    aware: bool  # consumed through ``_lowp`` / ``main_grad`` by the ops


def _is_aware(module: nn.Module, pname: str) -> bool:
    """Parameters whose consumers read ``_lowp`` and write ``main_grad``."""
    from ..nn.feed_forward import Linear
    from ..nn.layer_norm import QwenRMSNorm, RMSNorm
    from ..nn.moe.mlp import MoEMLPBase
    from ..nn.transformer.model import Embedding

    if isinstance(module, Linear):
        return pname == "weight"
    if isinstance(module, Embedding):
        return pname == "weight"
    if isinstance(module, RMSNorm) and not isinstance(module, QwenRMSNorm):
        return pname == "weight"
    if isinstance(module, MoEMLPBase):
        return pname in ("w1", "w2", "w3") and module.__class__.__name__ == "DroplessMoEMLP"
    return False


class ShardedParamRuntime:
    def __init__(
        self,
        model: nn.Module,
        *,
        group=None,
        param_dtype: Optional[torch.dtype] = None,
        reduce_dtype: torch.dtype = torch.float32,
        shard: bool = True,
        device: Optional[torch.device] = None,
    ):
        self.model = model
        self.replicate_group: Optional[dist.ProcessGroup] = None
        if group is not None and hasattr(group, "mesh_dim_names") and getattr(group, "ndim", 1) == 2:
            self.replicate_group = group.get_group(0)
            self.group = group.get_group(1)
        else:
            self.group = group
        distributed = dist.is_available() and dist.is_initialized()
        self.world_size = dist.get_world_size(self.group) if distributed else 1
        self.rank = dist.get_rank(self.group) if distributed else 0
        self.shard = shard and self.world_size > 1
        self.param_dtype = param_dtype
        self.reduce_dtype = reduce_dtype
        self.device = device
        self.slots: List[ParamSlot] = []
        self.master: Optional[torch.Tensor] = None
        self.lowp: Optional[torch.Tensor] = None
        self.main_grad: Optional[torch.Tensor] = None
        self.grad_shard: Optional[torch.Tensor] = None
        self._first_microbatch = True
        self._materialized = False
        self._plan()

    # ------------------------------------------------------------------------------------------------
    # planning and materialisation
    # ------------------------------------------------------------------------------------------------
    def _plan(self) -> None:
        seen: Dict[int, ParamSlot] = {}
        master_off = 0
        full_off = 0
        ws, rank = self.world_size, self.rank
        # sharded + aware parameters first so that their flat ranges are contiguous
        entries = []
        for mname, module in self.model.named_modules():
            for pname, p in module.named_parameters(recurse=False):
                if id(p) in seen or any(e[2] is p for e in entries):
                    continue
                fq = f"{mname}.{pname}" if mname else pname
                entries.append((fq, module, p, pname))
        # The two up-projections of a gated MLP go back to back (w1, then w3) in every flat buffer: stacked, they are one
        # GEMM operand [w1; w3] for the kernels that apply the activation in their epilogue.
        from ..nn.feed_forward import FeedForward

        follower = {}
        for _, module in self.model.named_modules():
            if isinstance(module, FeedForward) and module.w1.weight.shape == module.w3.weight.shape:
                follower[id(module.w1.weight)] = id(module.w3.weight)
        if follower:
            by_id = {id(e[2]): e for e in entries}
            moved = set(follower.values())
            ordered = []
            for e in entries:
                if id(e[2]) in moved:
                    continue
                ordered.append(e)
                nxt = follower.get(id(e[2]))
                if nxt is not None and nxt in by_id:
                    ordered.append(by_id[nxt])
            entries = ordered
        for fq, module, p, pname in entries:
            full_shape = tuple(p.shape)
            aware = _is_aware(module, pname)
            can_shard = self.shard and aware and len(full_shape) >= 1 and full_shape[0] % ws == 0 and full_shape[0] >= ws
            rows = full_shape[0] // ws if can_shard else (full_shape[0] if full_shape else 1)
            row_start = rank * rows if can_shard else 0
            inner = 1
            for s in full_shape[1:]:
                inner *= s
            local_numel = rows * inner if full_shape else 1
            full_numel = p.numel()
            # 16-byte alignment of every slot in every buffer (fp32: 4 elements, bf16: 8 elements)
            master_off = (master_off + 7) // 8 * 8
            full_off = (full_off + 7) // 8 * 8
            slot = ParamSlot(
                name=fq, param=p, full_shape=full_shape, sharded=can_shard, local_rows=rows, row_start=row_start,
                master_offset=master_off, local_numel=local_numel, full_offset=full_off if aware else -1,
                full_numel=full_numel, aware=aware,
            )
            self.slots.append(slot)
            seen[id(p)] = slot
            master_off += local_numel
            if aware:
                full_off += full_numel
        self._master_numel = (master_off + 7) // 8 * 8
        self._full_numel = (full_off + 7) // 8 * 8

    @property
    def materialized(self) -> bool:
        return self._materialized

    def materialize(self, device: torch.device) -> None:
        """Allocate the flat buffers on ``device`` and re-point every parameter at its master shard."""
        if self._materialized:
            return
        self.device = device
        self.master = torch.zeros(self._master_numel, dtype=torch.float32, device=device)
        if self._full_numel > 0:
            # without a low-precision compute dtype the full copy is fp32 (same layout, same code paths)
            lowp_dtype = self.param_dtype or torch.float32
            self._sym_lowp = self._sym_grad = None
            tensor_parallel = any(hasattr(s.param, "_tp_sharded") or hasattr(s.param, "_tp_partial_grad") for s in self.slots)
            if (self.shard and self.replicate_group is None and lowp_dtype == torch.bfloat16
                    and self.reduce_dtype == torch.float32 and not tensor_parallel):
                self._try_symmetric(device)
            if self._sym_grad is not None:
                self.lowp, self.main_grad = self._sym_lowp.tensor, self._sym_grad.tensor
            else:
                self.lowp = torch.zeros(self._full_numel, dtype=lowp_dtype, device=device)
                self.main_grad = torch.zeros(self._full_numel, dtype=self.reduce_dtype, device=device)
        if self.world_size > 1 or self.main_grad is None or self.reduce_dtype != torch.float32:
            self.grad_shard = torch.zeros(self._master_numel, dtype=torch.float32, device=device)
        else:
            self.grad_shard = None  # single rank, fp32: the shard of a gradient *is* the gradient (see grad_view)
        tied: Dict[int, nn.Parameter] = {}
        for slot in self.slots:
            old = slot.param
            local_shape = (slot.local_rows,) + slot.full_shape[1:] if slot.full_shape else ()
            view = self.master[slot.master_offset : slot.master_offset + slot.local_numel].view(local_shape)
            if old.device.type != "meta":
                src = old.data.to(device=device, dtype=torch.float32)
                view.copy_(src.narrow(0, slot.row_start, slot.local_rows) if slot.sharded else src)
            new = nn.Parameter(view, requires_grad=old.requires_grad)
            new._shard_info = ShardInfo(slot.full_shape, slot.row_start, slot.sharded)  # type: ignore[attr-defined]
            for attr in ("_tp_partial_grad", "_tp_sharded"):  # set by olmo_core_b200.parallel.tensor
                if hasattr(old, attr):
                    setattr(new, attr, getattr(old, attr))
            if slot.aware:
                new._lowp = self.lowp[slot.full_offset : slot.full_offset + slot.full_numel].view(slot.full_shape)  # type: ignore[attr-defined]
                new.main_grad = self.main_grad[slot.full_offset : slot.full_offset + slot.full_numel].view(slot.full_shape)  # type: ignore[attr-defined]
            tied[id(old)] = new
            slot.param = new
        # swap parameters inside the modules (handles tied parameters: same object everywhere)
        for module in self.model.modules():
            for pname, p in list(module.named_parameters(recurse=False)):
                if id(p) in tied:
                    module._parameters[pname] = tied[id(p)]
        self._materialized = True

    # ------------------------------------------------------------------------------------------------
    # peer-mapped buffers for the fused optimizer step
    # ------------------------------------------------------------------------------------------------
    @property
    def symmetric(self) -> bool:
        """True when gradients / parameters live in peer-mapped memory and the fused kernels do the collectives."""
        return getattr(self, "_sym_grad", None) is not None

    def _try_symmetric(self, device: torch.device) -> None:
        from .symmetric import SymmetricBuffer, symmetric_memory_enabled

        if not symmetric_memory_enabled(device, self.group):
            return
        try:
            self._sym_lowp = SymmetricBuffer(self._full_numel, torch.bfloat16, device, self.group)
            self._sym_grad = SymmetricBuffer(self._full_numel, torch.float32, device, self.group)
            from ..ops import _lib
            from ctypes import c_float, c_int, c_longlong, c_void_p

            _lib.register_signature("ocb_fused_partials", [])
            _lib.register_signature("ocb_peer_reduce_sumsq", [c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_float,
                                                              c_void_p, c_void_p, c_void_p, c_void_p])
            _lib.register_signature("ocb_adamw_peer_scatter", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                               c_int, c_longlong, c_longlong, c_float, c_float, c_float,
                                                               c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p])
            self._fused_scratch = torch.zeros(_lib.lib().ocb_fused_partials(), dtype=torch.float32, device=device)
            self._sumsq = torch.zeros(2, dtype=torch.float32, device=device)  # [sharded rows, replicated]
            self._sumsq_valid = False
            log.info(f"Sharded-parameter runtime uses peer-mapped buffers: {self._sym_grad}")
        except Exception as e:  # no peer access, allocation failure, ...: the NCCL path still works
            log.warning(f"Peer-mapped buffers unavailable ({type(e).__name__}: {e}); using NCCL collectives")
            self._sym_lowp = self._sym_grad = None

    def _fusable(self, slot: ParamSlot) -> bool:
        n = slot.local_numel if slot.sharded else slot.full_numel
        return slot.aware and n % 4 == 0 and slot.full_offset % 4 == 0 and slot.master_offset % 4 == 0

    def shard_range(self, slot: ParamSlot) -> Tuple[int, int]:
        """``(offset, count)`` of this rank's elements of ``slot`` inside the full flat buffers."""
        if slot.sharded:
            return slot.full_offset + self.rank * slot.local_numel, slot.local_numel
        return slot.full_offset, slot.full_numel

    @torch.no_grad()
    def _reduce_gradients_fused(self) -> None:
        from ..ops import _lib

        lib, stream = _lib.lib(), _lib.stream_ptr()
        sym = self._sym_grad
        self._sumsq.zero_()
        sym.barrier()  # every rank has finished accumulating into its gradient buffer
        for slot in self.slots:
            if not slot.param.requires_grad:
                continue
            out = self.grad_shard[slot.master_offset: slot.master_offset + slot.local_numel]
            if slot.aware and slot.param.grad is not None:
                raise RuntimeError(f"parameter '{slot.name}' received an autograd gradient besides its fused main_grad")
            if self._fusable(slot):
                offset, n = self.shard_range(slot)
                rc = lib.ocb_peer_reduce_sumsq(sym.peer_ptrs, sym.multicast_ptr, self.world_size, offset, n,
                                               1.0 / self.world_size, out.data_ptr(), self._fused_scratch.data_ptr(),
                                               self._sumsq[0 if slot.sharded else 1:].data_ptr(), stream)
                _lib.check(rc, "ocb_peer_reduce_sumsq")
                continue
            # small or oddly sized parameters: NCCL all-reduce of the whole tensor
            if slot.aware:
                full = self.main_grad[slot.full_offset: slot.full_offset + slot.full_numel]
                dist.all_reduce(full, op=dist.ReduceOp.SUM, group=self.group)
                src = full.view(slot.full_shape).narrow(0, slot.row_start, slot.local_rows).reshape(-1) if slot.sharded else full
                out.copy_(src).div_(self.world_size)
            else:
                g = slot.param.grad
                if g is None:
                    out.zero_()
                else:
                    out.copy_(g.reshape(-1).to(torch.float32))
                    slot.param.grad = None
                dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
                out.div_(self.world_size)
            self._sumsq[0 if slot.sharded else 1] += out.float().pow(2).sum()
        self._sumsq_valid = True

    # ------------------------------------------------------------------------------------------------
    # parameter synchronisation
    # ------------------------------------------------------------------------------------------------
    def _own_rows_lowp(self, slot: ParamSlot) -> torch.Tensor:
        full = self.lowp[slot.full_offset : slot.full_offset + slot.full_numel].view(slot.full_shape)
        return full.narrow(0, slot.row_start, slot.local_rows) if slot.sharded else full

    @torch.no_grad()
    def sync_lowp(self) -> None:
        """Refresh the resident low-precision copies from the fp32 master shards (cast + all-gather)."""
        if self.lowp is None:
            return
        for slot in self.slots:
            if slot.aware:
                self._own_rows_lowp(slot).copy_(slot.param.data)
        self.all_gather_lowp()

    @torch.no_grad()
    def all_gather_lowp(self, only_unfused: bool = False) -> None:
        """
        All-gather every sharded parameter's bf16 rows into the full resident copy (in place). With ``only_unfused``
        the parameters whose rows the fused optimizer kernel has already stored into all peers are left out.
        """
        if not self.shard or self.lowp is None:
            return
        sharded = [s for s in self.slots if s.aware and s.sharded and not (only_unfused and self._fusable(s))]
        if not sharded:
            return
        backend_batch = getattr(dist, "_coalescing_manager", None)
        if backend_batch is not None and self.lowp.is_cuda:
            with dist._coalescing_manager(group=self.group, device=self.lowp.device, async_ops=False):
                for slot in sharded:
                    full = self.lowp[slot.full_offset : slot.full_offset + slot.full_numel]
                    dist.all_gather_into_tensor(full, self._own_rows_lowp(slot).reshape(-1), group=self.group)
        else:
            for slot in sharded:
                full = self.lowp[slot.full_offset : slot.full_offset + slot.full_numel]
                dist.all_gather_into_tensor(full, self._own_rows_lowp(slot).reshape(-1).clone(), group=self.group)

    # ------------------------------------------------------------------------------------------------
    # gradients
    # ------------------------------------------------------------------------------------------------
    def grad_view(self, slot: ParamSlot) -> torch.Tensor:
        """fp32 gradient of this rank's rows of ``slot`` (valid after :meth:`reduce_gradients`)."""
        if self.grad_shard is None:
            assert slot.aware
            return self.main_grad[slot.full_offset : slot.full_offset + slot.full_numel].view(slot.full_shape)
        local_shape = (slot.local_rows,) + slot.full_shape[1:] if slot.full_shape else ()
        return self.grad_shard[slot.master_offset : slot.master_offset + slot.local_numel].view(local_shape)

    @torch.no_grad()
    def zero_grad(self) -> None:
        if self.main_grad is not None:
            self.main_grad.zero_()
        for slot in self.slots:
            slot.param.grad = None
        if self.symmetric:
            self._sumsq_valid = False

    @torch.no_grad()
    def adamw_scatter(self, slot: ParamSlot, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, step: torch.Tensor, *,
                      lr: float, betas: Tuple[float, float], eps: float, weight_decay: float,
                      step_factor: Optional[torch.Tensor], grad_scale: Optional[torch.Tensor]) -> bool:
        """
        Fused AdamW + all-gather for ``slot``: updates this rank's master rows and stores their bf16 copies into every
        peer's parameter buffer. Returns False (nothing done) when the slot does not qualify; ``step`` is incremented
        by the caller.
        """
        if not self.symmetric or not self._fusable(slot):
            return False
        from ..ops import _lib

        offset, n = self.shard_range(slot)
        sym = self._sym_lowp
        g = self.grad_shard[slot.master_offset: slot.master_offset + slot.local_numel]
        if slot.sharded:
            peers, mc, world = sym.peer_ptrs, sym.multicast_ptr, self.world_size
        else:  # replicated parameter: every rank computes the same update and writes only its own copy
            import ctypes

            peers, mc, world = (ctypes.c_void_p * 1)(sym.tensor.data_ptr()), None, 1
        rc = _lib.lib().ocb_adamw_peer_scatter(
            slot.param.data.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), g.data_ptr(), peers, mc, world, offset, n,
            lr, betas[0], betas[1], eps, weight_decay, step.data_ptr(), _lib.ptr(step_factor), _lib.ptr(grad_scale),
            _lib.stream_ptr())
        _lib.check(rc, "ocb_adamw_peer_scatter")
        return True

    def finish_scatter(self) -> None:
        """Barrier after the last :meth:`adamw_scatter` of a step: all peers' parameter stores have landed."""
        if self.symmetric:
            self._sym_lowp.barrier()

    @torch.no_grad()
    def reduce_gradients(self) -> None:
        """
        Average gradients over the data-parallel group: reduce-scatter for sharded parameters (each rank
        receives its rows), all-reduce for replicated ones. Afterwards ``grad_view(slot)`` is valid.
        """
        if self.symmetric:
            self._reduce_gradients_fused()
            return
        self._reduce_gradients_nccl()
        self._sync_tensor_parallel_partials()

    def _tp_groups(self):
        """Tensor-parallel groups that parameters of this model were sliced / marked with (usually none or one)."""
        seen = {}
        for slot in self.slots:
            g = getattr(slot.param, "_tp_partial_grad", None)
            if g is not None:
                seen[id(g)] = g
        return list(seen.values())

    @torch.no_grad()
    def _sync_tensor_parallel_partials(self) -> None:
        """Sum, over the tensor-parallel group, the gradients of replicated parameters that saw only a sequence shard."""
        for slot in self.slots:
            group = getattr(slot.param, "_tp_partial_grad", None)
            if group is None or not slot.param.requires_grad:
                continue
            g = self.grad_view(slot) if (slot.aware or self.grad_shard is not None) else slot.param.grad
            if g is not None:
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)

    @torch.no_grad()
    def _reduce_gradients_nccl(self) -> None:
        ws = self.world_size
        single_fp32 = self.grad_shard is None
        for slot in self.slots:
            if not slot.param.requires_grad:
                continue
            if slot.aware:
                full = self.main_grad[slot.full_offset : slot.full_offset + slot.full_numel]
                if slot.param.grad is not None:  # an op without main_grad support produced a regular gradient
                    g = slot.param.grad
                    if slot.sharded:
                        raise RuntimeError(f"parameter '{slot.name}' is sharded but received a local-shape autograd gradient")
                    full.view(slot.full_shape).add_(g.to(full.dtype))
                    slot.param.grad = None
                if single_fp32:
                    continue
                out = self.grad_shard[slot.master_offset : slot.master_offset + slot.local_numel]
                if ws == 1:
                    out.copy_(full)
                elif slot.sharded:
                    if not full.is_cuda:
                        # Gloo has no reduce-scatter: all-reduce the full gradient and keep our rows.
                        dist.all_reduce(full, op=dist.ReduceOp.SUM, group=self.group)
                        out.copy_(full.view(slot.full_shape).narrow(0, slot.row_start, slot.local_rows).reshape(-1)).div_(ws)
                    elif full.dtype == torch.float32:
                        dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.AVG, group=self.group)
                    else:
                        tmp = torch.empty(slot.local_numel, dtype=full.dtype, device=full.device)
                        dist.reduce_scatter_tensor(tmp, full, op=dist.ReduceOp.SUM, group=self.group)
                        out.copy_(tmp).div_(ws)
                else:
                    dist.all_reduce(full, op=dist.ReduceOp.SUM, group=self.group)
                    out.copy_(full).div_(ws)
            else:
                out = self.grad_shard[slot.master_offset : slot.master_offset + slot.local_numel] if not single_fp32 else None
                g = slot.param.grad
                if out is None:
                    # single rank without low-precision copies: keep autograd's gradient as is
                    continue
                if g is None:
                    out.zero_()
                else:
                    out.copy_(g.reshape(-1).to(torch.float32))
                    slot.param.grad = None
                if ws > 1:
                    dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
                    out.div_(ws)
        if self.replicate_group is not None and self.grad_shard is not None:
            dist.all_reduce(self.grad_shard, op=dist.ReduceOp.SUM, group=self.replicate_group)
            self.grad_shard.div_(dist.get_world_size(self.replicate_group))

    @torch.no_grad()
    def grad_norm_sq(self) -> torch.Tensor:
        """Squared global L2 norm of the (reduced) gradients as an fp32 scalar tensor on the device."""
        tp_group = next((getattr(s.param, "_tp_partial_grad", None) for s in self.slots
                         if getattr(s.param, "_tp_partial_grad", None) is not None), None)
        if tp_group is not None:
            # four kinds of gradients: rows split over data-parallel ranks or not, columns/heads split over the
            # tensor-parallel group or not; split ones are summed over the group that splits them, others count once
            buckets = torch.zeros(2, 2, dtype=torch.float32, device=self.device)
            for slot in self.slots:
                g = self.grad_view(slot) if (slot.aware or self.grad_shard is not None) else slot.param.grad
                if g is not None and slot.param.requires_grad:
                    dp_split = int(slot.sharded and self.grad_shard is not None)
                    buckets[dp_split, int(getattr(slot.param, "_tp_sharded", False))] += g.float().pow(2).sum()
            if self.world_size > 1:
                dist.all_reduce(buckets[1], op=dist.ReduceOp.SUM, group=self.group)
            tp_part = buckets[:, 1].sum()
            dist.all_reduce(tp_part, op=dist.ReduceOp.SUM, group=tp_group)
            return tp_part + buckets[:, 0].sum()
        if self.symmetric and self._sumsq_valid:
            # accumulated by the fused reduce kernels; rows are disjoint over ranks, replicated parameters count once
            sharded_part = self._sumsq[0].clone()
            dist.all_reduce(sharded_part, op=dist.ReduceOp.SUM, group=self.group)
            return sharded_part + self._sumsq[1]
        total = torch.zeros((), dtype=torch.float32, device=self.device)
        if self.grad_shard is None:
            optim_ops.sumsq(self.main_grad, out=total, accumulate=True)
            for slot in self.slots:
                if not slot.aware and slot.param.grad is not None:
                    total += slot.param.grad.float().pow(2).sum()
            return total
        # sharded rows are disjoint over ranks; replicated parameters must be counted once
        sharded_part = torch.zeros((), dtype=torch.float32, device=self.device)
        repl_part = torch.zeros((), dtype=torch.float32, device=self.device)
        run_start, run_end, run_sharded = None, None, None
        for slot in self.slots + [None]:
            if slot is not None and run_start is not None and slot.sharded == run_sharded and slot.master_offset <= run_end + 8:
                run_end = slot.master_offset + slot.local_numel
                continue
            if run_start is not None:
                seg = self.grad_shard[run_start:run_end]
                optim_ops.sumsq(seg, out=sharded_part if run_sharded else repl_part, accumulate=True)
            if slot is not None:
                run_start, run_end, run_sharded = slot.master_offset, slot.master_offset + slot.local_numel, slot.sharded
        if self.world_size > 1:
            dist.all_reduce(sharded_part, op=dist.ReduceOp.SUM, group=self.group)
        total = sharded_part + repl_part
        return total

    # ------------------------------------------------------------------------------------------------
    # micro-batch bookkeeping
    # ------------------------------------------------------------------------------------------------
    def named_slots(self) -> Iterable[Tuple[str, ParamSlot]]:
        for s in self.slots:
            yield s.name, s

    def slot_for(self, p: torch.Tensor) -> Optional[ParamSlot]:
        for s in self.slots:
            if s.param is p:
                return s
        return None

    def memory_summary(self) -> str:
        gb = 1 << 30
        parts = [f"master {self._master_numel * 4 / gb:.2f} GiB"]
        if self.lowp is not None:
            parts.append(f"lowp {self.lowp.numel() * self.lowp.element_size() / gb:.2f} GiB")
            parts.append(f"main_grad {self.main_grad.numel() * self.main_grad.element_size() / gb:.2f} GiB")
        if self.grad_shard is not None:
            parts.append(f"grad_shard {self.grad_shard.numel() * 4 / gb:.2f} GiB")
        return ", ".join(parts)

    # ------------------------------------------------------------------------------------------------
    # checkpoint views
    # ------------------------------------------------------------------------------------------------
    def sharded_tensor(self, slot: ParamSlot, local: torch.Tensor):
        """
        Present ``local`` (this rank's rows of a tensor shaped like ``slot``) as a DTensor sharded on dim 0,
        the form ``torch.distributed.checkpoint`` expects; replicated slots and single-rank runs get plain tensors.
        """
        if not slot.sharded or self.world_size == 1:
            return local
        from torch.distributed.device_mesh import DeviceMesh
        from torch.distributed.tensor import DTensor, Shard

        if not hasattr(self, "_ckpt_mesh"):
            ranks = dist.get_process_group_ranks(self.group) if self.group is not None else list(range(self.world_size))
            self._ckpt_mesh = DeviceMesh.from_group(self.group or dist.group.WORLD, local.device.type, mesh=ranks)
        return DTensor.from_local(local, self._ckpt_mesh, [Shard(0)], run_check=False)
