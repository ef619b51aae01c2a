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

Two memory modes. *Resident* (above) costs 6 bytes per parameter on every rank regardless of the world size and is
the fast path while that fits (a 7B model: 44 GB). *Streamed* is chosen when it would not (or with
``OLMO_CORE_B200_FSDP_STREAMED=1``): the transformer blocks keep only this rank's rows (bf16 ``lowp_shard``, fp32
``grad_shard``); a block's full bf16 weights are assembled into a two-slot ring one block ahead of the compute
(``ocb_peer_gather_segments``: plain loads from the owners' memory on a side stream, or NCCL all-gather), and its
full-size gradients leave the ring right after the block's backward (``ocb_peer_scatter_add_segments``: fp32
reductions into the owners' shards, or NCCL reduce-scatter). Per-GPU memory then scales with 1 / world size, which is
what a 32B model needs. Embeddings, the final norm and the LM head stay resident in both modes.

Parameters whose leading dimension is not a multiple of the world size are padded (the last ranks own fewer real
rows, the same split ``torch.chunk`` / FSDP2 use), never replicated.

Parameters consumed by ops that know about the low-precision copy (dense projections, embeddings, RMSNorm
weights, expert weights) are sharded; all others (biases, router weights, nGPT scalers, ...) are kept
replicated in fp32 and their gradients all-reduced.
"""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import optim as optim_ops

log = logging.getLogger(__name__)

__all__ = ["ShardedParamRuntime", "ShardInfo", "ParamSlot"]

STREAMED_ENV_VAR = "OLMO_CORE_B200_FSDP_STREAMED"
EARLY_REDUCE_ENV_VAR = "OLMO_CORE_B200_FSDP_EARLY_REDUCE"


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
    flat_numel: int = 0  # elements the full copy occupies in a flat buffer (padded rows included)
    padded_rows: int = 0  # leading dimension rounded up to a multiple of the world size (sharded slots)
    unit: int = -1  # streamed mode: index of the transformer block whose ring slot holds the full copy; -1 = resident
    block: int = -1  # resident mode: index of the transformer block that owns the parameter (-1: embeddings, head, ...)

    @property
    def real_local_rows(self) -> int:
        """Rows of this rank's shard that exist in the parameter (the rest is padding)."""
        if not self.sharded or not self.full_shape:
            return self.local_rows
        return max(0, min(self.local_rows, self.full_shape[0] - self.row_start))


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
        streamed: Optional[bool] = None,
    ):
        self.model = model
        self._streamed_request = streamed
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
        self.streamed = False
        self.units: List[List[ParamSlot]] = []
        self.lowp_shard: Optional[torch.Tensor] = None
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
        # Streamed mode: the parameters of transformer block i form unit i; their full copies live in a ring slot.
        unit_of: Dict[int, int] = {}
        blocks = getattr(self.model, "blocks", None)
        if self._want_streamed(entries) and blocks is not None and len(blocks) >= 2:
            for i, block in enumerate(blocks.values() if hasattr(blocks, "values") else blocks):
                for bp in block.parameters():
                    unit_of.setdefault(id(bp), i)
            self.streamed = True
        # Resident mode: which transformer block a parameter belongs to (its gradients can be reduced as soon as the last
        # micro-batch's backward has left that block).
        self._block_of: Dict[int, int] = {}
        if blocks is not None and not self.streamed:
            for i, block in enumerate(blocks.values() if hasattr(blocks, "values") else blocks):
                for bp in block.parameters():
                    self._block_of.setdefault(id(bp), i)
        unit_off: Dict[int, int] = {}
        for fq, module, p, pname in entries:
            full_shape = tuple(p.shape)
            aware = _is_aware(module, pname)
            can_shard = self.shard and aware and len(full_shape) >= 1
            inner = 1
            for s in full_shape[1:]:
                inner *= s
            if can_shard:
                rows = -(-full_shape[0] // ws)  # torch.chunk's split: ceil-sized shards, the last ones short or empty
                padded_rows = rows * ws
                row_start = rank * rows
            else:
                rows = full_shape[0] if full_shape else 1
                padded_rows = rows
                row_start = 0
            local_numel = rows * inner if full_shape else 1
            full_numel = p.numel()
            flat_numel = padded_rows * inner if full_shape else 1
            unit = unit_of.get(id(p), -1) if (aware and can_shard) else -1
            # 16-byte alignment of every slot in every buffer (fp32: 4 elements, bf16: 8 elements)
            master_off = (master_off + 7) // 8 * 8
            if unit >= 0:
                off = (unit_off.get(unit, 0) + 7) // 8 * 8
                unit_off[unit] = off + flat_numel
            else:
                full_off = (full_off + 7) // 8 * 8
                off = full_off
            slot = ParamSlot(
                name=fq, param=p, full_shape=full_shape, sharded=can_shard, local_rows=rows, row_start=row_start,
                master_offset=master_off, local_numel=local_numel, full_offset=off if aware else -1,
                full_numel=full_numel, aware=aware, padded_rows=padded_rows, unit=unit, flat_numel=flat_numel,
            )
            slot.block = self._block_of.get(id(p), -1)
            self.slots.append(slot)
            seen[id(p)] = slot
            master_off += local_numel
            if aware and unit < 0:
                full_off += flat_numel
        self._master_numel = (master_off + 7) // 8 * 8
        self._full_numel = (full_off + 7) // 8 * 8
        self._unit_numel = (max(unit_off.values()) + 7) // 8 * 8 if unit_off else 0
        if self.streamed:
            n_units = max(unit_off) + 1
            self.units = [[s for s in self.slots if s.unit == u] for u in range(n_units)]

    def _want_streamed(self, entries) -> bool:
        """Streamed mode on request, or when the resident layout would take more than 35 % of the device's memory."""
        if not self.shard:
            return False
        env = os.environ.get(STREAMED_ENV_VAR)
        if env is not None:
            return env not in ("0", "")
        if self._streamed_request is not None:
            return bool(self._streamed_request)
        if not torch.cuda.is_available():
            return False
        resident = 6 * sum(e[2].numel() for e in entries)
        try:
            total = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
        except Exception:
            return False
        return resident > 0.35 * total

    @property
    def materialized(self) -> bool:
        return self._materialized

    def materialize(self, device: torch.device) -> None:
        """Allocate the flat buffers on ``device`` and re-point every parameter at its master shard."""
        if self._materialized:
            return
        self.device = device
        self._check_memory(device)
        self.master = torch.zeros(self._master_numel, dtype=torch.float32, device=device)
        lowp_dtype = self.param_dtype or torch.float32  # without a compute dtype the full copy is fp32 (same layout)
        self._sym_lowp = self._sym_grad = None
        tensor_parallel = any(hasattr(s.param, "_tp_sharded") or hasattr(s.param, "_tp_partial_grad") for s in self.slots)
        peer_ok = (self.shard and self.replicate_group is None and lowp_dtype == torch.bfloat16
                   and self.reduce_dtype == torch.float32 and not tensor_parallel)
        if self._full_numel > 0:
            if peer_ok and not self.streamed:
                self._try_symmetric(device)
            if self._sym_grad is not None:
                self.lowp, self.main_grad = self._sym_lowp.tensor, self._sym_grad.tensor
            else:
                self.lowp = torch.zeros(self._full_numel, dtype=lowp_dtype, device=device)
                self.main_grad = torch.zeros(self._full_numel, dtype=self.reduce_dtype, device=device)
        if (self.world_size > 1 or self.main_grad is None or self.reduce_dtype != torch.float32
                or self.replicate_group is not None or self.streamed):
            self.grad_shard = torch.zeros(self._master_numel, dtype=torch.float32, device=device)
        else:
            self.grad_shard = None  # single rank, fp32: the shard of a gradient *is* the gradient (see grad_view)
        if self.streamed:
            self._materialize_streamed(device, lowp_dtype, peer_ok)
        elif self._sym_grad is not None:
            self._install_early_reduce(device)
        tied: Dict[int, nn.Parameter] = {}
        for slot in self.slots:
            old = slot.param
            local_shape = (slot.local_rows,) + slot.full_shape[1:] if slot.full_shape else ()
            view = self.master[slot.master_offset : slot.master_offset + slot.local_numel].view(local_shape)
            if old.device.type != "meta":
                src = old.data.to(device=device, dtype=torch.float32)
                if slot.sharded:
                    real = slot.real_local_rows
                    if real > 0:
                        view[:real].copy_(src.narrow(0, slot.row_start, real))
                else:
                    view.copy_(src)
            new = nn.Parameter(view, requires_grad=old.requires_grad)
            new._shard_info = ShardInfo(slot.full_shape, slot.row_start, slot.sharded)  # type: ignore[attr-defined]
            for attr in ("_tp_partial_grad", "_tp_sharded"):  # set by olmo_core_b200.parallel.tensor
                if hasattr(old, attr):
                    setattr(new, attr, getattr(old, attr))
            if slot.aware:
                lowp_buf, grad_buf = self._full_buffers(slot)
                new._lowp = lowp_buf[slot.full_offset : slot.full_offset + slot.full_numel].view(slot.full_shape)  # type: ignore[attr-defined]
                new.main_grad = grad_buf[slot.full_offset : slot.full_offset + slot.full_numel].view(slot.full_shape)  # type: ignore[attr-defined]
            tied[id(old)] = new
            slot.param = new
        # swap parameters inside the modules (handles tied parameters: same object everywhere)
        for module in self.model.modules():
            for pname, p in list(module.named_parameters(recurse=False)):
                if id(p) in tied:
                    module._parameters[pname] = tied[id(p)]
        self._materialized = True

    def _full_buffers(self, slot: ParamSlot) -> Tuple[torch.Tensor, torch.Tensor]:
        """The flat buffers that hold the full low-precision copy / full-size gradient of ``slot``."""
        if slot.unit >= 0:
            return self._ring_lowp[slot.unit % 2], self._ring_grad[slot.unit % 2]
        return self.lowp, self.main_grad

    def _check_memory(self, device: torch.device) -> None:
        """Refuse a layout that cannot fit instead of dying in an allocation half way through."""
        if device.type != "cuda":
            return
        from ..exceptions import OLMoConfigurationError

        master = 12 * self._master_numel  # fp32 master + two fp32 moments
        if self.streamed:
            state = master + 6 * self._master_numel + 6 * self._full_numel + 2 * 6 * self._unit_numel
        else:
            state = master + 6 * self._full_numel + (4 * self._master_numel if self.world_size > 1 else 0)
        total = torch.cuda.get_device_properties(device).total_memory
        if state > 0.95 * total:
            gb = 1 << 30
            raise OLMoConfigurationError(
                f"parameters, gradients and optimizer state need {state / gb:.1f} GiB per GPU "
                f"({'streamed' if self.streamed else 'resident'} layout: {self._full_numel * 6 / gb:.1f} GiB full copies, "
                f"{master / gb:.1f} GiB sharded state) but the device has {total / gb:.1f} GiB; use more data-parallel "
                f"ranks{'' if self.streamed else f' or set {STREAMED_ENV_VAR}=1'}")

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

    # -- resident mode: reduction overlapped with the last micro-batch's backward -------------------------------------
    def _install_early_reduce(self, device: torch.device) -> None:
        """
        Reduce a block's gradients on a side stream as soon as the backward pass of the LAST micro-batch of a step has
        left the block (the reference's FSDP reduce-scatters per block inside backward:
        src/olmo_core/train/train_module/transformer/train_module.py:565-584). Whoever drives the step announces the
        micro-batches with :meth:`begin_microbatch`; without that announcement everything is reduced in
        :meth:`reduce_gradients` as before. ``OLMO_CORE_B200_FSDP_EARLY_REDUCE=0`` switches the overlap off.
        """
        self._early_enabled = os.environ.get(EARLY_REDUCE_ENV_VAR, "1") != "0" and device.type == "cuda"
        self._early_reduced: set = set()
        self.early_reduce_blocks = 0  # blocks reduced behind their backward so far (diagnostics)
        self._last_microbatch = False
        self._early_stream = torch.cuda.Stream(device) if self._early_enabled else None
        blocks = getattr(self.model, "blocks", None)
        if not self._early_enabled or blocks is None:
            return
        for u, block in enumerate(blocks.values() if hasattr(blocks, "values") else blocks):
            block.register_full_backward_hook(lambda m, grad_in, grad_out, u=u: self._early_reduce_block(u))

    def begin_microbatch(self, index: int, count: int) -> None:
        """Called by the train module before the forward pass of micro-batch ``index`` of ``count``."""
        self._last_microbatch = index == count - 1

    @torch.no_grad()
    def _early_reduce_block(self, u: int) -> None:
        if not (getattr(self, "_early_enabled", False) and self._last_microbatch) or u in self._early_reduced:
            return
        slots = [s for s in self.slots if getattr(s, "block", -1) == u and s.param.requires_grad and self._fusable(s)]
        if not slots:
            return
        cur = torch.cuda.current_stream(self.device)
        side = self._early_stream
        side.wait_stream(cur)  # this block's weight gradients are complete on this rank
        with torch.cuda.stream(side):
            if not self._early_reduced:
                self._sumsq.zero_()
            self._sym_grad.barrier()  # ... and on every other rank
            self._launch_reduce(slots, side.cuda_stream)
        self._early_reduced.add(u)
        self.early_reduce_blocks += 1

    def _launch_reduce(self, slots, stream: int) -> None:
        from ..ops import _lib

        lib, sym = _lib.lib(), self._sym_grad
        for slot in slots:
            out = self.grad_shard[slot.master_offset: slot.master_offset + slot.local_numel]
            offset, n = self.shard_range(slot)
            rc = lib.ocb_peer_reduce_sumsq(sym.peer_ptrs, sym.multicast_ptr, self.world_size, offset, n,
                                           1.0 / self.world_size, out.data_ptr(), self._fused_scratch.data_ptr(),
                                           self._sumsq[0 if slot.sharded else 1:].data_ptr(), stream)
            _lib.check(rc, "ocb_peer_reduce_sumsq")

    @torch.no_grad()
    def _reduce_gradients_fused(self) -> None:
        from ..ops import _lib

        lib, stream = _lib.lib(), _lib.stream_ptr()
        sym = self._sym_grad
        early = getattr(self, "_early_reduced", set())
        if early:
            torch.cuda.current_stream(self.device).wait_stream(self._early_stream)  # their sums are in grad_shard / _sumsq
        else:
            self._sumsq.zero_()
        self._last_microbatch = False
        sym.barrier()  # every rank has finished accumulating into its gradient buffer
        for slot in self.slots:
            if not slot.param.requires_grad:
                continue
            if getattr(slot, "block", -1) in early and self._fusable(slot):
                continue  # reduced behind its block's backward
            out = self.grad_shard[slot.master_offset: slot.master_offset + slot.local_numel]
            if slot.aware and slot.param.grad is not None:
                raise RuntimeError(f"parameter '{slot.name}' received an autograd gradient besides its fused main_grad")
            if self._fusable(slot):
                self._launch_reduce([slot], stream)
                continue
            # small or oddly sized parameters: NCCL all-reduce of the whole tensor
            if slot.aware:
                full = self._flat(self.main_grad, slot)
                dist.all_reduce(full, op=dist.ReduceOp.SUM, group=self.group)
                src = full[self.rank * slot.local_numel: (self.rank + 1) * slot.local_numel] if slot.sharded else full
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
        if early:
            early.clear()

    # ------------------------------------------------------------------------------------------------
    # parameter synchronisation
    # ------------------------------------------------------------------------------------------------
    def _flat(self, buf: torch.Tensor, slot: ParamSlot) -> torch.Tensor:
        """The (padded) full extent of ``slot`` inside a flat full-size buffer."""
        return buf[slot.full_offset : slot.full_offset + slot.flat_numel]

    def _own_rows_lowp(self, slot: ParamSlot) -> torch.Tensor:
        """This rank's rows of the low-precision copy of ``slot`` (what the optimizer refreshes after an update)."""
        local_shape = (slot.local_rows,) + slot.full_shape[1:] if slot.full_shape else ()
        if slot.unit >= 0:
            return self.lowp_shard[slot.master_offset : slot.master_offset + slot.local_numel].view(local_shape)
        if not slot.sharded:
            return self.lowp[slot.full_offset : slot.full_offset + slot.full_numel].view(slot.full_shape)
        flat = self._flat(self.lowp, slot)
        return flat[self.rank * slot.local_numel : (self.rank + 1) * slot.local_numel].view(local_shape)

    @torch.no_grad()
    def sync_lowp(self) -> None:
        """Refresh the low-precision copies from the fp32 master shards (cast + all-gather of the resident part)."""
        if self.lowp is None and self.lowp_shard is None:
            return
        for slot in self.slots:
            if slot.aware:
                self._own_rows_lowp(slot).copy_(slot.param.data)
        self.all_gather_lowp()
        self.finish_scatter()

    @torch.no_grad()
    def all_gather_lowp(self, only_unfused: bool = False) -> None:
        """
        All-gather every resident sharded parameter's bf16 rows into the full copy (in place). With ``only_unfused`` the
        parameters whose rows the fused optimizer kernel has already stored into all peers are left out. Streamed
        blocks are not touched: their full copies are assembled block by block during the next forward pass.
        """
        if not self.shard or self.lowp is None:
            return
        sharded = [s for s in self.slots
                   if s.aware and s.sharded and s.unit < 0 and not (only_unfused and self._fusable(s))]
        if not sharded:
            return
        backend_batch = getattr(dist, "_coalescing_manager", None)
        if backend_batch is not None and self.lowp.is_cuda:
            with dist._coalescing_manager(group=self.group, device=self.lowp.device, async_ops=False):
                for slot in sharded:
                    dist.all_gather_into_tensor(self._flat(self.lowp, slot), self._own_rows_lowp(slot).reshape(-1),
                                                group=self.group)
        else:
            for slot in sharded:
                dist.all_gather_into_tensor(self._flat(self.lowp, slot), self._own_rows_lowp(slot).reshape(-1).clone(),
                                            group=self.group)

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
        if self.streamed and self._materialized:
            self._flush_dirty_units()
            self._wait_comm()
            self.grad_shard.zero_()  # streamed blocks accumulate their reduced gradients here across micro-batches
            for g in self._ring_grad:
                g.zero_()

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
        if self.streamed and self._materialized:
            self._slot_unit = [-1, -1]  # the ring holds last step's weights
            if self._sym_shard_lowp is not None:
                self._sym_shard_lowp.barrier()  # every rank's updated rows are in place before anybody gathers them

    @torch.no_grad()
    def reduce_gradients(self) -> None:
        """
        Average gradients over the data-parallel group: reduce-scatter for sharded parameters (each rank
        receives its rows), all-reduce for replicated ones. Afterwards ``grad_view(slot)`` is valid.
        """
        if self.symmetric:
            self._reduce_gradients_fused()
            return
        if self.streamed:
            self._flush_dirty_units()
            self._wait_comm()
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
            if slot.unit >= 0:
                continue  # reduced into grad_shard right after the block's backward
            if slot.aware:
                full = self._flat(self.main_grad, slot)
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
                        out.copy_(full[self.rank * slot.local_numel: (self.rank + 1) * slot.local_numel]).div_(ws)
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
    # streamed blocks: per-block gather ahead of the compute, per-block gradient reduction behind it
    # ------------------------------------------------------------------------------------------------
    def _materialize_streamed(self, device: torch.device, lowp_dtype: torch.dtype, peer_ok: bool) -> None:
        from .symmetric import SymmetricBuffer, symmetric_memory_enabled

        self._ring_lowp = [torch.zeros(self._unit_numel, dtype=lowp_dtype, device=device) for _ in range(2)]
        self._sym_shard_lowp = self._sym_ring_grad = None
        if peer_ok and device.type == "cuda" and symmetric_memory_enabled(device, self.group):
            try:
                import ctypes

                self._sym_shard_lowp = SymmetricBuffer(self._master_numel, torch.bfloat16, device, self.group)
                self._sym_ring_grad = SymmetricBuffer(2 * self._unit_numel, torch.float32, device, self.group)
                base = [int(p) for p in self._sym_ring_grad.handle.buffer_ptrs]
                self._ring_grad_peers = [(ctypes.c_void_p * len(base))(*[b + k * self._unit_numel * 4 for b in base])
                                         for k in range(2)]
            except Exception as e:
                log.warning(f"Peer-mapped shards unavailable ({type(e).__name__}: {e}); streaming blocks with NCCL")
                self._sym_shard_lowp = self._sym_ring_grad = None
        if self._sym_ring_grad is not None:
            flat = self._sym_ring_grad.tensor
            self._ring_grad = [flat[: self._unit_numel], flat[self._unit_numel:]]
            self.lowp_shard = self._sym_shard_lowp.tensor
        else:
            self._ring_grad = [torch.zeros(self._unit_numel, dtype=self.reduce_dtype, device=device) for _ in range(2)]
            self.lowp_shard = torch.zeros(self._master_numel, dtype=lowp_dtype, device=device)
        # Saved-for-backward weight views would trip autograd's version check when their ring slot is refilled between
        # a block's forward and its backward (with the same values); `.data` aliases carry their own version counter.
        self._ring_lowp_raw = [t.data for t in self._ring_lowp]
        self._slot_unit = [-1, -1]  # which block's weights each ring slot holds (or is being filled with)
        self._slot_dirty = [-1, -1]  # which block's gradients sit unreduced in each gradient slot
        self._gather_done: List[Optional[torch.cuda.Event]] = [None, None]
        self._reduce_done: List[Optional[torch.cuda.Event]] = [None, None]
        self._comm_stream = torch.cuda.Stream(device) if device.type == "cuda" else None
        self._unit_segs = [
            torch.tensor([[s.master_offset, s.full_offset, s.local_numel] for s in unit], dtype=torch.int64, device=device)
            for unit in self.units]
        blocks = self.model.blocks
        for u, block in enumerate(blocks.values() if hasattr(blocks, "values") else blocks):
            block.register_forward_pre_hook(lambda m, args, u=u: self._pre_forward(u))
            block.register_full_backward_pre_hook(lambda m, grad_out, u=u: self._pre_backward(u))
            block.register_full_backward_hook(lambda m, grad_in, grad_out, u=u: self._post_backward(u))
        log.info(f"Sharded-parameter runtime streams {len(self.units)} blocks through a two-slot ring "
                 f"({'peer memory' if self._sym_ring_grad is not None else 'collectives'}): {self.memory_summary()}")

    def _wait_comm(self) -> None:
        if self._comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._comm_stream)

    def _pre_forward(self, u: int) -> None:
        self._ensure_unit(u)
        in_backward = torch._C._current_graph_task_id() != -1  # a checkpointed block recomputing its forward
        if not in_backward and u + 1 < len(self.units):
            self._ensure_unit(u + 1, wait=False)

    def _pre_backward(self, u: int) -> None:
        self._ensure_unit(u)
        k = u % 2
        if self._slot_dirty[k] not in (-1, u):
            self._reduce_unit(self._slot_dirty[k])  # its post-backward hook never fired (input without gradient)
        if self._reduce_done[k] is not None:
            torch.cuda.current_stream(self.device).wait_event(self._reduce_done[k])  # slot cleared by its last user
        self._slot_dirty[k] = u
        if u > 0:
            self._ensure_unit(u - 1, wait=False)

    def _post_backward(self, u: int) -> None:
        if self._slot_dirty[u % 2] == u:
            self._reduce_unit(u)

    def _flush_dirty_units(self) -> None:
        for k in range(2):
            if self._slot_dirty[k] >= 0:
                self._reduce_unit(self._slot_dirty[k])

    @torch.no_grad()
    def _ensure_unit(self, u: int, wait: bool = True) -> None:
        """Have block ``u``'s full weights in its ring slot: start the gather if needed, optionally wait for it."""
        k = u % 2
        if self._slot_unit[k] != u:
            self._gather_unit(u)
        if wait and self._gather_done[k] is not None:
            torch.cuda.current_stream(self.device).wait_event(self._gather_done[k])

    @torch.no_grad()
    def _gather_unit(self, u: int) -> None:
        k = u % 2
        dst = self._ring_lowp_raw[k]
        if self._comm_stream is None:  # CPU / gloo
            for s in self.units[u]:
                own = self.lowp_shard[s.master_offset : s.master_offset + s.local_numel]
                dist.all_gather_into_tensor(dst[s.full_offset : s.full_offset + s.flat_numel], own.clone(), group=self.group)
            self._slot_unit[k] = u
            return
        cur = torch.cuda.current_stream(self.device)
        self._comm_stream.wait_stream(cur)  # the slot's previous occupant is no longer read, the shards are up to date
        with torch.cuda.stream(self._comm_stream):
            if self._sym_shard_lowp is not None:
                from ..ops import _lib

                rc = _lib.lib().ocb_peer_gather_segments(self._sym_shard_lowp.peer_ptrs, self.world_size,
                                                         self._unit_segs[u].data_ptr(), len(self.units[u]), dst.data_ptr(),
                                                         self._comm_stream.cuda_stream)
                _lib.check(rc, "ocb_peer_gather_segments")
            else:
                with dist._coalescing_manager(group=self.group, device=self.device, async_ops=False):
                    for s in self.units[u]:
                        own = self.lowp_shard[s.master_offset : s.master_offset + s.local_numel]
                        dist.all_gather_into_tensor(dst[s.full_offset : s.full_offset + s.flat_numel], own, group=self.group)
            ev = torch.cuda.Event()
            ev.record(self._comm_stream)
        self._gather_done[k] = ev
        self._slot_unit[k] = u

    @torch.no_grad()
    def _reduce_unit(self, u: int) -> None:
        """Average block ``u``'s full-size gradients over the ranks into the owners' shards and clear its ring slot."""
        k = u % 2
        ws = self.world_size
        src = self._ring_grad[k]
        self._slot_dirty[k] = -1
        if self._comm_stream is None:  # CPU / gloo: no reduce-scatter, all-reduce and keep our rows
            for s in self.units[u]:
                full = src[s.full_offset : s.full_offset + s.flat_numel]
                dist.all_reduce(full, op=dist.ReduceOp.SUM, group=self.group)
                mine = full[self.rank * s.local_numel : (self.rank + 1) * s.local_numel]
                self.grad_shard[s.master_offset : s.master_offset + s.local_numel].add_(mine.to(torch.float32), alpha=1.0 / ws)
                full.zero_()
            return
        cur = torch.cuda.current_stream(self.device)
        self._comm_stream.wait_stream(cur)  # the block's backward has written all of its gradients
        with torch.cuda.stream(self._comm_stream):
            if self._sym_ring_grad is not None:
                from ..ops import _lib

                self._sym_ring_grad.barrier()  # every rank has finished this block's backward
                rc = _lib.lib().ocb_peer_pull_reduce_segments(self._ring_grad_peers[k], ws, self.rank,
                                                              self._unit_segs[u].data_ptr(), len(self.units[u]),
                                                              self.grad_shard.data_ptr(), 1.0 / ws,
                                                              self._comm_stream.cuda_stream)
                _lib.check(rc, "ocb_peer_pull_reduce_segments")
                self._sym_ring_grad.barrier()  # every rank has collected its rows: the slots may be cleared and reused
                src.zero_()
            else:
                for s in self.units[u]:
                    full = src[s.full_offset : s.full_offset + s.flat_numel]
                    out = self.grad_shard[s.master_offset : s.master_offset + s.local_numel]
                    if full.dtype == torch.float32:
                        tmp = torch.empty_like(out)
                        dist.reduce_scatter_tensor(tmp, full, op=dist.ReduceOp.AVG, group=self.group)
                        out.add_(tmp)
                    else:
                        tmp = torch.empty(s.local_numel, dtype=full.dtype, device=full.device)
                        dist.reduce_scatter_tensor(tmp, full, op=dist.ReduceOp.SUM, group=self.group)
                        out.add_(tmp.to(torch.float32), alpha=1.0 / ws)
                src[: self._unit_numel].zero_()
            ev = torch.cuda.Event()
            ev.record(self._comm_stream)
        self._reduce_done[k] = ev

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
        if self.streamed and self.lowp_shard is not None:
            parts.append(f"lowp_shard {self.lowp_shard.numel() * self.lowp_shard.element_size() / gb:.2f} GiB")
            ring = sum(t.numel() * t.element_size() for t in self._ring_lowp + self._ring_grad)
            parts.append(f"block ring {ring / gb:.2f} GiB ({len(self.units)} streamed blocks)")
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
        if slot.padded_rows != slot.full_shape[0]:
            # uneven split: present only the rows that exist, with the global shape spelled out
            shape = torch.Size(slot.full_shape)
            stride = torch.empty(shape, device="meta").stride()
            return DTensor.from_local(local[: slot.real_local_rows], self._ckpt_mesh, [Shard(0)], run_check=False,
                                      shape=shape, stride=stride)
        return DTensor.from_local(local, self._ckpt_mesh, [Shard(0)], run_check=False)
