"""
Tensor-parallel linear layers whose collective runs INSIDE the GEMM kernel, over NVLink peer memory
(the all-gather → GEMM and GEMM → reduce-scatter pairs that the reference gets from DTensor redistributes around cuBLAS
calls: src/olmo_core/nn/feed_forward.py:172-204, src/olmo_core/nn/attention/__init__.py:690-760).

* :func:`gather_linear` — column-parallel projection of a sequence-sharded input: ``y = [x_0; ...; x_{tp-1}] @ W^T``.
  Every output tile loads its block of ``x`` directly from the rank that owns it (a plain TMA load from peer memory), so
  the gather never exists as a separate step and the NVLink transfer overlaps the tensor-core work tile by tile.
* :func:`linear_reduce_scatter` — row-parallel projection back to sequence shards: ``y_r = sum_ranks (x @ W^T)[rows of r]``.
  Every finished tile is added into the owner's fp32 shard with vector reductions over NVLink from the epilogue.

Both are autograd functions and each is the other's backward: the input gradient of ``gather_linear`` is a
GEMM → reduce-scatter, that of ``linear_reduce_scatter`` an all-gather → GEMM. Weight gradients need the gathered
operand as a whole, which is re-gathered with NCCL at that point (the forward never materialised it).

The peer-visible staging buffers are :class:`~olmo_core_b200.parallel.symmetric.SymmetricBuffer` s, cached per group and
size. Kernels on different ranks are ordered by the buffers' stream barrier: one before the kernel (every rank has
published its operand / zeroed its result) and one after it (every rank is done reading / adding). fp32 additions over
NVLink arrive in no fixed order, so the reduce-scatter is deterministic only up to fp32 rounding of a ``tp``-term sum.
On CPU tensors, and whenever peer memory is unavailable, the same functions fall back to ``torch.distributed``
collectives around a plain GEMM.
"""

from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import compute_weight, gemm
from .symmetric import SymmetricBuffer, symmetric_memory_enabled

__all__ = ["gather_linear", "gather_linear_multi", "linear_reduce_scatter", "fused_tp_available"]

ENV_VAR = "OLMO_CORE_B200_TP_FUSED"
_buffers: Dict[Tuple[int, str, int, torch.dtype], SymmetricBuffer] = {}


def fused_tp_available(x: torch.Tensor, group, rows_local: int) -> bool:
    """Peer memory is usable, the operand is bf16 on CUDA and the row shard is a whole number of 128-row tiles."""
    if os.environ.get(ENV_VAR, "1") == "0":
        return False
    if not x.is_cuda or x.dtype != torch.bfloat16 or rows_local % 128 != 0:
        return False
    return symmetric_memory_enabled(x.device, group) and dist.get_world_size(group) <= 8


def _buffer(group, tag: str, numel: int, dtype: torch.dtype, device: torch.device) -> SymmetricBuffer:
    key = (id(group), tag, numel, dtype)
    buf = _buffers.get(key)
    if buf is None:
        buf = SymmetricBuffer(numel, dtype, device, group)
        _buffers[key] = buf
    return buf


def _ptr_array(values) -> ctypes.Array:
    return (ctypes.c_void_p * len(values))(*[ctypes.c_void_p(int(v)) for v in values])


def _all_gather_rows(x: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty((x.shape[0] * dist.get_world_size(group), x.shape[1]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _reduce_scatter_rows(x: torch.Tensor, group) -> torch.Tensor:
    ws = dist.get_world_size(group)
    if x.is_cuda:
        out = torch.empty((x.shape[0] // ws, x.shape[1]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out
    full = x.contiguous()
    dist.all_reduce(full, group=group)
    return full.chunk(ws, dim=0)[dist.get_rank(group)].contiguous()


def _ag_gemm_multi(x_local: torch.Tensor, weights, trans_b: bool, group, tag: str):
    """
    ``[x_0; ...] @ op(w)`` for every ``w`` of ``weights`` with the gather inside the kernels: the shard is published once
    and every product pulls the peers' rows tile by tile. ``x_local [m, K]``; returns a list of ``[tp * m, N_i]`` bf16.
    """
    m, K = x_local.shape
    ws, rank = dist.get_world_size(group), dist.get_rank(group)
    stage = _buffer(group, f"ag-{tag}", m * K, torch.bfloat16, x_local.device)
    stage.tensor.view(m, K).copy_(x_local)
    stage.barrier()  # every rank's shard is in place
    outs = []
    for w in weights:
        N = w.shape[0] if trans_b else w.shape[1]
        out = torch.empty((ws * m, N), dtype=torch.bfloat16, device=x_local.device)
        rc = _lib.lib().ocb_gemm_bf16_tp(stage.peer_ptrs, w.data_ptr(), _ptr_array([out.data_ptr()]), m, N, K, K, w.stride(0),
                                         out.stride(0), ws, rank, 1, 0, 0 if trans_b else 1, _lib.EPI_BF16,
                                         _lib.status_buffer(x_local.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "ocb_gemm_bf16_tp")
        outs.append(out)
    stage.barrier()  # nobody still reads a shard when its owner reuses the staging buffer
    return outs


def _ag_gemm(x_local: torch.Tensor, w: torch.Tensor, trans_b: bool, group, tag: str) -> torch.Tensor:
    return _ag_gemm_multi(x_local, [w], trans_b, group, tag)[0]


def _gemm_rs_multi(xs, weights, trans_b: bool, group, tag: str) -> torch.Tensor:
    """
    Rows ``[r*m, (r+1)*m)`` of ``sum_i sum_ranks xs[i] @ op(weights[i])`` on rank ``r``: every product adds its tiles into
    the owners' fp32 shards from its epilogue, between one pair of barriers. ``xs[i] [tp * m, K_i]``; returns ``[m, N]``.
    """
    M = xs[0].shape[0]
    N = weights[0].shape[0] if trans_b else weights[0].shape[1]
    ws, rank = dist.get_world_size(group), dist.get_rank(group)
    m = M // ws
    acc = _buffer(group, f"rs-{tag}", m * N, torch.float32, xs[0].device)
    acc.tensor.zero_()
    acc.barrier()  # every shard is zero before the first partial product arrives
    for x, w in zip(xs, weights):
        rc = _lib.lib().ocb_gemm_bf16_tp(_ptr_array([x.data_ptr()]), w.data_ptr(), acc.peer_ptrs, m, N, x.shape[1], x.stride(0),
                                         w.stride(0), N, ws, rank, 0, 1, 0 if trans_b else 1, _lib.EPI_F32_RED_PEER,
                                         _lib.status_buffer(x.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "ocb_gemm_bf16_tp")
    acc.barrier()  # all partial products have landed
    return acc.tensor.view(m, N).to(torch.bfloat16)


def _gemm_rs(x: torch.Tensor, w: torch.Tensor, trans_b: bool, group, tag: str) -> torch.Tensor:
    return _gemm_rs_multi([x], [w], trans_b, group, tag)


class _GatherLinearMulti(torch.autograd.Function):
    """Several column-parallel projections of one sequence-sharded input (q / k / v; the two halves of a gated MLP)."""

    @staticmethod
    def forward(ctx, x_local, group, tag, *weights):  # type: ignore[override]
        ws_ = [compute_weight(w, torch.bfloat16) for w in weights]
        x2 = x_local.reshape(-1, x_local.shape[-1]).contiguous()
        ctx.fused = fused_tp_available(x2, group, x2.shape[0])
        if ctx.fused:
            ys = _ag_gemm_multi(x2, ws_, True, group, tag)
        else:
            x_full = _all_gather_rows(x2, group)
            ys = [gemm(x_full, w, trans_b=True) for w in ws_]
        ctx.save_for_backward(x2, *ws_)
        ctx.group, ctx.tag, ctx.weight_refs, ctx.x_shape = group, tag, weights, x_local.shape
        return tuple(ys)

    @staticmethod
    def backward(ctx, *dys):  # type: ignore[override]
        x2, *ws_ = ctx.saved_tensors
        group = ctx.group
        dys = [dy.reshape(-1, dy.shape[-1]).contiguous() for dy in dys]
        if ctx.fused:
            dx = _gemm_rs_multi(dys, ws_, False, group, ctx.tag)
        else:
            partial = gemm(dys[0], ws_[0], trans_b=False)
            for dy, w in zip(dys[1:], ws_[1:]):
                partial = partial + gemm(dy, w, trans_b=False)
            dx = _reduce_scatter_rows(partial, group)
        x_full = _all_gather_rows(x2, group)
        dws = []
        for dy, weight in zip(dys, ctx.weight_refs):
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                gemm(dy, x_full, trans_a=True, trans_b=False, out=main_grad, accumulate=True)
                dws.append(None)
            else:
                dws.append(gemm(dy, x_full, trans_a=True, trans_b=False, out_dtype=torch.float32).to(weight.dtype))
        return (dx.view(ctx.x_shape), None, None, *dws)


class _GatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, weight, group, tag):  # type: ignore[override]
        w = compute_weight(weight, torch.bfloat16)
        x2 = x_local.reshape(-1, x_local.shape[-1]).contiguous()
        ctx.fused = fused_tp_available(x2, group, x2.shape[0])
        y = _ag_gemm(x2, w, True, group, tag) if ctx.fused else gemm(_all_gather_rows(x2, group), w, trans_b=True)
        ctx.save_for_backward(x2, w)
        ctx.group, ctx.tag, ctx.weight_ref, ctx.x_shape = group, tag, weight, x_local.shape
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x2, w = ctx.saved_tensors
        weight, group = ctx.weight_ref, ctx.group
        dy = dy.reshape(-1, dy.shape[-1]).contiguous()
        # dx_local = reduce-scatter(dy @ W): the partial products leave through the epilogue
        dx = _gemm_rs(dy, w, False, group, ctx.tag) if ctx.fused else _reduce_scatter_rows(gemm(dy, w, trans_b=False), group)
        x_full = _all_gather_rows(x2, group)
        main_grad = getattr(weight, "main_grad", None)
        if main_grad is not None:
            gemm(dy, x_full, trans_a=True, trans_b=False, out=main_grad, accumulate=True)
            dw = None
        else:
            dw = gemm(dy, x_full, trans_a=True, trans_b=False, out_dtype=torch.float32).to(weight.dtype)
        return dx.view(ctx.x_shape), dw, None, None


class _LinearReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, group, tag):  # type: ignore[override]
        w = compute_weight(weight, torch.bfloat16)
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        ws = dist.get_world_size(group)
        ctx.fused = x2.shape[0] % ws == 0 and fused_tp_available(x2, group, x2.shape[0] // ws)
        y = _gemm_rs(x2, w, True, group, tag) if ctx.fused else _reduce_scatter_rows(gemm(x2, w, trans_b=True), group)
        ctx.save_for_backward(x2, w)
        ctx.group, ctx.tag, ctx.weight_ref, ctx.x_shape = group, tag, weight, x.shape
        return y

    @staticmethod
    def backward(ctx, dy_local):  # type: ignore[override]
        x2, w = ctx.saved_tensors
        weight, group = ctx.weight_ref, ctx.group
        dy_local = dy_local.reshape(-1, dy_local.shape[-1]).contiguous()
        # dx = all-gather(dy_local) @ W: the gather rides on the operand loads
        dx = _ag_gemm(dy_local, w, False, group, ctx.tag) if ctx.fused else gemm(_all_gather_rows(dy_local, group), w, trans_b=False)
        dy_full = _all_gather_rows(dy_local, group)
        main_grad = getattr(weight, "main_grad", None)
        if main_grad is not None:
            gemm(dy_full, x2, trans_a=True, trans_b=False, out=main_grad, accumulate=True)
            dw = None
        else:
            dw = gemm(dy_full, x2, trans_a=True, trans_b=False, out_dtype=torch.float32).to(weight.dtype)
        return dx.view(ctx.x_shape), dw, None, None


def gather_linear_multi(x_local: torch.Tensor, weights, group, tag: str = "x"):
    """
    :func:`gather_linear` for several weights that share the input: the shard is published once, and the input gradient is
    reduced once for all of them. Returns one ``[tp * m, N_i]`` tensor per weight.
    """
    return _GatherLinearMulti.apply(x_local, group, tag, *weights)


def gather_linear(x_local: torch.Tensor, weight: torch.Tensor, group, tag: str = "x") -> torch.Tensor:
    """
    ``x_local [.., m, K]`` is this rank's ROW shard (rows = flattened leading dimensions) of the full input;
    ``weight [N_local, K]`` its column-parallel slice. Returns ``[tp * m, N_local]`` (rank-major row order).
    ``tag`` keys the staging buffer: calls whose operands are alive at the same time need different tags.
    """
    return _GatherLinear.apply(x_local, weight, group, tag)


def linear_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, group, tag: str = "y") -> torch.Tensor:
    """
    ``x [.., tp * m, K_local]`` (rank-major rows) times this rank's row-parallel slice ``weight [N, K_local]``, summed
    over the group; returns this rank's rows ``[m, N]``.
    """
    return _LinearReduceScatter.apply(x, weight, group, tag)
