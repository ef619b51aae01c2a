"""
Autograd ops for the memory-bound kernels in ``csrc/elementwise.cu``: RMSNorm (with the residual add
of the reordered-norm block fused in), fused QK-norm + rotary embedding, SwiGLU and the embedding
lookup. Every op has a PyTorch reference path, used on CPU and as the oracle in the GPU tests, that
restates the reference formulas (src/olmo_core/nn/layer_norm.py:215-236, src/olmo_core/nn/rope.py:470-578,
src/olmo_core/nn/feed_forward.py:165-171).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib

__all__ = [
    "rms_norm",
    "rms_norm_reference",
    "norm_rope",
    "norm_rope_reference",
    "swiglu",
    "swiglu_reference",
    "embedding",
]


def _partials(device: torch.device, cols: int) -> torch.Tensor:
    n = _lib.lib().ocb_norm_bwd_partials()
    return torch.empty((n, cols), dtype=torch.float32, device=device)


def _as_rows(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    return x2


def _ld(t: torch.Tensor) -> int:
    return t.stride(0) if t.size(0) > 1 else max(t.stride(0), t.size(1))


def _accumulate_param_grad(weight: torch.Tensor, partial: torch.Tensor, n_partial: int) -> Optional[torch.Tensor]:
    """Reduce per-block partials into ``weight.main_grad`` (returns None) or into a fresh gradient."""
    cols = partial.shape[1]
    main_grad = getattr(weight, "main_grad", None)
    if main_grad is not None:
        rc = _lib.lib().ocb_reduce_partials(partial.data_ptr(), main_grad.data_ptr(), n_partial, cols, 1,
                                           _lib.dt(main_grad), _lib.stream_ptr())
        _lib.check(rc, "ocb_reduce_partials")
        return None
    dw = torch.empty(cols, dtype=torch.float32, device=partial.device)
    rc = _lib.lib().ocb_reduce_partials(partial.data_ptr(), dw.data_ptr(), n_partial, cols, 0, _lib.DT_F32,
                                       _lib.stream_ptr())
    _lib.check(rc, "ocb_reduce_partials")
    return dw.to(weight.dtype).view_as(weight)


def _lowp_or_self(weight: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if weight is None:
        return None
    lowp = getattr(weight, "_lowp", None)
    return lowp if lowp is not None else weight


# ------------------------------------------------------------------------------------------------------
# RMSNorm
# ------------------------------------------------------------------------------------------------------


def rms_norm_reference(
    x: torch.Tensor,
    weight: Optional[torch.Tensor],
    eps: float,
    residual: Optional[torch.Tensor] = None,
    group: Optional[int] = None,
) -> torch.Tensor:
    """fp32 statistics, weight multiply in fp32, cast back to the input dtype, then the residual add."""
    og = x.dtype
    xf = x.float()
    if group is not None and group != x.shape[-1]:
        xf = xf.view(*x.shape[:-1], -1, group)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    y = y.view(x.shape).to(og)
    if residual is not None:
        y = residual + y
    return y


class _RMSNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual, eps: float, group: int):  # type: ignore[override]
        x2 = _as_rows(x)
        rows, cols = x2.shape
        w = _lowp_or_self(weight)
        r2 = _as_rows(residual) if residual is not None else None
        y = torch.empty((rows, cols), dtype=x2.dtype, device=x2.device)
        rstd = torch.empty(rows * (cols // group), dtype=torch.float32, device=x2.device)
        rc = _lib.lib().ocb_rmsnorm_fwd(
            x2.data_ptr(), _lib.ptr(w), _lib.ptr(r2), y.data_ptr(), rstd.data_ptr(), rows, cols, group,
            _ld(x2), _ld(y), _ld(r2) if r2 is not None else 0, eps, _lib.dt(x2),
            _lib.dt(w) if w is not None else _lib.DT_F32, _lib.stream_ptr(),
        )
        _lib.check(rc, "ocb_rmsnorm_fwd")
        ctx.save_for_backward(x2, w if w is not None else torch.empty(0, device=x2.device), rstd)
        ctx.weight_ref = weight
        ctx.has_weight = weight is not None
        ctx.has_residual = residual is not None
        ctx.group = group
        ctx.x_shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x2, w, rstd = ctx.saved_tensors
        rows, cols = x2.shape
        dy2 = _as_rows(dy)
        if dy2.dtype != x2.dtype:
            dy2 = dy2.to(x2.dtype)
        dx = torch.empty_like(x2)
        need_dw = ctx.has_weight and ctx.needs_input_grad[1]
        partial = _partials(x2.device, ctx.group) if need_dw else None
        rc = _lib.lib().ocb_rmsnorm_bwd(
            dy2.data_ptr(), x2.data_ptr(), w.data_ptr() if ctx.has_weight else None, rstd.data_ptr(), dx.data_ptr(),
            _lib.ptr(partial), rows, cols, ctx.group, _ld(dy2), _ld(x2), _ld(dx), _lib.dt(x2),
            _lib.dt(w) if ctx.has_weight else _lib.DT_F32, _lib.stream_ptr(),
        )
        _lib.check(rc, "ocb_rmsnorm_bwd")
        dw = None
        if need_dw:
            dw = _accumulate_param_grad(ctx.weight_ref, partial, partial.shape[0])
        dres = dy if ctx.has_residual else None
        return dx.view(ctx.x_shape), dw, dres, None, None


def rms_norm(
    x: torch.Tensor,
    weight: Optional[torch.Tensor],
    eps: float = 1e-6,
    residual: Optional[torch.Tensor] = None,
    group: Optional[int] = None,
) -> torch.Tensor:
    """
    ``residual + rmsnorm(x) * weight``. ``group`` is the width of one normalisation group (defaults to the
    last dimension; pass ``head_dim`` for a per-head norm over a ``[..., n_heads*head_dim]`` tensor).
    """
    group = group or x.shape[-1]
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and group % 8 == 0 and group <= 32768:
        return _RMSNormFunction.apply(x, weight, residual, float(eps), int(group))
    from .param import full_param

    return rms_norm_reference(x, full_param(weight), eps, residual, group)


# ------------------------------------------------------------------------------------------------------
# Fused QK-norm + RoPE
# ------------------------------------------------------------------------------------------------------

NORM_NONE, NORM_FULL, NORM_HEAD = 0, 1, 2


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def norm_rope_reference(
    x: torch.Tensor,
    weight: Optional[torch.Tensor],
    sin: torch.Tensor,
    cos: torch.Tensor,
    n_heads: int,
    eps: float,
    norm_mode: int,
    pos_ids: Optional[torch.Tensor] = None,
    pos_offset: int = 0,
) -> torch.Tensor:
    """``x``: [B, S, n_heads*head_dim]. Norm (full row or per head) -> cast -> fp32 rotate-half RoPE -> cast."""
    B, S, D = x.shape
    hd = D // n_heads
    y = x
    if norm_mode == NORM_FULL:
        y = rms_norm_reference(x, weight, eps)
    elif norm_mode == NORM_HEAD:
        y = rms_norm_reference(x, weight, eps, group=hd)
    if pos_ids is None:
        s = sin[pos_offset : pos_offset + S][None, :, None, :]
        c = cos[pos_offset : pos_offset + S][None, :, None, :]
    else:
        idx = pos_ids.view(B, S).long()
        s = sin[idx][:, :, None, :]
        c = cos[idx][:, :, None, :]
    yf = y.view(B, S, n_heads, hd).float()
    out = yf * c + _rotate_half(yf) * s
    return out.to(x.dtype).view(B, S, D)


class _NormRopeFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, sin, cos, n_heads: int, eps: float, norm_mode: int, pos_ids, pos_offset: int):  # type: ignore[override]
        B, S, D = x.shape
        hd = D // n_heads
        x2 = x.reshape(B * S, D)
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        w = _lowp_or_self(weight) if norm_mode != NORM_NONE else None
        y = torch.empty((B * S, D), dtype=x.dtype, device=x.device)
        n_stats = 0 if norm_mode == NORM_NONE else (B * S if norm_mode == NORM_FULL else B * S * n_heads)
        rstd = torch.empty(max(n_stats, 1), dtype=torch.float32, device=x.device)
        pos = None if pos_ids is None else pos_ids.reshape(-1).to(torch.int32).contiguous()
        rc = _lib.lib().ocb_norm_rope_fwd(
            x2.data_ptr(), _lib.ptr(w), y.data_ptr(), rstd.data_ptr(), sin.data_ptr(), cos.data_ptr(), _lib.ptr(pos),
            B * S, n_heads, hd, S, pos_offset, norm_mode, _ld(x2), _ld(y), eps, _lib.dt(x2),
            _lib.dt(w) if w is not None else _lib.DT_F32, _lib.stream_ptr(),
        )
        _lib.check(rc, "ocb_norm_rope_fwd")
        empty = torch.empty(0, device=x.device)
        ctx.save_for_backward(x2 if norm_mode != NORM_NONE else empty, w if w is not None else empty, rstd, sin, cos,
                              pos if pos is not None else empty)
        ctx.weight_ref = weight
        ctx.cfg = (B, S, D, n_heads, hd, norm_mode, pos_offset, pos is not None, x.dtype)
        return y.view(B, S, D)

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x2, w, rstd, sin, cos, pos = ctx.saved_tensors
        B, S, D, n_heads, hd, norm_mode, pos_offset, has_pos, x_dtype = ctx.cfg
        dy2 = dy.reshape(B * S, D)
        if dy2.stride(1) != 1:
            dy2 = dy2.contiguous()
        if dy2.dtype != x_dtype:
            dy2 = dy2.to(x_dtype)
        dx = torch.empty((B * S, D), dtype=x_dtype, device=dy.device)
        need_dw = norm_mode != NORM_NONE and ctx.needs_input_grad[1]
        wcols = D if norm_mode == NORM_FULL else hd
        partial = _partials(dy.device, wcols) if need_dw else None
        rc = _lib.lib().ocb_norm_rope_bwd(
            dy2.data_ptr(), x2.data_ptr() if norm_mode != NORM_NONE else None,
            w.data_ptr() if norm_mode != NORM_NONE else None, rstd.data_ptr(), dx.data_ptr(), _lib.ptr(partial),
            sin.data_ptr(), cos.data_ptr(), pos.data_ptr() if has_pos else None, B * S, n_heads, hd, S, pos_offset,
            norm_mode, _ld(dy2), _ld(x2) if norm_mode != NORM_NONE else 0, _ld(dx), _lib.dt(dy2),
            _lib.dt(w) if norm_mode != NORM_NONE else _lib.DT_F32, _lib.stream_ptr(),
        )
        _lib.check(rc, "ocb_norm_rope_bwd")
        dw = _accumulate_param_grad(ctx.weight_ref, partial, partial.shape[0]) if need_dw else None
        return dx.view(B, S, D), dw, None, None, None, None, None, None, None


def norm_rope(
    x: torch.Tensor,
    weight: Optional[torch.Tensor],
    sin: torch.Tensor,
    cos: torch.Tensor,
    n_heads: int,
    eps: float = 1e-6,
    norm_mode: int = NORM_FULL,
    pos_ids: Optional[torch.Tensor] = None,
    pos_offset: int = 0,
) -> torch.Tensor:
    """
    Optional RMSNorm (full-width as in OLMo-2, or per head) followed by rotate-half RoPE, in one pass.
    ``x`` is ``[B, S, n_heads*head_dim]``; ``sin``/``cos`` are fp32 ``[max_pos, head_dim]`` tables.
    """
    hd = x.shape[-1] // n_heads
    half = hd // 2
    pvh = half // 8 if half % 8 == 0 else 0
    ok = (
        x.is_cuda
        and x.dtype in (torch.bfloat16, torch.float32)
        and sin.is_cuda
        and sin.dtype == torch.float32
        and sin.shape[-1] == hd
        and pvh > 0
        and (pvh & (pvh - 1)) == 0
        and pvh <= 32
        and n_heads * pvh <= 512
    )
    if ok:
        return _NormRopeFunction.apply(x, weight, sin.contiguous(), cos.contiguous(), n_heads, float(eps),
                                       int(norm_mode), pos_ids, int(pos_offset))
    from .param import full_param

    return norm_rope_reference(x, full_param(weight), sin, cos, n_heads, eps, norm_mode, pos_ids, pos_offset)


# ------------------------------------------------------------------------------------------------------
# SwiGLU
# ------------------------------------------------------------------------------------------------------


def swiglu_reference(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return F.silu(a) * b


class _SwiGLUFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):  # type: ignore[override]
        a2, b2 = _as_rows(a), _as_rows(b)
        rows, cols = a2.shape
        out = torch.empty((rows, cols), dtype=a2.dtype, device=a2.device)
        rc = _lib.lib().ocb_swiglu_fwd(a2.data_ptr(), b2.data_ptr(), out.data_ptr(), rows, cols, _ld(a2), _ld(b2),
                                      _ld(out), _lib.dt(a2), _lib.stream_ptr())
        _lib.check(rc, "ocb_swiglu_fwd")
        ctx.save_for_backward(a2, b2)
        ctx.shape = a.shape
        return out.view(a.shape)

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        a2, b2 = ctx.saved_tensors
        rows, cols = a2.shape
        d2 = _as_rows(dout)
        if d2.dtype != a2.dtype:
            d2 = d2.to(a2.dtype)
        da = torch.empty((rows, cols), dtype=a2.dtype, device=a2.device)
        db = torch.empty((rows, cols), dtype=a2.dtype, device=a2.device)
        rc = _lib.lib().ocb_swiglu_bwd(d2.data_ptr(), a2.data_ptr(), b2.data_ptr(), da.data_ptr(), db.data_ptr(), rows,
                                      cols, _ld(d2), _ld(a2), _ld(b2), _ld(da), _ld(db), _lib.dt(a2), _lib.stream_ptr())
        _lib.check(rc, "ocb_swiglu_bwd")
        return da.view(ctx.shape), db.view(ctx.shape)


def swiglu(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``silu(a) * b`` (the gate of the SwiGLU MLP)."""
    if a.is_cuda and a.dtype in (torch.bfloat16, torch.float32) and a.dtype == b.dtype and a.shape[-1] % 8 == 0:
        return _SwiGLUFunction.apply(a, b)
    return swiglu_reference(a, b)


# ------------------------------------------------------------------------------------------------------
# Embedding
# ------------------------------------------------------------------------------------------------------


class _EmbeddingFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, out_dtype):  # type: ignore[override]
        table = _lowp_or_self(weight)
        if table.dtype != out_dtype:
            table = table.to(out_dtype)
        if ids.device != table.device or ids.dtype != torch.int64:
            # the kernel dereferences both pointers on the table's device: token ids left on the host (or 32-bit ones)
            # would be read as garbage addresses
            ids = ids.to(device=table.device, dtype=torch.int64)
        flat = ids.reshape(-1).contiguous()
        rows, dim = flat.numel(), table.shape[1]
        out = torch.empty((rows, dim), dtype=out_dtype, device=table.device)
        rc = _lib.lib().ocb_embedding_fwd(flat.data_ptr(), table.data_ptr(), out.data_ptr(), rows, dim, table.shape[0],
                                         _lib.dt(out), _lib.stream_ptr())
        _lib.check(rc, "ocb_embedding_fwd")
        ctx.save_for_backward(flat)
        ctx.weight_ref = weight
        return out.view(*ids.shape, dim)

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        (flat,) = ctx.saved_tensors
        weight = ctx.weight_ref
        d2 = _as_rows(dout)
        if d2.dtype not in (torch.bfloat16, torch.float32):
            d2 = d2.float()
        main_grad = getattr(weight, "main_grad", None)
        target = main_grad if main_grad is not None and main_grad.dtype == torch.float32 else torch.zeros(
            weight.shape, dtype=torch.float32, device=weight.device)
        rc = _lib.lib().ocb_embedding_bwd(flat.data_ptr(), d2.data_ptr(), target.data_ptr(), flat.numel(), weight.shape[1],
                                         weight.shape[0], _lib.dt(d2), _lib.stream_ptr())
        _lib.check(rc, "ocb_embedding_bwd")
        if target is main_grad:
            return None, None, None
        return None, target.to(weight.dtype), None


def embedding(ids: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Row gather ``weight[ids]`` with a scatter-add backward into an fp32 gradient."""
    out_dtype = out_dtype or (getattr(weight, "_lowp", weight)).dtype
    if weight.is_cuda and out_dtype in (torch.bfloat16, torch.float32) and weight.shape[1] % 8 == 0:
        return _EmbeddingFunction.apply(ids, weight, out_dtype)
    from .param import full_param

    return F.embedding(ids, full_param(weight)).to(out_dtype)
