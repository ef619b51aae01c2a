"""
Cross-entropy (+ z-loss) ops.

* :func:`cross_entropy_with_z_loss` -- the materialised-logits loss, numerically the reference's
  ``cross_entropy_loss`` (src/olmo_core/nn/functional/cross_entropy_loss.py:12-50): fp32 log-softmax,
  ``ignore_index`` masking, ``z = mult * logsumexp(logits)^2`` over non-ignored tokens.
* :func:`fused_linear_cross_entropy` -- the LM-head projection and the loss in one op that never holds the
  full ``[N, V]`` logits (the role Liger's kernel plays at src/olmo_core/nn/functional/cross_entropy_loss.py:67-124).
  Rows are processed in chunks: tcgen05 GEMM for the chunk's logits, one kernel that turns them into
  per-row losses and (in place) their gradient, then the dgrad / wgrad GEMMs. Like the reference's fused
  path, gradients are produced during the forward pass and only rescaled in backward.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import compute_weight, gemm

__all__ = ["cross_entropy_with_z_loss", "fused_linear_cross_entropy", "cross_entropy_rows"]


def cross_entropy_rows(
    logits: torch.Tensor,
    labels: torch.Tensor,
    *,
    ignore_index: int = -100,
    z_loss_multiplier: float = 0.0,
    grad_scale: Optional[torch.Tensor] = None,
    dlogits: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    Per-row CE and z-loss of ``logits`` ``[rows, V]`` (CUDA, bf16/fp32). When ``dlogits`` is given (it may
    alias ``logits``) the gradient ``grad_scale * d(ce + z)/dlogits`` is written to it.
    """
    rows, vocab = logits.shape
    ce = torch.empty(rows, dtype=torch.float32, device=logits.device)
    z = torch.empty(rows, dtype=torch.float32, device=logits.device)
    labels = labels.reshape(-1)
    if labels.dtype != torch.int64 or labels.device != logits.device:
        labels = labels.to(device=logits.device, dtype=torch.int64)  # the kernel reads them on the logits' device
    labels = labels.contiguous()
    rc = _lib.lib().ocb_cross_entropy_fwd_bwd(
        logits.data_ptr(), labels.data_ptr(), ce.data_ptr(), z.data_ptr(), _lib.ptr(dlogits), rows, vocab,
        logits.stride(0), dlogits.stride(0) if dlogits is not None else 0, ignore_index, float(z_loss_multiplier),
        _lib.ptr(grad_scale), _lib.dt(logits), _lib.stream_ptr(),
    )
    _lib.check(rc, "ocb_cross_entropy_fwd_bwd")
    return ce, z


class _CrossEntropyFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index: int, z_mult: float):  # type: ignore[override]
        l2 = logits.reshape(-1, logits.shape[-1])
        if l2.stride(1) != 1:
            l2 = l2.contiguous()
        dl = torch.empty_like(l2)
        ce, z = cross_entropy_rows(l2, labels, ignore_index=ignore_index, z_loss_multiplier=z_mult, dlogits=dl)
        ctx.save_for_backward(dl)
        ctx.shape = logits.shape
        return ce.sum(), z.sum()

    @staticmethod
    def backward(ctx, g_ce, g_z):  # type: ignore[override]
        (dl,) = ctx.saved_tensors
        # d(ce)/dlogits and d(z)/dlogits are stored summed; both outputs are consumed as ce + z.
        g = g_ce if g_ce is not None else g_z
        return (dl * g.to(dl.dtype)).view(ctx.shape), None, None, None


def cross_entropy_with_z_loss(
    logits: torch.Tensor,
    labels: torch.Tensor,
    *,
    ignore_index: int = -100,
    reduction: str = "mean",
    compute_z_loss: bool = False,
    z_loss_multiplier: float = 1e-4,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """
    Returns ``(ce_loss, z_loss or None)`` for ``logits`` ``[..., V]`` and ``labels`` ``[...]``.
    ``reduction``: ``"sum"``, ``"mean"`` (over non-ignored tokens) or ``"none"``.
    """
    labels_flat = labels.reshape(-1)
    if (logits.is_cuda and reduction in ("sum", "mean") and logits.dtype in (torch.bfloat16, torch.float32)
            and logits.shape[-1] % 8 == 0):
        ce, z = _CrossEntropyFunction.apply(logits, labels_flat, ignore_index, z_loss_multiplier if compute_z_loss else 0.0)
        if reduction == "mean":
            denom = (labels_flat != ignore_index).sum().clamp(min=1).to(ce.dtype)
            ce = ce / denom
            z = z / denom
        return ce, (z if compute_z_loss else None)

    lf = logits.float().reshape(-1, logits.shape[-1])
    loss = F.cross_entropy(lf, labels_flat, ignore_index=ignore_index, reduction=reduction)
    if reduction == "none":
        loss = loss.view(labels.shape)
    if not compute_z_loss:
        return loss, None
    mask = (labels_flat != ignore_index).to(lf.dtype)
    zsq = torch.logsumexp(lf, dim=-1).pow(2)
    if reduction == "mean":
        z = z_loss_multiplier * (zsq * mask).sum() / mask.sum().clamp(min=1)
    elif reduction == "sum":
        z = z_loss_multiplier * (zsq * mask).sum()
    else:
        # per-token values are returned for EVERY position, ignored ones included, as the reference does
        # (src/olmo_core/nn/functional/cross_entropy_loss.py:41-50): whoever reduces them applies the mask
        z = (z_loss_multiplier * zsq).view(labels.shape)
    return loss, z


class _FusedLinearCEFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, weight, labels, scale, ignore_index: int, z_mult: float, chunk_rows: int):  # type: ignore[override]
        w = compute_weight(weight, torch.bfloat16)
        h2 = h.reshape(-1, h.shape[-1])
        if h2.dtype != torch.bfloat16:
            h2 = h2.to(torch.bfloat16)
        if h2.stride(1) != 1:
            h2 = h2.contiguous()
        labels = labels.reshape(-1)
        rows, d = h2.shape
        V = w.shape[0]
        need_dh = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        main_grad = getattr(weight, "main_grad", None) if need_dw else None
        dw = None
        if need_dw and main_grad is None:
            dw = torch.zeros((V, d), dtype=torch.float32, device=h.device)
        dh = torch.empty_like(h2) if need_dh else None
        ce_sum = torch.zeros((), dtype=torch.float32, device=h.device)
        z_sum = torch.zeros((), dtype=torch.float32, device=h.device)
        logits = torch.empty((min(chunk_rows, rows), V), dtype=torch.bfloat16, device=h.device)
        compute_grad = need_dh or need_dw
        for r0 in range(0, rows, chunk_rows):
            r1 = min(rows, r0 + chunk_rows)
            lg = logits[: r1 - r0]
            gemm(h2[r0:r1], w, trans_b=True, out=lg)
            ce, z = cross_entropy_rows(lg, labels[r0:r1], ignore_index=ignore_index, z_loss_multiplier=z_mult,
                                       grad_scale=scale, dlogits=lg if compute_grad else None)
            ce_sum += ce.sum()
            z_sum += z.sum()
            if need_dh:
                gemm(lg, w, trans_b=False, out=dh[r0:r1])
            if need_dw:
                gemm(lg, h2[r0:r1], trans_a=True, trans_b=False, out=main_grad if main_grad is not None else dw,
                     accumulate=True)
        ctx.save_for_backward(dh if dh is not None else torch.empty(0, device=h.device),
                              dw if dw is not None else torch.empty(0, device=h.device))
        ctx.h_shape = h.shape
        ctx.h_dtype = h.dtype
        ctx.w_dtype = weight.dtype
        ctx.fused_main_grad = main_grad is not None
        ctx.has = (need_dh, need_dw)
        return ce_sum * scale, z_sum * scale

    @staticmethod
    def backward(ctx, g_ce, g_z):  # type: ignore[override]
        dh, dw = ctx.saved_tensors
        need_dh, need_dw = ctx.has
        g = g_ce if g_ce is not None else g_z
        gh = None
        gw = None
        if need_dh:
            gh = (dh * g.to(dh.dtype)).view(ctx.h_shape).to(ctx.h_dtype)
        if need_dw and not ctx.fused_main_grad:
            gw = (dw * g).to(ctx.w_dtype)
        # With a main_grad buffer the weight gradient was accumulated during forward, which is only
        # correct for an upstream gradient of one (the train module calls backward on the loss itself).
        return gh, gw, None, None, None, None, None


def fused_linear_cross_entropy(
    h: torch.Tensor,
    weight: torch.Tensor,
    labels: torch.Tensor,
    *,
    ignore_index: int = -100,
    z_loss_multiplier: Optional[float] = None,
    scale: Optional[torch.Tensor] = None,
    chunk_rows: int = 4096,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """
    ``(scale * sum CE, scale * sum z-loss or None)`` of ``h @ weight.T`` against ``labels`` without
    materialising the logits. ``scale`` is a scalar tensor (e.g. ``1 / loss_div_factor``); default 1.
    """
    z_mult = float(z_loss_multiplier) if z_loss_multiplier is not None else 0.0
    if h.is_cuda:
        if scale is None:
            scale = torch.ones((), dtype=torch.float32, device=h.device)
        elif not torch.is_tensor(scale):
            scale = torch.tensor(float(scale), dtype=torch.float32, device=h.device)
        else:
            scale = scale.to(device=h.device, dtype=torch.float32).reshape(())
        ce, z = _FusedLinearCEFunction.apply(h, weight, labels, scale, ignore_index, z_mult, int(chunk_rows))
        return ce, (z if z_loss_multiplier is not None else None)
    from .param import full_param

    logits = F.linear(h, full_param(weight, h.dtype))
    ce, z = cross_entropy_with_z_loss(logits, labels, ignore_index=ignore_index, reduction="sum",
                                      compute_z_loss=z_loss_multiplier is not None,
                                      z_loss_multiplier=z_mult)
    if scale is not None:
        ce = ce * scale
        z = z * scale if z is not None else None
    return ce, z
