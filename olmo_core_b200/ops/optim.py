"""
Optimizer-side kernels: the SkipStep-AdamW update over flat fp32 ranges and the sum of squares used for
the global gradient norm. Math is the reference's ``adamw_step`` (src/olmo_core/optim/adamw.py:12-47):
every term of the update is multiplied by a device-resident ``step_factor`` so that a skipped step costs
no host synchronisation.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib

__all__ = ["adamw_step_", "adamw_step_reference_", "sumsq", "cast_to_bf16_"]


def adamw_step_reference_(
    p: torch.Tensor,
    m: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    *,
    lr: float,
    betas,
    eps: float,
    weight_decay: float,
    step: torch.Tensor,
    step_factor: Optional[torch.Tensor] = None,
    grad_scale: Optional[torch.Tensor] = None,
    lowp: Optional[torch.Tensor] = None,
) -> None:
    """PyTorch restatement (CPU path and test oracle). ``step`` is the count *before* this update."""
    beta1, beta2 = betas
    f = step_factor if step_factor is not None else torch.ones((), device=p.device)
    g = g.to(torch.float32)
    if grad_scale is not None:
        g = g * grad_scale
    p.mul_(1 - f * (lr * weight_decay))
    m.lerp_(g.to(m.dtype), (f * (1 - beta1)).to(m.dtype))
    v.mul_(1 - f * (1 - beta2))
    v.add_(f * (1 - beta2) * g * g)
    t = step + 1
    bc1 = 1 - beta1**t
    bc2 = 1 - beta2**t
    denom = v.sqrt() / bc2.sqrt() + eps
    p.sub_(f * (lr / bc1) * m / denom)
    if lowp is not None:
        lowp.copy_(p)


def adamw_step_(
    p: torch.Tensor,
    m: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    *,
    lr: float,
    betas,
    eps: float,
    weight_decay: float,
    step: torch.Tensor,
    step_factor: Optional[torch.Tensor] = None,
    grad_scale: Optional[torch.Tensor] = None,
    lowp: Optional[torch.Tensor] = None,
) -> None:
    """
    In-place SkipStep-AdamW on contiguous fp32 ``p, m, v`` with gradient ``g`` (fp32 or bf16). ``step``,
    ``step_factor`` and ``grad_scale`` (the clipping coefficient) are fp32 scalar tensors on the same device
    so nothing synchronises. ``lowp`` optionally receives the bf16 copy of the updated parameters. The
    caller advances ``step`` by ``step_factor`` afterwards.
    """
    use_kernel = (
        p.is_cuda and p.dtype == torch.float32 and m.dtype == torch.float32 and v.dtype == torch.float32
        and p.is_contiguous() and m.is_contiguous() and v.is_contiguous() and g.is_contiguous()
        and g.dtype in (torch.float32, torch.bfloat16) and (lowp is None or (lowp.dtype == torch.bfloat16 and lowp.is_contiguous()))
        and p.data_ptr() % 16 == 0 and m.data_ptr() % 16 == 0 and v.data_ptr() % 16 == 0 and g.data_ptr() % 16 == 0
        and (lowp is None or lowp.data_ptr() % 8 == 0)
    )
    if not use_kernel:
        adamw_step_reference_(p, m, v, g, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, step=step,
                              step_factor=step_factor, grad_scale=grad_scale, lowp=lowp)
        return

    def scalar(t):
        if t is None:
            return None
        if t.dtype != torch.float32 or not t.is_cuda:
            t = t.to(device=p.device, dtype=torch.float32)
        return t

    step_t, sf_t, gs_t = scalar(step), scalar(step_factor), scalar(grad_scale)
    rc = _lib.lib().ocb_adamw_step(
        p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), _lib.ptr(lowp), p.numel(), float(lr), float(betas[0]),
        float(betas[1]), float(eps), float(weight_decay), _lib.ptr(step_t), _lib.ptr(sf_t), _lib.ptr(gs_t), _lib.dt(g),
        _lib.stream_ptr(),
    )
    _lib.check(rc, "ocb_adamw_step")


_scratch: dict = {}


def sumsq(x: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """``sum(x**2)`` as an fp32 scalar tensor (optionally accumulated into ``out``)."""
    if not x.is_cuda or x.dtype not in (torch.float32, torch.bfloat16) or not x.is_contiguous():
        s = x.float().pow(2).sum()
        if out is None:
            return s
        if accumulate:
            out.add_(s)
        else:
            out.copy_(s)
        return out
    if out is None:
        out = torch.zeros((), dtype=torch.float32, device=x.device)
        accumulate = False
    key = (x.device.index, torch.cuda.current_stream().cuda_stream)
    scratch = _scratch.get(key)
    if scratch is None:
        scratch = torch.empty(_lib.lib().ocb_sumsq_partials(), dtype=torch.float32, device=x.device)
        _scratch[key] = scratch
    rc = _lib.lib().ocb_sumsq(x.data_ptr(), x.numel(), scratch.data_ptr(), out.data_ptr(), 1 if accumulate else 0,
                             _lib.dt(x), _lib.stream_ptr())
    _lib.check(rc, "ocb_sumsq")
    return out


def cast_to_bf16_(src: torch.Tensor, dst: torch.Tensor) -> None:
    """``dst <- bf16(src)`` for flat fp32 ``src``."""
    if src.is_cuda and src.dtype == torch.float32 and dst.dtype == torch.bfloat16 and src.is_contiguous() and dst.is_contiguous():
        rc = _lib.lib().ocb_cast_f32_to_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), _lib.stream_ptr())
        _lib.check(rc, "ocb_cast_f32_to_bf16")
    else:
        dst.copy_(src)
