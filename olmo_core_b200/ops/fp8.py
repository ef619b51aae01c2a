"""
Scaled 8-bit floating-point linear layers on the tcgen05 tensor cores (the role torchao's ``Float8Linear`` plays for the
reference: src/olmo_core/float8/__init__.py:25-162, src/olmo_core/float8/ao.py:153-239).

All three products of a linear layer run as e4m3 x e4m3 GEMMs with fp32 accumulation (``csrc/gemm_sm100.cu``,
``kind::f8f6f4``). Every operand is quantised dynamically along its reduction dimension, one fp32 scale per row of the
K-major matrix the tensor cores read (``csrc/fp8_sm100.cu``); the product of the two scales is applied in the epilogue::

    forward   y  = q(x) q(W)^T                 x by row,         W by row (output channel)
    dgrad     dx = q(dy) q(W^T)^T              dy by row,        W by column (transposed copy)
    wgrad     dW = q(dy^T) q(x^T)^T            dy, x by column (transposed copies), fp32 accumulate into ``main_grad``

``recipe="rowwise_with_gw_hp"`` keeps the weight gradient in bf16. A "tensorwise" recipe is served by the same row-wise
kernels (finer scales, same cost). On CPU the functions emulate the quantisation in PyTorch: the numerical oracle.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .gemm import compute_weight, gemm

__all__ = ["quantize_rowwise", "quantize_colwise_transposed", "gemm_fp8", "fp8_linear", "Float8LinearFunction",
           "cached_weight_cast", "E4M3_MAX"]

E4M3_MAX = 448.0


def _scale(amax: torch.Tensor, pow2: bool) -> torch.Tensor:
    s = amax.float().clamp(min=1e-12) / E4M3_MAX
    return torch.exp2(torch.ceil(torch.log2(s))) if pow2 else s


def quantize_rowwise(x: torch.Tensor, pow2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [R, C]`` bf16 -> (``q [R, C]`` e4m3 bytes, ``scale [R]`` fp32) with ``x ~ q * scale[:, None]``."""
    R, C = x.shape
    if not x.is_cuda:
        s = _scale(x.abs().amax(dim=1), pow2)
        return (x.float() / s[:, None]).to(torch.float8_e4m3fn).view(torch.uint8), s
    x = x if x.stride(1) == 1 else x.contiguous()
    q = torch.empty((R, C), dtype=torch.uint8, device=x.device)
    s = torch.empty(R, dtype=torch.float32, device=x.device)
    rc = _lib.lib().ocb_quantize_e4m3_rowwise(x.data_ptr(), q.data_ptr(), s.data_ptr(), R, C, x.stride(0), q.stride(0),
                                              int(pow2), _lib.stream_ptr())
    _lib.check(rc, "ocb_quantize_e4m3_rowwise")
    return q, s


def quantize_colwise_transposed(x: torch.Tensor, pow2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [R, C]`` bf16 -> (``q_t [C, R]`` e4m3 bytes, ``scale [C]``) with ``x^T ~ q_t * scale[:, None]``."""
    R, C = x.shape
    if not x.is_cuda:
        s = _scale(x.abs().amax(dim=0), pow2)
        return (x.float().t() / s[:, None]).to(torch.float8_e4m3fn).contiguous().view(torch.uint8), s
    x = x if x.stride(1) == 1 else x.contiguous()
    ld = (R + 15) // 16 * 16  # the GEMM wants row strides that are multiples of 16 bytes
    q = torch.empty((C, ld), dtype=torch.uint8, device=x.device)[:, :R]
    s = torch.empty(C, dtype=torch.float32, device=x.device)
    scratch = torch.empty(C, dtype=torch.float32, device=x.device)
    rc = _lib.lib().ocb_quantize_e4m3_colwise_t(x.data_ptr(), q.data_ptr(), s.data_ptr(), scratch.data_ptr(), R, C,
                                                x.stride(0), q.stride(0), int(pow2), _lib.stream_ptr())
    _lib.check(rc, "ocb_quantize_e4m3_colwise_t")
    return q, s


def gemm_fp8(a_q: torch.Tensor, a_scale: torch.Tensor, b_q: torch.Tensor, b_scale: torch.Tensor, *,
             out: Optional[torch.Tensor] = None, accumulate: bool = False,
             out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``out (=|+=) (a_q @ b_q^T) * a_scale[:, None] * b_scale[None, :]``; ``a_q [M, K]``, ``b_q [N, K]`` e4m3 bytes."""
    M, K = a_q.shape
    N = b_q.shape[0]
    if b_q.shape[1] != K:
        raise ValueError("fp8 GEMM inner dimensions differ")
    if not a_q.is_cuda:
        res = (a_q.view(torch.float8_e4m3fn).float() @ b_q.view(torch.float8_e4m3fn).float().t()) \
            * a_scale[:, None] * b_scale[None, :]
        if out is None:
            return res.to(out_dtype)
        out.add_(res.to(out.dtype)) if accumulate else out.copy_(res.to(out.dtype))
        return out
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype, device=a_q.device)
    if out.dtype == torch.bfloat16 and not accumulate:
        epi = _lib.EPI_BF16
    elif out.dtype == torch.float32:
        epi = _lib.EPI_F32_ACC if accumulate else _lib.EPI_F32
    else:
        raise _lib.KernelError("the fp8 GEMM writes bf16, or fp32 (optionally accumulating)")
    rc = _lib.lib().ocb_gemm_fp8(a_q.data_ptr(), b_q.data_ptr(), out.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(),
                                 M, N, K, a_q.stride(0), b_q.stride(0), out.stride(0), epi,
                                 _lib.status_buffer(a_q.device).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "ocb_gemm_fp8")
    return out


def cached_weight_cast(cache: Optional[dict], key: str, make, version: int = 0):
    """
    ``make()`` once per optimizer step: ``cache`` is a dict owned by the layer and emptied by
    :func:`olmo_core_b200.float8.refresh_float8_scales` after every parameter update, so the quantised copies of a weight
    are shared by all micro-batches of a step and by forward and backward (the effect the reference gets from casting
    weights once before the sharded all-gather: src/olmo_core/float8/__init__.py:141-162). ``None`` disables caching.
    ``version`` (the parameter's autograd version counter) additionally drops an entry when the weight was rewritten by
    an ordinary in-place tensor operation, e.g. when a checkpoint is loaded.
    """
    if cache is None:
        return make()
    hit = cache.get(key)
    if hit is None or hit[0] != version:
        hit = cache[key] = (version, make())
    return hit[1]


class Float8LinearFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, pow2: bool, wgrad_high_precision: bool, cache: Optional[dict] = None):  # type: ignore[override]
        w = compute_weight(weight, torch.bfloat16)
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
        xq, sx = quantize_rowwise(x2, pow2)
        wq, sw = cached_weight_cast(cache, "row", lambda: quantize_rowwise(w, pow2), weight._version)
        y = gemm_fp8(xq, sx, wq, sw)
        ctx.save_for_backward(x2, w)
        ctx.opts = (pow2, wgrad_high_precision)
        ctx.cache = cache
        ctx.weight_ref, ctx.x_shape, ctx.x_dtype = weight, x.shape, x.dtype
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x2, w = ctx.saved_tensors
        pow2, wgrad_hp = ctx.opts
        weight = ctx.weight_ref
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = (dy2 if dy2.dtype == torch.bfloat16 else dy2.to(torch.bfloat16)).contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dyq, sdy = quantize_rowwise(dy2, pow2)
            wtq, swt = cached_weight_cast(ctx.cache, "col_t", lambda: quantize_colwise_transposed(w, pow2), weight._version)  # [K, N]
            dx = gemm_fp8(dyq, sdy, wtq, swt).view(ctx.x_shape).to(ctx.x_dtype)
        main_grad = getattr(weight, "main_grad", None)
        dw = None
        if main_grad is not None or ctx.needs_input_grad[1]:
            if wgrad_hp:
                if main_grad is not None:
                    gemm(dy2, x2, trans_a=True, trans_b=False, out=main_grad, accumulate=True)
                else:
                    dw = gemm(dy2, x2, trans_a=True, trans_b=False, out_dtype=torch.float32).to(weight.dtype)
            else:
                dytq, sdyt = quantize_colwise_transposed(dy2, pow2)  # [N, M]
                xtq, sxt = quantize_colwise_transposed(x2, pow2)  # [K, M]
                if main_grad is not None:
                    gemm_fp8(dytq, sdyt, xtq, sxt, out=main_grad, accumulate=True)
                else:
                    dw = gemm_fp8(dytq, sdyt, xtq, sxt, out_dtype=torch.float32).to(weight.dtype)
        return dx, dw, None, None, None


def fp8_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *, pow2_scales: bool = False,
               wgrad_high_precision: bool = False, weight_cache: Optional[dict] = None) -> torch.Tensor:
    """``x @ weight^T (+ bias)`` through the 8-bit kernels; dimensions must be multiples of 16."""
    y = Float8LinearFunction.apply(x, weight, pow2_scales, wgrad_high_precision, weight_cache)
    return y if bias is None else y + bias.to(y.dtype)
