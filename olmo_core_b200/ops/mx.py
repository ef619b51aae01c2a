"""
Micro-scaling (MX) fp8 linear layers: e4m3 elements with one E8M0 power-of-two scale per 32 elements of the reduction
dimension, multiplied by ``tcgen05.mma.kind::mxf8f6f4.block_scale`` (``csrc/gemm_mx_sm100.cu``), quantised by
``csrc/mx_quant_sm100.cu``. This is the role of torchao's ``MXLinear`` in the reference
(src/olmo_core/float8/ao.py:190-239, enabled through src/olmo_core/float8/__init__.py:118-130).

Each of the three products of a linear layer quantises its operands along that product's own reduction dimension::

    forward   y  = q_K(x)  q_K(W)^T          x [M, K] and W [N, K] by rows
    dgrad     dx = q_N(dy) q_N(W^T)^T        dy [M, N] by rows, W by columns (transposed copy [K, N])
    wgrad     dW = q_M(dy^T) q_M(x^T)^T      dy and x by columns (transposed copies), fp32, optionally into ``main_grad``

The scales travel in the tensor core's own layout (512-byte blocks of 128 rows x 4 scales); :func:`scales_as_matrix`
unpacks them for inspection. On CPU the functions emulate the same arithmetic in PyTorch: the numerical oracle.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .fp8 import cached_weight_cast
from .gemm import compute_weight

__all__ = ["MX_BLOCK", "quantize_mx_rowwise", "quantize_mx_colwise_transposed", "scales_as_matrix", "scales_from_matrix",
           "dequantize_mx", "gemm_mx", "mx_linear", "MXLinearFunction", "mx_supported"]

MX_BLOCK = 32
_MODES = {"rceil": 0, "floor": 1, "ceil": 2, "even": 3}

_lib_sigs_done = False


def _lib_mx():
    global _lib_sigs_done
    lib = _lib.lib()
    if not _lib_sigs_done:
        from ctypes import c_int, c_longlong, c_void_p

        _lib.register_signature("ocb_quantize_mx_rowwise", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong,
                                                            c_int, c_void_p])
        _lib.register_signature("ocb_quantize_mx_colwise_t", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong,
                                                              c_longlong, c_int, c_void_p])
        _lib.register_signature("ocb_gemm_mx", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                c_longlong, c_longlong, c_longlong, c_int, c_void_p, c_void_p])
        _lib_sigs_done = True
    return lib


def mx_supported(rows: int, in_features: int, out_features: int) -> bool:
    """All three products need their reduction dimension to be a multiple of 128 and 16-byte row pitches."""
    return rows % 128 == 0 and in_features % 128 == 0 and out_features % 128 == 0


def _scale_index(rows: int, k: int, device) -> torch.Tensor:
    """Byte offset of the scale of (row, block) in the packed layout, as an int64 [rows, k // 32] tensor."""
    r = torch.arange(rows, device=device)[:, None]
    b = torch.arange(k // MX_BLOCK, device=device)[None, :]
    k_atoms = k // 128
    return ((r >> 7) * k_atoms + (b >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (b & 3)


def _scale_bytes(rows: int, k: int) -> int:
    return (rows + 127) // 128 * (k // 128) * 512


def scales_as_matrix(sf: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """Packed scale bytes -> ``[rows, k // 32]`` uint8 matrix of biased exponents."""
    return sf[_scale_index(rows, k, sf.device)]


def scales_from_matrix(e: torch.Tensor, k: int) -> torch.Tensor:
    """``[rows, k // 32]`` uint8 exponents -> packed scale bytes (padding rows hold exponent 127 = 1.0)."""
    rows = e.shape[0]
    sf = torch.full((_scale_bytes(rows, k),), 127, dtype=torch.uint8, device=e.device)
    sf[_scale_index(rows, k, e.device)] = e
    return sf


def _exponents(amax: torch.Tensor, mode: str) -> torch.Tensor:
    """Biased E8M0 exponent of the scale for a block maximum (same bit arithmetic as the kernel)."""
    if mode == "rceil":
        bits = (amax.float() / 448.0).view(torch.int32)
        e = (bits >> 23) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    else:
        bits = amax.float().view(torch.int32)
        if mode == "even":
            bits = bits + (1 << 19)
        ea = bits >> 23
        if mode == "ceil":
            ea = ea + ((bits & 0x7FFFFF) != 0).to(torch.int32)
        e = (ea - 8).clamp(min=0)
    return e.clamp(max=253)


def _emulate_quantize(x: torch.Tensor, mode: str) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [R, K] -> (e4m3 bytes [R, K], exponents [R, K // 32]), blocks along the last dimension."""
    R, K = x.shape
    xb = x.float().view(R, K // MX_BLOCK, MX_BLOCK)
    e = _exponents(xb.abs().amax(dim=-1), mode)
    inv = ((254 - e) << 23).view(torch.float32)
    q = (xb * inv[..., None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8).view(R, K)
    return q, e.to(torch.uint8)


def quantize_mx_rowwise(x: torch.Tensor, mode: str = "rceil") -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [R, K]`` bf16 -> (``q [R, K]`` e4m3 bytes, packed scales) with blocks of 32 along ``K`` (``K % 128 == 0``)."""
    R, K = x.shape
    if K % 128 != 0:
        raise ValueError("MX quantisation needs a reduction dimension that is a multiple of 128")
    if not x.is_cuda:
        q, e = _emulate_quantize(x, mode)
        return q, scales_from_matrix(e, K)
    x = x if (x.stride(1) == 1 and x.dtype == torch.bfloat16) else x.to(torch.bfloat16).contiguous()
    q = torch.empty((R, K), dtype=torch.uint8, device=x.device)
    sf = torch.empty(_scale_bytes(R, K), dtype=torch.uint8, device=x.device)
    rc = _lib_mx().ocb_quantize_mx_rowwise(x.data_ptr(), q.data_ptr(), sf.data_ptr(), R, K, x.stride(0), q.stride(0),
                                           _MODES[mode], _lib.stream_ptr())
    _lib.check(rc, "ocb_quantize_mx_rowwise")
    return q, sf


def quantize_mx_colwise_transposed(x: torch.Tensor, mode: str = "rceil") -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [R, C]`` bf16 -> (``q_t [C, R]`` e4m3 bytes, packed scales of ``q_t``), blocks of 32 along ``R`` (``R % 128 == 0``)."""
    R, C = x.shape
    if R % 128 != 0:
        raise ValueError("MX quantisation needs a reduction dimension that is a multiple of 128")
    if not x.is_cuda:
        q, e = _emulate_quantize(x.t().contiguous(), mode)
        return q, scales_from_matrix(e, R)
    x = x if (x.stride(1) == 1 and x.dtype == torch.bfloat16) else x.to(torch.bfloat16).contiguous()
    q = torch.empty((C, R), dtype=torch.uint8, device=x.device)
    sf = torch.empty(_scale_bytes(C, R), dtype=torch.uint8, device=x.device)
    rc = _lib_mx().ocb_quantize_mx_colwise_t(x.data_ptr(), q.data_ptr(), sf.data_ptr(), R, C, x.stride(0), q.stride(0),
                                             _MODES[mode], _lib.stream_ptr())
    _lib.check(rc, "ocb_quantize_mx_colwise_t")
    return q, sf


def dequantize_mx(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    """fp32 values of a quantised ``[R, K]`` operand."""
    R, K = q.shape
    e = scales_as_matrix(sf, R, K).to(torch.int32)
    scale = torch.exp2((e - 127).float())
    return (q.view(torch.float8_e4m3fn).float().view(R, K // MX_BLOCK, MX_BLOCK) * scale[..., None]).view(R, K)


def gemm_mx(a_q: torch.Tensor, a_sf: torch.Tensor, b_q: torch.Tensor, b_sf: torch.Tensor, *,
            out: Optional[torch.Tensor] = None, accumulate: bool = False,
            out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``out (=|+=) dequant(a_q) @ dequant(b_q)^T``; ``a_q [M, K]``, ``b_q [N, K]`` e4m3 bytes with packed scales."""
    M, K = a_q.shape
    N = b_q.shape[0]
    if b_q.shape[1] != K:
        raise ValueError("MX GEMM inner dimensions differ")
    if not a_q.is_cuda:
        res = dequantize_mx(a_q, a_sf) @ dequantize_mx(b_q, b_sf).t()
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
        raise _lib.KernelError("the MX GEMM writes bf16, or fp32 (optionally accumulating)")
    rc = _lib_mx().ocb_gemm_mx(a_q.data_ptr(), b_q.data_ptr(), out.data_ptr(), a_sf.data_ptr(), b_sf.data_ptr(), M, N, K,
                               a_q.stride(0), b_q.stride(0), out.stride(0), epi,
                               _lib.status_buffer(a_q.device).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "ocb_gemm_mx")
    return out


class MXLinearFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, mode: str, cache: Optional[dict] = None):  # type: ignore[override]
        w = compute_weight(weight, torch.bfloat16)
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
        xq, sx = quantize_mx_rowwise(x2, mode)
        wq, sw = cached_weight_cast(cache, "mx_row", lambda: quantize_mx_rowwise(w, mode), weight._version)
        y = gemm_mx(xq, sx, wq, sw)
        ctx.save_for_backward(x2, w)
        ctx.mode = mode
        ctx.cache = cache
        ctx.weight_ref, ctx.x_shape, ctx.x_dtype = weight, x.shape, x.dtype
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x2, w = ctx.saved_tensors
        mode = ctx.mode
        weight = ctx.weight_ref
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = (dy2 if dy2.dtype == torch.bfloat16 else dy2.to(torch.bfloat16)).contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dyq, sdy = quantize_mx_rowwise(dy2, mode)
            wtq, swt = cached_weight_cast(ctx.cache, "mx_col_t", lambda: quantize_mx_colwise_transposed(w, mode), weight._version)  # [K, N], blocks along N
            dx = gemm_mx(dyq, sdy, wtq, swt).view(ctx.x_shape).to(ctx.x_dtype)
        main_grad = getattr(weight, "main_grad", None)
        dw = None
        if main_grad is not None or ctx.needs_input_grad[1]:
            dytq, sdyt = quantize_mx_colwise_transposed(dy2, mode)  # [N, M], blocks along the tokens
            xtq, sxt = quantize_mx_colwise_transposed(x2, mode)  # [K, M]
            if main_grad is not None:
                gemm_mx(dytq, sdyt, xtq, sxt, out=main_grad, accumulate=True)
            else:
                dw = gemm_mx(dytq, sdyt, xtq, sxt, out_dtype=torch.float32).to(weight.dtype)
        return dx, dw, None, None


def mx_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
              scale_rounding: str = "rceil", weight_cache: Optional[dict] = None) -> torch.Tensor:
    """
    ``x @ weight^T (+ bias)`` with MX-quantised operands in all three products. Shapes that the block layout cannot
    serve (token count, input or output width not a multiple of 128) run the bf16 GEMM instead.
    """
    rows = x.numel() // x.shape[-1]
    if not mx_supported(rows, weight.shape[1], weight.shape[0]):
        from .gemm import linear

        return linear(x, weight, bias)
    mode = scale_rounding if scale_rounding in _MODES else "rceil"
    y = MXLinearFunction.apply(x, weight, mode, weight_cache)
    return y if bias is None else y + bias.to(y.dtype)
