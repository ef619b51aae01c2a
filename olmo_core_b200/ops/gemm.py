"""
bf16 GEMM on tcgen05 tensor cores and the autograd-aware linear layer built on it.

``gemm`` drives ``csrc/gemm_sm100.cu`` (TMA -> 128B-swizzled smem -> ``tcgen05.mma`` -> TMEM -> epilogue).
``linear`` is the op behind every dense projection of the models (it replaces ``nn.Linear`` /
``F.linear`` used by the reference at src/olmo_core/nn/attention/__init__.py:379-390,
src/olmo_core/nn/feed_forward.py:161-171 and src/olmo_core/nn/lm_head.py:174). On CPU tensors both fall
back to ``torch.matmul``, which is also the numerical oracle in the tests.

Weight-gradient fusion: when the weight carries a ``main_grad`` attribute (an fp32 buffer owned by the
sharded-parameter runtime) the wgrad GEMM accumulates straight into it from its epilogue
(``C += A^T B`` in fp32) and autograd sees no gradient for the weight.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib

__all__ = ["gemm", "linear", "LinearFunction", "compute_weight", "swiglu_mlp", "stacked_pair"]


def _row_stride(t: torch.Tensor) -> int:
    if t.dim() != 2 or t.stride(1) != 1:
        raise _lib.KernelError("GEMM operands must be 2-D with unit inner stride")
    return t.stride(0) if t.size(0) > 1 else max(t.stride(0), t.size(1))


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    trans_a: bool = False,
    trans_b: bool = True,
    out: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """
    ``out (=|+=) op(a) @ op(b)`` with fp32 accumulation.

    Stored shapes: ``a`` is ``[M, K]`` (or ``[K, M]`` when ``trans_a``), ``b`` is ``[N, K]`` when
    ``trans_b`` (the ``nn.Linear`` weight layout) or ``[K, N]`` otherwise. Both must be bf16 on CUDA;
    ``out`` may be bf16 or fp32.
    """
    if trans_a:
        K, M = a.shape
    else:
        M, K = a.shape
    if trans_b:
        N, Kb = b.shape
    else:
        Kb, N = b.shape
    if K != Kb:
        raise ValueError(f"GEMM inner dimensions differ: {K} vs {Kb}")

    if not a.is_cuda:
        af = a.float().t() if trans_a else a.float()
        bf = b.float().t() if trans_b else b.float()
        res = af @ bf
        if out is None:
            return res.to(out_dtype or a.dtype)
        if accumulate:
            out.add_(res.to(out.dtype))
        else:
            out.copy_(res.to(out.dtype))
        return out

    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise _lib.KernelError(f"tcgen05 GEMM takes bfloat16 operands, got {a.dtype} and {b.dtype}")
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=a.device)
    if out.shape != (M, N):
        raise ValueError(f"output has shape {tuple(out.shape)}, expected {(M, N)}")
    if out.dtype == torch.bfloat16:
        epi = _lib.EPI_BF16_ACC if accumulate else _lib.EPI_BF16
    elif out.dtype == torch.float32:
        epi = _lib.EPI_F32_ACC if accumulate else _lib.EPI_F32
    else:
        raise _lib.KernelError(f"unsupported GEMM output dtype {out.dtype}")
    if M == 0 or N == 0:
        return out
    if K == 0:
        if not accumulate:
            out.zero_()
        return out
    rc = _lib.lib().ocb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
        _row_stride(a), _row_stride(b), _row_stride(out),
        1 if trans_a else 0, 0 if trans_b else 1, epi,
        _lib.status_buffer(a.device).data_ptr(), _lib.stream_ptr(),
    )
    _lib.check(rc, "ocb_gemm_bf16")
    return out


def compute_weight(weight: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """
    The tensor to feed the tensor cores for ``weight``: its resident low-precision copy when the
    sharded-parameter runtime attached one (``weight._lowp``), else a cast of the parameter itself.
    """
    lowp = getattr(weight, "_lowp", None)
    if lowp is not None and lowp.dtype == dtype:
        return lowp
    return weight if weight.dtype == dtype else weight.to(dtype)


class LinearFunction(torch.autograd.Function):
    """``y = x @ W^T`` for CUDA bf16 activations, with dgrad/wgrad on the same kernel."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        w = compute_weight(weight, torch.bfloat16)
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        y = gemm(x2, w, trans_b=True)
        ctx.save_for_backward(x2, w)
        ctx.weight_ref = weight
        ctx.x_shape = x.shape
        ctx.x_dtype = x.dtype
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy: torch.Tensor):  # type: ignore[override]
        x2, w = ctx.saved_tensors
        weight = ctx.weight_ref
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != torch.bfloat16:
            dy2 = dy2.to(torch.bfloat16)
        if dy2.stride(1) != 1:
            dy2 = dy2.contiguous()
        dx = None
        dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, trans_b=False).view(ctx.x_shape)
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                gemm(dy2, x2, trans_a=True, trans_b=False, out=main_grad, accumulate=True)
                if hasattr(weight, "grad_added_to_main_grad"):
                    weight.grad_added_to_main_grad = True
            else:
                dw = gemm(dy2, x2, trans_a=True, trans_b=False, out_dtype=torch.float32)
                if dw.dtype != weight.dtype:
                    dw = dw.to(weight.dtype)
        return dx, dw


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """
    Dense projection. CUDA + (bf16 activations or an attached low-precision weight copy) runs the
    tcgen05 kernel; anything else (CPU, fp32 debugging runs) uses ``F.linear``.
    """
    lowp = getattr(weight, "_lowp", None)
    if x.is_cuda and ((x.dtype == torch.bfloat16 and lowp is None) or (lowp is not None and lowp.dtype == torch.bfloat16)):
        y = LinearFunction.apply(x, weight)
        if bias is not None:
            y = y + bias.to(y.dtype)
        return y
    from .param import full_param

    b = None if bias is None else bias.to(x.dtype)
    return torch.nn.functional.linear(x, full_param(weight, x.dtype), b)


def grouped_gemm(x: torch.Tensor, weight: torch.Tensor, offsets: torch.Tensor, *, trans_b: bool,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """
    ``y[rows of group g] = x[rows of group g] @ op(W_g)`` in ONE kernel launch. ``x``: ``[R, K]`` bf16 sorted by group;
    ``offsets``: int32 ``[G + 1]`` device tensor of row prefix sums (read by the kernel: no host sync);
    ``weight``: the ``G`` operands stacked, ``[G * N, K]`` with ``trans_b`` (``y = x W^T``) else ``[G * K, N]``.
    """
    G = offsets.numel() - 1
    R, K = x.shape
    N = weight.shape[0] // G if trans_b else weight.shape[1]
    if (weight.shape[1] if trans_b else weight.shape[0] // G) != K:
        raise ValueError("grouped GEMM inner dimensions differ")
    if out is None:
        out = torch.empty((R, N), dtype=torch.bfloat16, device=x.device)
    if R == 0:
        return out
    if offsets.dtype != torch.int32 or not offsets.is_cuda:
        raise _lib.KernelError("offsets must be an int32 CUDA tensor")
    rc = _lib.lib().ocb_grouped_gemm_bf16(
        x.data_ptr(), weight.data_ptr(), out.data_ptr(), offsets.data_ptr(), G, 1, R, 0, N, K, _row_stride(x),
        _row_stride(weight), _row_stride(out), 0 if trans_b else 1, _lib.EPI_BF16,
        _lib.status_buffer(x.device).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "ocb_grouped_gemm_bf16")
    return out


def grouped_gemm_wgrad(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor, out: torch.Tensor, *,
                       accumulate: bool) -> torch.Tensor:
    """
    ``out_g (=|+=) a[rows of g]^T @ b[rows of g]`` for every group in one launch: ``a [R, M]``, ``b [R, N]`` bf16 sorted by
    group, ``out [G * M, N]`` fp32 (or bf16 without accumulation). Groups without rows give zeros (or leave ``out`` as is
    when accumulating).
    """
    G = offsets.numel() - 1
    R, M = a.shape
    N = b.shape[1]
    if out.shape != (G * M, N):
        raise ValueError(f"output has shape {tuple(out.shape)}, expected {(G * M, N)}")
    if out.dtype == torch.float32:
        epi = _lib.EPI_F32_ACC if accumulate else _lib.EPI_F32
    elif out.dtype == torch.bfloat16 and not accumulate:
        epi = _lib.EPI_BF16
    else:
        raise _lib.KernelError("grouped wgrad writes fp32 (optionally accumulating) or bf16")
    if R == 0:
        if not accumulate:
            out.zero_()
        return out
    rc = _lib.lib().ocb_grouped_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), offsets.data_ptr(), G, 2, R, M, N, 0, _row_stride(a), _row_stride(b),
        _row_stride(out), 1, epi, _lib.status_buffer(a.device).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "ocb_grouped_gemm_bf16")
    return out


class MultiLinearFunction(torch.autograd.Function):
    """
    Several projections of ONE input (``q, k, v = x W_q^T, x W_k^T, x W_v^T``; the two up-projections of a gated MLP).
    Forward is one GEMM per weight on a single saved copy of ``x``. Backward accumulates the input gradient across the
    projections in the GEMM epilogue (``dx = dy_0 W_0``, then ``dx += dy_i W_i``), so the element-wise additions that
    autograd would run to sum the per-projection gradients never happen.
    """

    @staticmethod
    def forward(ctx, x: torch.Tensor, *weights: torch.Tensor):  # type: ignore[override]
        ws = [compute_weight(w, torch.bfloat16) for w in weights]
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, *ws)
        ctx.weight_refs = weights
        ctx.x_shape, ctx.x_dtype = x.shape, x.dtype
        return tuple(gemm(x2, w, trans_b=True).view(*x.shape[:-1], w.shape[0]) for w in ws)

    @staticmethod
    def backward(ctx, *dys: torch.Tensor):  # type: ignore[override]
        x2, *ws = ctx.saved_tensors
        dx = None
        dws = []
        for i, (dy, w, weight) in enumerate(zip(dys, ws, ctx.weight_refs)):
            if dy is None:
                dws.append(None)
                continue
            dy2 = dy.reshape(-1, dy.shape[-1])
            if dy2.dtype != torch.bfloat16:
                dy2 = dy2.to(torch.bfloat16)
            if dy2.stride(1) != 1:
                dy2 = dy2.contiguous()
            if ctx.needs_input_grad[0]:
                if dx is None:
                    dx = gemm(dy2, w, trans_b=False)
                else:
                    gemm(dy2, w, trans_b=False, out=dx, accumulate=True)
            dw = None
            if ctx.needs_input_grad[1 + i]:
                main_grad = getattr(weight, "main_grad", None)
                if main_grad is not None:
                    gemm(dy2, x2, trans_a=True, trans_b=False, out=main_grad, accumulate=True)
                    if hasattr(weight, "grad_added_to_main_grad"):
                        weight.grad_added_to_main_grad = True
                else:
                    dw = gemm(dy2, x2, trans_a=True, trans_b=False, out_dtype=torch.float32)
                    if dw.dtype != weight.dtype:
                        dw = dw.to(weight.dtype)
            dws.append(dw)
        if dx is not None:
            dx = dx.view(ctx.x_shape)
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        return (dx, *dws)


def multi_linear(x: torch.Tensor, projections) -> tuple:
    """
    ``tuple(p(x) for p in projections)`` for bias-free ``Linear`` modules, through :class:`MultiLinearFunction` when
    the kernel path applies to all of them; otherwise each projection runs on its own.
    """
    plain = x.is_cuda and all(
        getattr(p, "bias", None) is None and getattr(p, "float8", None) is None
        and ((x.dtype == torch.bfloat16 and getattr(p.weight, "_lowp", None) is None)
             or (getattr(p.weight, "_lowp", None) is not None and p.weight._lowp.dtype == torch.bfloat16))
        for p in projections)
    if not plain:
        return tuple(p(x) for p in projections)
    return MultiLinearFunction.apply(x, *[p.weight for p in projections])


# ------------------------------------------------------------------------------------------------------
# Gated MLP with the activation inside the GEMM epilogues
# ------------------------------------------------------------------------------------------------------


def stacked_pair(first: torch.Tensor, second: torch.Tensor) -> Optional[torch.Tensor]:
    """
    ``[first; second]`` as ONE matrix without copying, when the two equally shaped row-major matrices sit back to back
    in memory (the sharded-parameter runtime lays out ``w1`` / ``w3`` of a gated MLP, and their gradient buffers, that
    way). ``None`` when they do not.
    """
    if (first.shape != second.shape or first.dtype != second.dtype or first.dim() != 2 or not first.is_contiguous()
            or not second.is_contiguous() or first.device != second.device
            or second.data_ptr() != first.data_ptr() + first.numel() * first.element_size()):
        return None
    if first.untyped_storage().data_ptr() != second.untyped_storage().data_ptr():
        return None
    rows, cols = first.shape
    return first.as_strided((2 * rows, cols), (cols, 1), first.storage_offset())


class SwiGLUMLPFunction(torch.autograd.Function):
    """
    ``y = (silu(x W1^T) * (x W3^T)) W2^T`` in three GEMM launches forward and four backward, with no element-wise
    kernel in between (reference: src/olmo_core/nn/feed_forward.py:161-171 runs three GEMMs, ``silu`` and a product):

    * forward: one GEMM over ``[W1; W3]`` whose epilogue stores ``a | b`` and ``h = silu(a) * b``; ``y = h W2^T``;
    * backward: ``dh = dy W2`` goes through the activation in the epilogue (``da | db`` stored, ``dh`` never is);
      ``dx = [da | db] [W1; W3]`` and ``d[W1; W3] += [da | db]^T x`` are one GEMM each; ``dW2 += dy^T h``.
    """

    @staticmethod
    def forward(ctx, x, w1, w3, w2, save_activation=True):  # type: ignore[override]
        w13 = stacked_pair(w1._lowp, w3._lowp)
        w2l = w2._lowp
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M, K = x2.shape
        H = w1.shape[0]
        ab = torch.empty((M, 2 * H), dtype=torch.bfloat16, device=x2.device)
        h = torch.empty((M, H), dtype=torch.bfloat16, device=x2.device)
        rc = _lib.lib().ocb_gemm_swiglu_fwd(x2.data_ptr(), w13.data_ptr(), ab.data_ptr(), h.data_ptr(), M, H, K, K, K, 2 * H,
                                            H, _lib.status_buffer(x2.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "ocb_gemm_swiglu_fwd")
        y = gemm(h, w2l, trans_b=True)
        if save_activation:
            ctx.save_for_backward(x2, ab, h, w13, w2l)
        else:
            ctx.save_for_backward(x2, ab, w13, w2l)  # h comes back out of the backward kernel's epilogue
        ctx.saved_h = bool(save_activation)
        ctx.weight_refs = (w1, w3, w2)
        ctx.x_shape, ctx.x_dtype = x.shape, x.dtype
        return y.view(*x.shape[:-1], w2l.shape[0])

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        if ctx.saved_h:
            x2, ab, h, w13, w2l = ctx.saved_tensors
        else:
            x2, ab, w13, w2l = ctx.saved_tensors
            h = None
        w1, w3, w2 = ctx.weight_refs
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != torch.bfloat16:
            dy2 = dy2.to(torch.bfloat16)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        M, D = dy2.shape
        H = w1.shape[0]
        dab = torch.empty_like(ab)
        h_out = None
        if h is None:
            h = h_out = torch.empty((M, H), dtype=torch.bfloat16, device=ab.device)
        rc = _lib.lib().ocb_gemm_swiglu_bwd(dy2.data_ptr(), w2l.data_ptr(), ab.data_ptr(), dab.data_ptr(),
                                            None if h_out is None else h_out.data_ptr(), M, H, D, D, H,
                                            2 * H, 2 * H, H, _lib.status_buffer(dy2.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "ocb_gemm_swiglu_bwd")
        gemm(dy2, h, trans_a=True, trans_b=False, out=w2.main_grad, accumulate=True)
        g13 = stacked_pair(w1.main_grad, w3.main_grad)
        gemm(dab, x2, trans_a=True, trans_b=False, out=g13, accumulate=True)
        for w in (w1, w3, w2):
            if hasattr(w, "grad_added_to_main_grad"):
                w.grad_added_to_main_grad = True
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dab, w13, trans_b=False).view(ctx.x_shape)
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        return dx, None, None, None, None


def swiglu_mlp(x: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor, *,
               save_activation: bool = True) -> Optional[torch.Tensor]:
    """
    The gated MLP through :class:`SwiGLUMLPFunction`, or ``None`` when its conditions do not hold: CUDA, bf16 resident
    copies of the three weights with ``w1`` / ``w3`` (and their fp32 gradient buffers) back to back in memory, sizes
    that are multiples of 8. The caller then runs the projections one by one.
    """
    if not x.is_cuda or x.shape[-1] % 8 != 0 or w1.shape[0] % 8 != 0:
        return None
    for w in (w1, w3, w2):
        lp, mg = getattr(w, "_lowp", None), getattr(w, "main_grad", None)
        if lp is None or mg is None or lp.dtype != torch.bfloat16 or mg.dtype != torch.float32 or lp.shape != w.shape:
            return None
        if getattr(w, "_tp_sharded", False) or not w.requires_grad:
            return None
    if stacked_pair(w1._lowp, w3._lowp) is None or stacked_pair(w1.main_grad, w3.main_grad) is None:
        return None
    return SwiGLUMLPFunction.apply(x, w1, w3, w2, save_activation)
