"""
Normalisation layers and their config (API of src/olmo_core/nn/layer_norm.py:25-386).

All RMS variants resolve to one GPU implementation, the fused kernel in
``olmo_core_b200/ops/csrc/elementwise.cu`` (fp32 statistics, 128-bit accesses, optional fused residual
add); the names ``rms``, ``fused_rms`` and ``cute_rms`` are accepted so that existing configs load.
CPU tensors take the PyTorch restatement of the same formula.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import DType, StrEnum
from ..exceptions import OLMoConfigurationError
from ..ops.elementwise import rms_norm
from .config import ModuleConfig

__all__ = [
    "LayerNormType",
    "LayerNormConfig",
    "LayerNorm",
    "RMSNorm",
    "QwenRMSNorm",
    "CuTeRMSNorm",
    "FusedRMSNorm",
    "L2Norm",
]


class LayerNormType(StrEnum):
    default = "default"
    rms = "rms"
    qwen_rms = "qwen_rms"
    cute_rms = "cute_rms"
    fused_rms = "fused_rms"
    l2_norm = "l2_norm"


@dataclass
class LayerNormConfig(ModuleConfig):
    name: LayerNormType = LayerNormType.default
    eps: Optional[float] = None
    elementwise_affine: Optional[bool] = None
    bias: Optional[bool] = None
    full_precision: Optional[bool] = None
    dtype: Optional[DType] = None

    def num_params(self, size: int) -> int:
        # every kind but the L2 norm has a weight and, unless switched off, a bias
        # (src/olmo_core/nn/layer_norm.py:73-91: the RMS kinds inherit the layer norm's ``bias=True`` default)
        affine = self.elementwise_affine if self.elementwise_affine is not None else self.name != LayerNormType.l2_norm
        if not affine:
            return 0
        has_bias = self.bias if self.bias is not None else self.name != LayerNormType.l2_norm
        return size * (2 if has_bias else 1)

    def build(self, size: int, init_device: str = "cpu") -> "LayerNorm":
        kwargs = self.as_dict(exclude_none=True)
        kwargs.pop("name")
        if (dtype := kwargs.pop("dtype", None)) is not None:
            kwargs["dtype"] = DType(dtype).as_pt() if not isinstance(dtype, torch.dtype) else dtype
        classes = {
            LayerNormType.default: LayerNorm,
            LayerNormType.rms: RMSNorm,
            LayerNormType.qwen_rms: QwenRMSNorm,
            LayerNormType.cute_rms: CuTeRMSNorm,
            LayerNormType.fused_rms: FusedRMSNorm,
            LayerNormType.l2_norm: L2Norm,
        }
        try:
            if self.name == LayerNormType.l2_norm:
                kwargs.pop("elementwise_affine", None)
                kwargs.pop("bias", None)
                kwargs.pop("eps", None)
                kwargs.pop("full_precision", None)
                kwargs.pop("dtype", None)
                return L2Norm(size=size)
            return classes[self.name](size=size, init_device=init_device, **kwargs)
        except TypeError as e:
            raise OLMoConfigurationError(f"invalid options for '{self.name}' {self.__class__.__name__}, {e}") from e


class LayerNorm(nn.Module):
    """Standard layer norm, optionally computed in fp32 regardless of the input dtype."""

    def __init__(
        self,
        *,
        size: int,
        eps: float = 1e-5,
        elementwise_affine: bool = True,
        bias: bool = True,
        full_precision: bool = True,
        dtype: torch.dtype = torch.float32,
        init_device: str = "cpu",
    ):
        super().__init__()
        self.normalized_shape = (size,)
        self.eps = eps
        self.full_precision = full_precision
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(size, dtype=dtype, device=init_device))
            if bias:
                self.bias = nn.Parameter(torch.zeros(size, dtype=dtype, device=init_device))
            else:
                self.register_parameter("bias", None)
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.weight is not None and self.weight.device.type != "meta":
            nn.init.ones_(self.weight)
        if self.bias is not None and self.bias.device.type != "meta":
            nn.init.zeros_(self.bias)

    def extra_repr(self) -> str:
        return f"{self.normalized_shape[0]}, eps={self.eps}, affine={self.weight is not None}"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        og = x.dtype
        if self.full_precision:
            w = None if self.weight is None else self.weight.float()
            b = None if self.bias is None else self.bias.float()
            return F.layer_norm(x.float(), self.normalized_shape, w, b, self.eps).to(og)
        w = None if self.weight is None else self.weight.to(og)
        b = None if self.bias is None else self.bias.to(og)
        return F.layer_norm(x, self.normalized_shape, w, b, self.eps)


class RMSNorm(LayerNorm):
    """``x * rsqrt(mean(x^2) + eps) * weight (+ bias)`` with fp32 math; output in the input dtype. As in the reference the
    bias exists unless ``bias=False`` is given (every model factory gives it)."""

    def __init__(
        self,
        *,
        size: int,
        eps: float = 1e-5,
        elementwise_affine: bool = True,
        bias: bool = True,
        full_precision: bool = True,
        dtype: torch.dtype = torch.float32,
        init_device: str = "cpu",
    ):
        super().__init__(size=size, eps=eps, elementwise_affine=elementwise_affine, bias=bias,
                         full_precision=full_precision, dtype=dtype, init_device=init_device)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, group: Optional[int] = None) -> torch.Tensor:
        """``residual``, when given, is added to the normalised output inside the same kernel."""
        if self.bias is None:
            return rms_norm(x, self.weight, self.eps, residual=residual, group=group)
        y = rms_norm(x, self.weight, self.eps, group=group) + self.bias.to(x.dtype)
        return y if residual is None else residual + y


class FusedRMSNorm(RMSNorm):
    """Alias of :class:`RMSNorm` (the reference's Triton-backed variant)."""


class CuTeRMSNorm(RMSNorm):
    """Alias of :class:`RMSNorm` (the reference's QuACK-backed variant)."""


class QwenRMSNorm(RMSNorm):
    """RMS norm that rounds to the input dtype *before* multiplying by the weight."""

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, group: Optional[int] = None) -> torch.Tensor:
        og = x.dtype
        xf = x.float()
        y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(og)
        if self.weight is not None:
            y = self.weight.to(og) * y
        if self.bias is not None:
            y = y + self.bias.to(og)
        return y if residual is None else residual + y


class L2Norm(nn.Module):
    """Scale to unit L2 norm along the last dimension (used by nGPT)."""

    def __init__(self, *, size: int):
        super().__init__()
        self.size = size

    def reset_parameters(self) -> None:
        pass

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return l2_normalize(x)


def l2_normalize(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    return (x.float() / torch.linalg.vector_norm(x.float(), dim=dim, keepdim=True).clamp(min=1e-12)).to(x.dtype)
