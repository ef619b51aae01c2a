"""
Gated MLP ``w2(act(w1 x) * w3 x)`` and its nGPT variant (API of src/olmo_core/nn/feed_forward.py:30-283).

On CUDA the three projections run on the tcgen05 GEMM (``ops.gemm.linear``) and the gate is the fused
SwiGLU kernel; tensor-parallel execution shards ``w1``/``w3`` by rows and ``w2`` by columns with the
sequence-parallel all-gather / reduce-scatter provided by ``olmo_core_b200.parallel.tensor``.
"""

from __future__ import annotations

import functools
import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import DType, StrEnum
from ..exceptions import OLMoConfigurationError
from ..ops.elementwise import swiglu
from ..ops.gemm import linear, multi_linear, swiglu_mlp
from .config import ModuleConfig
from .layer_norm import l2_normalize

__all__ = ["ActivationFunction", "FeedForwardType", "FeedForwardConfig", "FeedForward", "NormalizedFeedForward"]


class ActivationFunction(StrEnum):
    silu = "silu"
    gelu_tanh = "gelu_tanh"

    def build(self) -> Callable[[torch.Tensor], torch.Tensor]:
        if self == ActivationFunction.silu:
            return F.silu
        if self == ActivationFunction.gelu_tanh:
            return functools.partial(F.gelu, approximate="tanh")
        raise NotImplementedError(self)


class FeedForwardType(StrEnum):
    default = "default"
    normalized = "normalized"


@dataclass
class FeedForwardConfig(ModuleConfig):
    hidden_size: int
    name: FeedForwardType = FeedForwardType.default
    bias: Optional[bool] = None
    dtype: Optional[DType] = None
    activation: ActivationFunction = ActivationFunction.silu

    def num_params(self, d_model: int) -> int:
        has_bias = self.bias if self.bias is not None else self.name != FeedForwardType.normalized
        n = 3 * d_model * self.hidden_size
        if has_bias:
            n += 2 * self.hidden_size + d_model
        if self.name == FeedForwardType.normalized:
            n += 2 * self.hidden_size
        return n

    def build(self, d_model: int, *, dtype: Optional[torch.dtype] = None, init_device: str = "cpu") -> "FeedForward":
        kwargs = self.as_dict(exclude_none=True)
        kwargs.pop("name")
        kwargs.update(d_model=d_model, init_device=init_device)
        if self.dtype is not None:
            kwargs["dtype"] = self.dtype.as_pt()
        elif dtype is not None:
            kwargs["dtype"] = dtype
        try:
            if self.name == FeedForwardType.default:
                return FeedForward(**kwargs)
            if self.name == FeedForwardType.normalized:
                if kwargs.get("activation", ActivationFunction.silu) != ActivationFunction.silu:
                    raise OLMoConfigurationError("NormalizedFeedForward only supports 'silu' activation")
                kwargs.pop("activation", None)
                kwargs.pop("bias", None)
                return NormalizedFeedForward(**kwargs)
            raise NotImplementedError(self.name)
        except TypeError as e:
            raise OLMoConfigurationError(f"invalid options for '{self.name}' {self.__class__.__name__}, {e}") from e


class _Proj(nn.Module):
    """Weight (+ optional bias) holder with ``nn.Linear``'s parameter names, applied through ``ops.linear``."""

    def __init__(self, in_features: int, out_features: int, bias: bool, dtype: torch.dtype, device: str):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device))
        else:
            self.register_parameter("bias", None)
        if device != "meta":
            nn.init.trunc_normal_(self.weight, std=0.02, a=-0.06, b=0.06)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        f8 = getattr(self, "float8", None)  # set by Float8Config.apply_float8_linear
        if f8 is not None and f8.get("mx") is not None:
            from ..ops.mx import mx_linear

            return mx_linear(x, self.weight, self.bias, scale_rounding=str(getattr(f8["mx"], "scale_rounding", "rceil")),
                             weight_cache=f8.get("weight_cache"))
        if f8 is not None and x.is_cuda and x.numel() // x.shape[-1] % 16 == 0:
            from ..ops.fp8 import fp8_linear

            return fp8_linear(x, self.weight, self.bias, pow2_scales=bool(f8.get("pow2_scales")),
                              wgrad_high_precision=str(f8.get("recipe")) == "rowwise_with_gw_hp",
                              weight_cache=f8.get("weight_cache"))
        return linear(x, self.weight, self.bias)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


Linear = _Proj


class FeedForward(nn.Module):
    def __init__(
        self,
        *,
        d_model: int,
        hidden_size: int,
        bias: bool = True,
        dtype: torch.dtype = torch.float32,
        init_device: str = "cpu",
        activation: ActivationFunction = ActivationFunction.silu,
    ):
        super().__init__()
        self.d_model = d_model
        self.hidden_size = hidden_size
        self.activation = ActivationFunction(activation)
        self._act = self.activation.build()
        self.w1 = _Proj(d_model, hidden_size, bias, dtype, init_device)
        self.w2 = _Proj(hidden_size, d_model, bias, dtype, init_device)
        self.w3 = _Proj(d_model, hidden_size, bias, dtype, init_device)
        self.recompute_activation = False
        """Do not keep ``silu(a) * b`` for the backward pass; the fused backward kernel re-derives it ('selected_ops')."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if (self.activation == ActivationFunction.silu and x.is_cuda and self.w1.bias is None
                and all(getattr(w, "float8", None) is None for w in (self.w1, self.w2, self.w3))):
            y = swiglu_mlp(x, self.w1.weight, self.w3.weight, self.w2.weight,  # activation inside the GEMM epilogues
                           save_activation=not self.recompute_activation)
            if y is not None:
                return y
        a, b = multi_linear(x, (self.w1, self.w3))  # one saved input, input gradients summed in the GEMM epilogue
        if self.activation == ActivationFunction.silu:
            return self.w2(swiglu(a, b))
        return self.w2(self._act(a) * b)

    def apply_tp(self, tp_mesh, input_layout=None, output_layout=None, use_local_output: bool = True,
                 float8_enabled: bool = False) -> None:
        """
        ``w1`` / ``w3`` column-parallel, ``w2`` row-parallel over ``tp_mesh``
        (src/olmo_core/nn/feed_forward.py:173-204). The layouts are fixed here: the input arrives sharded along the
        sequence, is gathered inside the up-projection GEMMs, and the output returns to sequence shards through the
        down-projection's epilogue, so the layout arguments are accepted and ignored.
        """
        del input_layout, output_layout, use_local_output, float8_enabled
        from ..parallel.tensor import shard_feed_forward_

        shard_feed_forward_(self, tp_mesh)

    def num_flops_per_token(self, seq_len: int) -> int:
        return 6 * sum(p.numel() for p in self.parameters())


class NormalizedFeedForward(FeedForward):
    """nGPT MLP: unit-norm weight rows plus learned per-channel scales ``sw1``/``sw3``."""

    def __init__(self, *, d_model: int, hidden_size: int, dtype: torch.dtype = torch.float32, init_device: str = "cpu",
                 activation: ActivationFunction = ActivationFunction.silu):
        if ActivationFunction(activation) != ActivationFunction.silu:
            raise OLMoConfigurationError(f"NormalizedFeedForward only supports 'silu' activation, got '{activation}'")
        super().__init__(d_model=d_model, hidden_size=hidden_size, bias=False, dtype=dtype, init_device=init_device)
        self.sw_init_value = 1.0
        self.sw_init_scaling = 1.0
        self.sw1 = nn.Parameter(torch.empty(hidden_size, dtype=dtype, device=init_device))
        self.sw3 = nn.Parameter(torch.empty(hidden_size, dtype=dtype, device=init_device))
        self.sqrt_d_model = math.sqrt(d_model)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.sw1.device.type != "meta":
            nn.init.constant_(self.sw1, self.sw_init_scaling)
            nn.init.constant_(self.sw3, self.sw_init_scaling)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        sw1 = self.sw1 * ((self.sw_init_value / self.sw_init_scaling) * self.sqrt_d_model)
        sw3 = self.sw3 * (self.sw_init_value / self.sw_init_scaling)
        return self.w2(F.silu(sw1.to(x.dtype) * self.w1(x)) * (sw3.to(x.dtype) * self.w3(x)))

    def apply_tp(self, *args, **kwargs) -> None:
        raise NotImplementedError("TP is not implemented yet for the normalized feed-forward variant")

    @torch.no_grad()
    def normalize_matrices(self) -> None:
        for w, dim in ((self.w1.weight, -1), (self.w3.weight, -1), (self.w2.weight, 0)):
            w.copy_(l2_normalize(w, dim=dim))
