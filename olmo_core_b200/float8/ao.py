"""
Names of src/olmo_core/float8/ao.py:54-239: the enumerations and config classes through which float8 training is
configured. They select options of this package's own 8-bit kernels (:mod:`olmo_core_b200.ops.fp8`); nothing here needs
torchao.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..config import Config, StrEnum
from ..exceptions import OLMoConfigurationError

__all__ = ["AOScalingType", "AOScalingGranularity", "AOCastConfig", "AOFloat8GemmConfig", "AOFloat8LinearRecipe",
           "AOKernelPreference", "AOMXFP8Dim1CastKernelChoice", "AOScaleCalculationMode", "AOFloat8LinearConfig",
           "AOMXLinearConfig"]


class AOScalingType(StrEnum):
    dynamic = "dynamic"  # scales are computed from the tensor at every use
    disabled = "disabled"  # the operand stays in high precision


class AOScalingGranularity(StrEnum):
    tensorwise = "tensorwise"
    axiswise = "axiswise"  # one scale per row of the operand as the GEMM reads it


@dataclass
class AOCastConfig(Config):
    scaling_type: AOScalingType = AOScalingType.dynamic
    scaling_granularity: AOScalingGranularity = AOScalingGranularity.tensorwise
    target_dtype: Optional[str] = None  # "float8_e4m3fn" (default) or "float8_e5m2"


@dataclass
class AOFloat8GemmConfig(Config):
    use_fast_accum: bool = False  # accumulation is always fp32 in tensor memory here


class AOKernelPreference(StrEnum):
    auto = "auto"
    emulated = "emulated"  # quantise, then multiply in high precision (what CPU tensors always do)


class AOMXFP8Dim1CastKernelChoice(StrEnum):
    torch = "torch"
    cuda = "cuda"
    triton = "triton"


class AOScaleCalculationMode(StrEnum):
    floor = "floor"
    rceil = "rceil"
    ceil = "ceil"
    even = "even"


class AOFloat8LinearRecipe(StrEnum):
    tensorwise = "tensorwise"
    rowwise = "rowwise"
    rowwise_with_gw_hp = "rowwise_with_gw_hp"


@dataclass
class AOFloat8LinearConfig(Config):
    """
    Options of the row-wise scaled fp8 linear layers, with the field names of the reference's config
    (src/olmo_core/float8/ao.py:151-186). ``enable_fsdp_float8_all_gather`` keeps one set of quantised weight copies per
    optimizer step (the effect of casting before the sharded all-gather); ``round_scales_to_power_of_2`` rounds every
    scale up to a power of two; ``emulate`` and ``pad_inner_dim`` are accepted without effect (CPU tensors always take the
    emulated path, CUDA tensors the tensor-core kernels). The per-operand cast configs and
    per-GEMM configs are accepted: every operand is scaled dynamically along its reduction dimension here, and a cast
    config whose ``scaling_type`` is "disabled" for the weight-gradient operands selects the high-precision weight
    gradient (what the ``rowwise_with_gw_hp`` recipe does).
    """

    cast_config_input: Optional[AOCastConfig] = None
    cast_config_input_for_grad_weight: Optional[AOCastConfig] = None
    cast_config_weight: Optional[AOCastConfig] = None
    cast_config_weight_for_grad_input: Optional[AOCastConfig] = None
    cast_config_grad_output: Optional[AOCastConfig] = None
    cast_config_grad_output_for_grad_weight: Optional[AOCastConfig] = None
    gemm_config_output: Optional[AOFloat8GemmConfig] = None
    gemm_config_grad_input: Optional[AOFloat8GemmConfig] = None
    gemm_config_grad_weight: Optional[AOFloat8GemmConfig] = None
    enable_fsdp_float8_all_gather: Optional[bool] = None
    pad_inner_dim: Optional[bool] = None
    emulate: Optional[bool] = None
    force_recompute_fp8_weight_in_bwd: Optional[bool] = None  # accepted, no effect (as in the reference)
    round_scales_to_power_of_2: Optional[bool] = None
    recipe: Optional[AOFloat8LinearRecipe] = None

    @classmethod
    def recommended(cls, **kwargs) -> "AOFloat8LinearConfig":
        kwargs.setdefault("enable_fsdp_float8_all_gather", True)
        kwargs.setdefault("force_recompute_fp8_weight_in_bwd", True)
        kwargs.setdefault("round_scales_to_power_of_2", True)
        return cls(**kwargs)

    @property
    def wgrad_high_precision(self) -> bool:
        """True when the configs of the weight-gradient operands switch their cast off."""
        for cfg in (self.cast_config_input_for_grad_weight, self.cast_config_grad_output_for_grad_weight):
            if cfg is not None and str(getattr(cfg, "scaling_type", "")).split(".")[-1] == "disabled":
                return True
        return False


@dataclass
class AOMXLinearConfig(Config):
    """
    Micro-scaling linear layers (fields of src/olmo_core/float8/ao.py:189-232): e4m3 elements in blocks of 32 along the
    reduction dimension, one E8M0 scale per block. ``scale_calculation_mode``: "floor" (the format's default rule),
    "rceil" (tightest power of two that avoids saturation; what ``mxfp8_cublas_rceil`` selects), "ceil" or "even".
    The cast kernels and the GEMM are this package's own, so ``kernel_preference`` / ``mxfp8_cast_kernel_choice`` are
    accepted for compatibility and select nothing.
    """

    block_size: Optional[int] = None
    elem_dtype: Optional[str] = None
    elem_dtype_weight_override: Optional[str] = None
    elem_dtype_grad_output_override: Optional[str] = None
    kernel_preference: Optional[str] = None
    mxfp8_cast_kernel_choice: Optional[str] = None
    scale_calculation_mode: Optional[str] = None

    def __post_init__(self):
        if self.block_size not in (None, 32):
            raise OLMoConfigurationError(f"MX block size must be 32, got {self.block_size}")
        for name in ("elem_dtype", "elem_dtype_weight_override", "elem_dtype_grad_output_override"):
            value = getattr(self, name)
            if value is not None and str(value).split(".")[-1] not in ("float8_e4m3fn", "float8_e4m3"):
                raise OLMoConfigurationError(f"{name}={value!r}: the MX kernels implement e4m3 elements only")
        if self.scale_calculation_mode is not None and str(self.scale_calculation_mode).split(".")[-1] not in (
                "floor", "rceil", "ceil", "even"):
            raise OLMoConfigurationError(f"unknown scale_calculation_mode {self.scale_calculation_mode!r}")

    @property
    def scale_rounding(self) -> str:
        return str(self.scale_calculation_mode).split(".")[-1] if self.scale_calculation_mode is not None else "floor"

    @classmethod
    def mxfp8_cublas_rceil(cls, **kwargs) -> "AOMXLinearConfig":
        kwargs.setdefault("mxfp8_cast_kernel_choice", "cuda")
        kwargs.setdefault("scale_calculation_mode", "rceil")
        return cls(**kwargs)
