"""
Names of src/olmo_core/float8/ao.py:54-239: the enumerations and config classes through which float8 training is
configured. They select options of this package's own 8-bit kernels (:mod:`olmo_core_b200.ops.fp8`); nothing here needs
torchao.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..config import Config, StrEnum
from . import AOFloat8LinearConfig, AOFloat8LinearRecipe, AOMXLinearConfig

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
