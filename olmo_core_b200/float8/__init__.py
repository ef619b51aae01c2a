"""
Float8 training configuration (API of src/olmo_core/float8/__init__.py:17-162 and src/olmo_core/float8/ao.py:54-239).

The reference swaps ``nn.Linear`` for torchao's ``Float8Linear`` / ``MXLinear``. Here the same config classes select
the in-tree 8-bit linear ops: ``ao`` / ``ao_recipe`` the row-wise scaled e4m3 GEMM (``olmo_core_b200.ops.fp8``:
per-token activation scale, per-output-channel weight scale, power-of-two rounding optional, fp32 accumulation), and
``ao_mx`` the block-scaled MX GEMM (``olmo_core_b200.ops.mx``: one E8M0 scale per 32 reduction elements, applied by
``tcgen05.mma.kind::mxf8f6f4.block_scale``). Forward, dgrad and wgrad all run in 8 bits unless the recipe keeps the
weight gradient in bf16.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from fnmatch import fnmatch
from typing import Any, List, Optional

import torch
import torch.nn as nn

from ..config import Config
from ..exceptions import OLMoConfigurationError
from .ao import AOFloat8LinearConfig, AOFloat8LinearRecipe, AOMXLinearConfig

__all__ = ["Float8Config", "AOFloat8LinearConfig", "AOFloat8LinearRecipe", "AOMXLinearConfig", "refresh_float8_scales"]


@dataclass
class Float8Config(Config):
    ao: Optional[AOFloat8LinearConfig] = None
    ao_recipe: Optional[AOFloat8LinearRecipe] = None
    ao_mx: Optional[AOMXLinearConfig] = None
    modules_to_ignore: Optional[List[str]] = None
    enabled: bool = True
    cache_weight_casts: bool = False
    """Keep the quantised copies of every weight (one byte per parameter and layout) for all micro-batches of a step;
    implied by ``ao.enable_fsdp_float8_all_gather``."""

    def __post_init__(self):
        if sum(x is not None for x in (self.ao, self.ao_recipe, self.ao_mx)) > 1:
            raise OLMoConfigurationError("specify at most one of 'ao', 'ao_recipe' and 'ao_mx'")

    @property
    def should_precompute_float8_dynamic_scale_for_fsdp(self) -> bool:
        """Whether quantised weights are prepared once per optimizer step (src/olmo_core/float8/__init__.py:54-62)."""
        if self.ao_recipe is not None or self.ao_mx is not None:
            return False
        return bool(self.ao is not None and self.ao.enable_fsdp_float8_all_gather)

    @property
    def recipe(self) -> AOFloat8LinearRecipe:
        if self.ao_recipe is not None:
            return AOFloat8LinearRecipe(self.ao_recipe)
        if self.ao is not None and self.ao.recipe is not None:
            return AOFloat8LinearRecipe(self.ao.recipe)
        if self.ao is not None and self.ao.wgrad_high_precision:
            return AOFloat8LinearRecipe.rowwise_with_gw_hp
        return AOFloat8LinearRecipe.tensorwise if self.ao is not None else AOFloat8LinearRecipe.rowwise

    def apply_float8_linear(self, model: nn.Module, modules_to_ignore: Optional[List[str]] = None) -> None:
        """Mark every eligible projection (all dims multiples of 16, not the LM head) to run in fp8."""
        if not self.enabled:
            return
        from ..nn.feed_forward import Linear

        ignore = set(self.modules_to_ignore or []) | set(modules_to_ignore or []) | {"lm_head.w_out"}
        pow2 = bool(self.ao is not None and self.ao.round_scales_to_power_of_2)
        for name, module in model.named_modules():
            if not isinstance(module, Linear):
                continue
            if any(name == pat or fnmatch(name, pat) for pat in ignore):
                continue
            if module.in_features % 16 != 0 or module.out_features % 16 != 0:
                continue
            # "cast the weights once per step" (the reference's fp8 all-gather + scale precompute) = keep the quantised
            # copies of a weight until the next parameter update: one extra byte per parameter and layout
            keep = (self.ao is not None and self.ao.enable_fsdp_float8_all_gather) or self.cache_weight_casts
            cache = {} if keep else None
            module.float8 = dict(recipe=self.recipe, pow2_scales=pow2, mx=self.ao_mx,  # type: ignore[attr-defined]
                                 weight_cache=cache)


def refresh_float8_scales(model: nn.Module) -> None:
    """
    Hook after each optimizer step (src/olmo_core/nn/transformer/model.py:617-635 calls torchao's scale precompute
    there): activation scales are computed inside the quantisation kernels, so only the cached quantised weights have to
    be dropped; the first micro-batch of the next step re-creates them from the updated parameters.
    """
    for module in model.modules():
        f8 = getattr(module, "float8", None)
        if isinstance(f8, dict) and f8.get("weight_cache") is not None:
            f8["weight_cache"].clear()
