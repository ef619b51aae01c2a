"""
Model configuration: :class:`TransformerConfig`, :class:`TransformerBlockConfig` and the named model
sizes (API of src/olmo_core/nn/transformer/config.py:40-2067).

The named sizes (``olmo2_7B``, ``olmo3_32B``, ``llama3_8B``, ``qwen3_4B``, ``gemma3_12B`` ...) are generated
from the table :data:`MODEL_SIZES` -- one row of hyper-parameters per model, layered on the generic builders
``llama_like`` / ``llama_like_moe`` / ``ngpt_like`` / ``gemma3_like`` / ``qwen3_5_like``.
"""

from __future__ import annotations

import logging
import math
from dataclasses import InitVar, dataclass, field
from fnmatch import fnmatch
from itertools import cycle, islice
from typing import Any, Callable, Dict, List, Optional, Union

from ...config import UNSET, DType, StrEnum
from ...exceptions import OLMoConfigurationError
from ...utils import ensure_multiple_of
from ..attention import (
    AttentionBackendName,
    AttentionConfig,
    AttentionType,
    GateConfig,
    GateGranularity,
    SequenceMixerConfig,
    SlidingWindowAttentionConfig,
)
from ..buffer_cache import BufferCache
from ..config import ModelConfig, ModuleConfig
from ..feed_forward import ActivationFunction, FeedForwardConfig, FeedForwardType
from ..layer_norm import LayerNormConfig, LayerNormType
from ..lm_head import LMHeadConfig, LMHeadType
from ..moe import MoEConfig, MoERouterConfig, MoEType
from ..rope import RoPEConfig, RoPEScalingConfig, RoPEType
from .init import InitMethod

__all__ = [
    "TransformerType",
    "TransformerBlockType",
    "TransformerDataParallelWrappingStrategy",
    "TransformerActivationCheckpointingMode",
    "TransformerBlockConfig",
    "TransformerConfig",
    "MODEL_SIZES",
    "resolve_block_configs",
    "validate_block_resolution_config",
]

log = logging.getLogger(__name__)


class TransformerDataParallelWrappingStrategy(StrEnum):
    """Granularity at which parameters are grouped for sharded data parallelism."""

    full = "full"
    blocks = "blocks"
    fine_grained = "fine_grained"


class TransformerActivationCheckpointingMode(StrEnum):
    full = "full"
    selected_blocks = "selected_blocks"
    selected_modules = "selected_modules"
    selected_ops = "selected_ops"
    budget = "budget"


class TransformerType(StrEnum):
    default = "default"
    normalized = "normalized"
    moe = "moe"


class TransformerBlockType(StrEnum):
    default = "default"
    default_scaled = "default_scaled"
    reordered_norm = "reordered_norm"
    peri_norm = "peri_norm"
    normalized = "normalized"
    moe = "moe"
    moe_reordered_norm = "moe_reordered_norm"
    moe_hybrid = "moe_hybrid"
    moe_hybrid_reordered_norm = "moe_hybrid_reordered_norm"


@dataclass
class TransformerBlockConfig(ModuleConfig):
    sequence_mixer: SequenceMixerConfig = field(default=UNSET)
    attention: InitVar[Optional[AttentionConfig]] = None  # deprecated alias of ``sequence_mixer``
    layer_norm: Optional[LayerNormConfig] = None
    feed_forward: Optional[FeedForwardConfig] = None
    feed_forward_moe: Optional[MoEConfig] = None
    name: TransformerBlockType = TransformerBlockType.default
    dropout: Optional[float] = None
    attention_residual_alpha: Optional[float] = None
    feed_forward_residual_alpha: Optional[float] = None

    def __post_init__(self, attention: Optional[AttentionConfig] = None):
        if attention is not None and not isinstance(attention, property):
            if self.sequence_mixer is not UNSET:
                raise OLMoConfigurationError("Cannot specify both 'attention' and 'sequence_mixer' in TransformerBlockConfig.")
            self.sequence_mixer = attention
        if self.sequence_mixer is UNSET:
            raise OLMoConfigurationError("TransformerBlockConfig requires 'sequence_mixer' to be set.")

    def build(self, *, d_model: int, block_idx: int, n_layers: int, init_device: str = "cpu",
              cache: Optional[BufferCache] = None):
        from . import block as B

        classes = {
            TransformerBlockType.default: B.TransformerBlock,
            TransformerBlockType.default_scaled: B.LayerNormScaledTransformerBlock,
            TransformerBlockType.reordered_norm: B.ReorderedNormTransformerBlock,
            TransformerBlockType.peri_norm: B.PeriNormTransformerBlock,
            TransformerBlockType.normalized: B.NormalizedTransformerBlock,
            TransformerBlockType.moe: B.MoETransformerBlock,
            TransformerBlockType.moe_reordered_norm: B.MoEReorderedNormTransformerBlock,
            TransformerBlockType.moe_hybrid: B.MoEHybridTransformerBlock,
            TransformerBlockType.moe_hybrid_reordered_norm: B.MoEHybridReorderedNormTransformerBlock,
        }
        kwargs = self.as_dict(exclude_none=True, recurse=False)
        kwargs.pop("name")
        kwargs.update(d_model=d_model, block_idx=block_idx, n_layers=n_layers, init_device=init_device, cache=cache)
        block_cls = classes.get(TransformerBlockType(self.name))
        if block_cls is None:
            raise NotImplementedError(self.name)
        try:
            return block_cls(**kwargs)
        except TypeError as e:
            raise OLMoConfigurationError(f"invalid options for '{self.name}' {self.__class__.__name__}, {e}") from e

    def num_params(self, d_model: int) -> int:
        n = self.sequence_mixer.num_params(d_model)
        ln = self.layer_norm.num_params(d_model) if self.layer_norm is not None else 0
        if self.name == TransformerBlockType.normalized:
            n += 2 * d_model
        n += ln  # the mixer's norm
        if self.feed_forward is not None:
            n += self.feed_forward.num_params(d_model) + ln
        if self.feed_forward_moe is not None:
            n += self.feed_forward_moe.num_params(d_model) + ln
        if self.name == TransformerBlockType.peri_norm:
            n += 2 * ln
        return n

    def num_active_params(self, d_model: int) -> int:
        n = self.num_params(d_model)
        if self.feed_forward_moe is not None:
            n -= self.feed_forward_moe.num_params(d_model) - self.feed_forward_moe.num_active_params(d_model)
        return n


def validate_block_resolution_config(n_layers: int, block, block_pattern: Optional[List[str]] = None,
                                     block_overrides: Optional[Dict[int, TransformerBlockConfig]] = None) -> None:
    if not isinstance(block, dict):
        if block_pattern is not None:
            raise OLMoConfigurationError("`block_pattern` is not supported when `block` is not a dict of named blocks.")
        return
    if not block_pattern:
        raise OLMoConfigurationError("`block_pattern` must be provided and non-empty when `block` is a dict of named blocks.")
    if block_overrides is not None:
        raise OLMoConfigurationError("`block_overrides` is not supported when `block` is a dict of named blocks.")
    unknown = set(block_pattern) - set(block)
    if unknown:
        raise OLMoConfigurationError(f"Every name in `block_pattern` must exist in `block`. Unknown names: {unknown}.")


def resolve_block_configs(n_layers: int, block, block_pattern: Optional[List[str]] = None,
                          block_overrides: Optional[Dict[int, TransformerBlockConfig]] = None) -> List[TransformerBlockConfig]:
    """The block config of every layer, after applying the name pattern or the per-index overrides."""
    validate_block_resolution_config(n_layers, block, block_pattern, block_overrides)
    if isinstance(block, dict):
        assert block_pattern is not None
        return [block[name] for name in islice(cycle(block_pattern), n_layers)]
    configs = [block] * n_layers
    for idx, override in (block_overrides or {}).items():
        configs[int(idx)] = override
    return configs


# ----------------------------------------------------------------------------------------------------------
# Named sizes. Each row: (builder, fixed builder arguments, overridable defaults).
# ----------------------------------------------------------------------------------------------------------

_OLMO2 = dict(block_name=TransformerBlockType.reordered_norm, qk_norm=True, rope_theta=500_000)
_QWEN3 = dict(head_dim=128, rope_theta=1_000_000, rope_full_precision=False, qk_norm=True, use_head_qk_norm=True)

MODEL_SIZES: Dict[str, Dict[str, Any]] = {
    # name: fixed = always passed, defaults = may be overridden by the caller's kwargs
    "olmo2_1M": dict(fixed=dict(d_model=12, hidden_size_multiplier=1.0, layer_norm_eps=1e-6), defaults=dict(n_layers=4, n_heads=4, head_dim=4, **_OLMO2)),
    "olmo2_14M": dict(fixed=dict(d_model=128, layer_norm_eps=1e-6), defaults=dict(n_layers=4, n_heads=8, **_OLMO2)),
    "olmo2_30M": dict(fixed=dict(d_model=256, layer_norm_eps=1e-6), defaults=dict(n_layers=4, n_heads=8, **_OLMO2)),
    "olmo2_60M": dict(fixed=dict(d_model=384, hidden_size_multiplier=1.5, layer_norm_eps=1e-6), defaults=dict(n_layers=8, n_heads=8, **_OLMO2)),
    "olmo2_100M": dict(fixed=dict(d_model=512, hidden_size_multiplier=1.5, layer_norm_eps=1e-6), defaults=dict(n_layers=12, n_heads=8, **_OLMO2)),
    "olmo2_190M": dict(fixed=dict(d_model=768, hidden_size_multiplier=1.5, layer_norm_eps=1e-6), defaults=dict(n_layers=12, n_heads=12, **_OLMO2)),
    "olmo2_370M": dict(fixed=dict(d_model=1024, hidden_size_multiplier=1.5, layer_norm_eps=1e-6), defaults=dict(n_layers=16, n_heads=16, **_OLMO2)),
    "olmo2_600M": dict(fixed=dict(hidden_size_multiplier=1.5, layer_norm_eps=1e-6), defaults=dict(d_model=1344, n_layers=16, n_heads=16, **_OLMO2)),
    "olmo2_760M": dict(fixed=dict(d_model=1536, hidden_size_multiplier=1.5, layer_norm_eps=1e-6), defaults=dict(n_layers=16, n_heads=16, **_OLMO2)),
    "olmo2_1B": dict(fixed=dict(d_model=2048, hidden_size_multiplier=1.5, layer_norm_eps=1e-6), defaults=dict(n_layers=18, n_heads=16, **_OLMO2)),
    "olmo2_1B_v2": dict(fixed=dict(d_model=2048, layer_norm_eps=1e-6), defaults=dict(n_layers=16, n_heads=16, hidden_size_multiplier=1.5, **_OLMO2)),
    "olmo2_3B": dict(fixed=dict(d_model=3328, hidden_size_multiplier=1.5, layer_norm_eps=1e-6), defaults=dict(n_layers=16, n_heads=16, **_OLMO2)),
    "olmo2_7B": dict(fixed=dict(d_model=4096, layer_norm_eps=1e-6), defaults=dict(n_layers=32, n_heads=32, **_OLMO2)),
    "olmo2_13B": dict(fixed=dict(d_model=5120, layer_norm_eps=1e-6), defaults=dict(n_layers=40, n_heads=40, **_OLMO2)),
    "olmo2_32B": dict(fixed=dict(d_model=5120, layer_norm_eps=1e-6),
                      defaults=dict(n_layers=64, n_heads=40, n_kv_heads=8, hidden_size_multiple_of=512,
                                    hidden_size_multiplier=27648 / (8 * 5120 / 3), **_OLMO2)),
    "llama2_271M": dict(fixed=dict(d_model=1024), defaults=dict(n_layers=16, n_heads=8, rope_theta=10_000)),
    "llama2_1B": dict(fixed=dict(d_model=2048), defaults=dict(n_layers=18, n_heads=16, rope_theta=10_000)),
    "llama2_7B": dict(fixed=dict(d_model=4096), defaults=dict(n_layers=32, n_heads=32, rope_theta=10_000)),
    "llama2_13B": dict(fixed=dict(d_model=5120), defaults=dict(n_layers=40, n_heads=40, rope_theta=10_000)),
    "llama2_26B": dict(fixed=dict(d_model=5120), defaults=dict(n_layers=80, n_heads=40, rope_theta=10_000)),
    "llama2_70B": dict(fixed=dict(d_model=8192, hidden_size_multiplier=1.3, hidden_size_multiple_of=4096),
                       defaults=dict(n_layers=80, n_heads=64, n_kv_heads=8, rope_theta=10_000)),
    "llama3_1B": dict(fixed=dict(d_model=2048, hidden_size_multiplier=1.5), defaults=dict(n_layers=16, n_heads=32, n_kv_heads=8, rope_theta=500_000)),
    "llama3_8B": dict(fixed=dict(d_model=4096, hidden_size_multiplier=1.3, hidden_size_multiple_of=1024),
                      defaults=dict(n_layers=32, n_heads=32, n_kv_heads=8, rope_theta=500_000)),
    "llama3_70B": dict(fixed=dict(d_model=8196, hidden_size_multiplier=1.3, hidden_size_multiple_of=4096),
                       defaults=dict(n_layers=80, n_heads=64, n_kv_heads=8, rope_theta=500_000)),
    "llama3_405B": dict(fixed=dict(d_model=16384, hidden_size_multiplier=1.2, hidden_size_multiple_of=4096),
                        defaults=dict(n_layers=126, n_heads=128, n_kv_heads=8, rope_theta=500_000)),
    "qwen3_0_6B": dict(fixed=dict(d_model=1024, ffn=3072), defaults=dict(n_layers=28, n_heads=16, n_kv_heads=8, tie_word_embeddings=True, **_QWEN3)),
    "qwen3_1_7B": dict(fixed=dict(d_model=2048, ffn=6144), defaults=dict(n_layers=28, n_heads=16, n_kv_heads=8, tie_word_embeddings=True, **_QWEN3)),
    "qwen3_4B": dict(fixed=dict(d_model=2560, ffn=9728), defaults=dict(n_layers=36, n_heads=32, n_kv_heads=8, tie_word_embeddings=True, **_QWEN3)),
    "qwen3_8B": dict(fixed=dict(d_model=4096, ffn=12288), defaults=dict(n_layers=36, n_heads=32, n_kv_heads=8, **_QWEN3)),
    "qwen3_14B": dict(fixed=dict(d_model=5120, ffn=17408), defaults=dict(n_layers=48, n_heads=40, n_kv_heads=8, **_QWEN3)),
    "qwen3_32B": dict(fixed=dict(d_model=5120, ffn=25600), defaults=dict(n_layers=64, n_heads=40, n_kv_heads=8, **_QWEN3)),
}
_OLMO3_BASE = {
    "olmo3_1M": "olmo2_1M", "olmo3_14M": "olmo2_14M", "olmo3_30M": "olmo2_30M", "olmo3_60M": "olmo2_60M",
    "olmo3_100M": "olmo2_100M", "olmo3_190M": "olmo2_190M", "olmo3_370M": "olmo2_370M", "olmo3_600M": "olmo2_600M",
    "olmo3_760M": "olmo2_760M", "olmo3_1B": "olmo2_1B_v2", "olmo3_3B": "olmo2_3B", "olmo3_7B": "olmo2_7B",
    "olmo3_13B": "olmo2_13B", "olmo3_32B": "olmo2_32B",
}
_GEMMA3 = {"gemma3_1B": (2304, 26, 8, 4, 9216), "gemma3_4B": (2560, 34, 16, 4, 10240),
           "gemma3_12B": (3840, 48, 24, 8, 15360), "gemma3_27B": (5376, 62, 32, 16, 21504)}
_QWEN3_5 = {"qwen3_5_0_8B": (1024, 24, 8, 2, 3584, 16, 16), "qwen3_5_4B": (2560, 32, 16, 4, 9216, 16, 32),
            "qwen3_5_9B": (4096, 32, 16, 4, 12288, 16, 32), "qwen3_5_27B": (5120, 64, 24, 4, 17408, 16, 48)}
_MOE = {  # name: (block type, MoE type, experts, top_k, shared MLP?, dense MLP?)
    "smallmoe": dict(d_model=768, n_layers=12, n_heads=12, block=TransformerBlockType.moe_reordered_norm, moe=MoEType.default,
                     experts=32, top_k=4, shared=True, dense=False),
    "small_hybrid_moe": dict(d_model=768, n_layers=12, n_heads=12, block=TransformerBlockType.moe_hybrid_reordered_norm,
                             moe=MoEType.default, experts=32, top_k=4, shared=False, dense=True),
    "olmoe_1B_7B": dict(d_model=2048, n_layers=16, n_heads=16, block=TransformerBlockType.moe_reordered_norm,
                        moe=MoEType.dropless, experts=64, top_k=8, shared=False, dense=False),
}


def _sliding_window_default() -> SlidingWindowAttentionConfig:
    return SlidingWindowAttentionConfig(pattern=[4096, 4096, 4096, -1], force_full_attention_on_first_layer=False,
                                        force_full_attention_on_last_layer=True)


@dataclass
class TransformerConfig(ModelConfig):
    d_model: int
    vocab_size: int
    n_layers: int
    block: Union[TransformerBlockConfig, Dict[str, TransformerBlockConfig]]
    lm_head: LMHeadConfig
    embedding_norm: Optional[LayerNormConfig] = None
    name: TransformerType = TransformerType.default
    dtype: DType = DType.float32
    init_method: InitMethod = InitMethod.normal
    init_seed: int = 0
    init_std: float = 0.02
    embedding_init_std: Optional[float] = None
    freeze_params: Optional[List[str]] = None
    block_pattern: Optional[List[str]] = None
    block_overrides: Optional[Dict[int, TransformerBlockConfig]] = None
    embed_scale: Optional[float] = None
    tie_word_embeddings: bool = False

    def __post_init__(self):
        if self.tie_word_embeddings and self.name == TransformerType.normalized:
            raise OLMoConfigurationError("Tying word embeddings is not supported with the normalized transformer")
        validate_block_resolution_config(self.n_layers, self.block, self.block_pattern, self.block_overrides)

    # -- building --------------------------------------------------------------------------------------
    def build(self, *, init_device: str = "cpu"):
        from .model import MoETransformer, NormalizedTransformer, Transformer

        common = dict(
            d_model=self.d_model, vocab_size=self.vocab_size, n_layers=self.n_layers, block=self.block,
            lm_head=self.lm_head, dtype=DType(self.dtype).as_pt(), init_method=self.init_method, init_device=init_device,
            init_seed=self.init_seed, init_std=self.init_std, embedding_init_std=self.embedding_init_std,
            block_overrides=self.block_overrides, block_pattern=self.block_pattern,
        )
        if self.name == TransformerType.default:
            model = Transformer(embedding_norm=self.embedding_norm, embed_scale=self.embed_scale,
                                tie_word_embeddings=self.tie_word_embeddings, **common)
        elif self.name == TransformerType.normalized:
            if self.embedding_norm is not None:
                raise OLMoConfigurationError("the normalized transformer takes no embedding norm")
            model = NormalizedTransformer(**common)
        elif self.name == TransformerType.moe:
            model = MoETransformer(embedding_norm=self.embedding_norm, tie_word_embeddings=self.tie_word_embeddings, **common)
        else:
            raise NotImplementedError(self.name)
        for pname, param in model.named_parameters():
            if any(fnmatch(pname, pat) for pat in (self.freeze_params or [])):
                param.requires_grad = False
        return model

    @property
    def resolved_block_configs(self) -> List[TransformerBlockConfig]:
        return resolve_block_configs(self.n_layers, self.block, self.block_pattern, self.block_overrides)

    # -- parameter counts ------------------------------------------------------------------------------
    def _count(self, active: bool) -> int:
        n = self.d_model * self.vocab_size
        if self.embedding_norm is not None:
            n += self.embedding_norm.num_params(self.d_model)
        for b in self.resolved_block_configs:
            n += b.num_active_params(self.d_model) if active else b.num_params(self.d_model)
        n += self.lm_head.num_params(self.d_model, self.vocab_size)
        if self.tie_word_embeddings:
            n -= self.d_model * self.vocab_size
        return n

    @property
    def num_params(self) -> int:
        return self._count(active=False)

    @property
    def num_active_params(self) -> int:
        return self._count(active=True)

    @property
    def num_non_embedding_params(self) -> int:
        return self.num_params - self.d_model * self.vocab_size

    @property
    def num_active_non_embedding_params(self) -> int:
        return self.num_active_params - self.d_model * self.vocab_size

    def num_flops_per_token(self, seq_len: int) -> int:
        """Analytic FLOPs per token, the quantity the MFU meter divides by (built on the meta device)."""
        return self.build(init_device="meta").num_flops_per_token(seq_len)

    # -- generic builders ------------------------------------------------------------------------------
    @classmethod
    def llama_like(
        cls,
        *,
        d_model: int,
        vocab_size: int,
        n_layers: int,
        n_heads: int,
        n_kv_heads: Optional[int] = None,
        head_dim: Optional[int] = None,
        gate: Optional[GateConfig] = None,
        qk_norm: bool = False,
        use_head_qk_norm: bool = False,
        layer_norm_eps: float = 1e-5,
        layer_norm_name: Optional[LayerNormType] = None,
        rope_theta: int = 500_000,
        rope_type: Optional[RoPEType] = None,
        rope_full_precision: bool = True,
        no_global_rope: bool = False,
        hidden_size_multiple_of: int = 256,
        hidden_size_multiplier: Optional[float] = None,
        fused_ops: bool = False,
        use_flash: Optional[bool] = None,
        attn_backend: Optional[AttentionBackendName] = None,
        sliding_window: Optional[SlidingWindowAttentionConfig] = None,
        block_name: TransformerBlockType = TransformerBlockType.default,
        block_mods: Optional[Dict[int, Callable[[TransformerBlockConfig], TransformerBlockConfig]]] = None,
        dtype: DType = DType.float32,
        rope_scaling: Optional[RoPEScalingConfig] = None,
        feed_forward: Optional[FeedForwardConfig] = None,
        feed_forward_moe: Optional[MoEConfig] = None,
        **kwargs,
    ) -> "TransformerConfig":
        """Llama-style decoder: RMSNorm, RoPE, SwiGLU MLP with hidden size ``8/3 d`` rounded up."""
        hidden = int(8 * d_model / 3)
        if hidden_size_multiplier is not None:
            hidden = int(hidden_size_multiplier * hidden)
        hidden = ensure_multiple_of(hidden, hidden_size_multiple_of)
        norm_name = layer_norm_name or (LayerNormType.fused_rms if fused_ops else LayerNormType.rms)
        norm = LayerNormConfig(name=norm_name, eps=layer_norm_eps, bias=False, dtype=dtype)
        att_type = AttentionType.default
        if rope_type is None:
            rope_type = RoPEType.default
            if fused_ops and n_kv_heads is None:
                att_type, rope_type = AttentionType.fused, RoPEType.fused
        if feed_forward is None and feed_forward_moe is None:
            feed_forward = FeedForwardConfig(hidden_size=hidden, bias=False, dtype=dtype)
        block = TransformerBlockConfig(
            name=block_name,
            sequence_mixer=AttentionConfig(
                name=att_type, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, bias=False,
                rope=RoPEConfig(name=rope_type, theta=rope_theta, full_precision=rope_full_precision,
                                no_global_rope=no_global_rope, scaling=rope_scaling),
                gate=gate, qk_norm=norm if qk_norm else None, use_head_qk_norm=use_head_qk_norm if qk_norm else None,
                use_flash=use_flash, backend=attn_backend, sliding_window=sliding_window, dtype=dtype,
            ),
            feed_forward=feed_forward,
            feed_forward_moe=feed_forward_moe,
            layer_norm=norm,
        )
        overrides = kwargs.pop("block_overrides", None)
        if block_mods and overrides:
            raise OLMoConfigurationError("`block_mods` and `block_overrides` cannot be used together.")
        if block_mods:
            overrides = {i: mod(block.copy()) for i, mod in block_mods.items()}
        return cls(d_model=d_model, vocab_size=vocab_size, n_layers=n_layers, block=block,
                   lm_head=LMHeadConfig(layer_norm=norm, bias=False, dtype=dtype), dtype=dtype,
                   block_overrides=overrides, **kwargs)

    @classmethod
    def llama_like_moe(
        cls,
        *,
        d_model: int,
        vocab_size: int,
        n_layers: int,
        n_heads: int,
        num_experts: int,
        top_k: int,
        expert_hidden_size: int,
        shared_expert_hidden_size: Optional[int] = None,
        dropless: bool = False,
        capacity_factor: Optional[float] = None,
        lb_loss_weight: float = 0.01,
        z_loss_weight: Optional[float] = 0.001,
        reordered_norm: bool = False,
        hybrid: bool = False,
        **kwargs,
    ) -> "TransformerConfig":
        block_name = {
            (False, False): TransformerBlockType.moe,
            (True, False): TransformerBlockType.moe_reordered_norm,
            (False, True): TransformerBlockType.moe_hybrid,
            (True, True): TransformerBlockType.moe_hybrid_reordered_norm,
        }[(reordered_norm, hybrid)]
        shared = None if shared_expert_hidden_size is None else FeedForwardConfig(hidden_size=shared_expert_hidden_size, bias=False)
        return cls.llama_like(
            d_model=d_model, vocab_size=vocab_size, n_layers=n_layers, n_heads=n_heads, name=TransformerType.moe,
            block_name=block_name, qk_norm=kwargs.pop("qk_norm", reordered_norm),
            feed_forward_moe=MoEConfig(
                name=MoEType.dropless if dropless else MoEType.default, num_experts=num_experts,
                hidden_size=expert_hidden_size, capacity_factor=capacity_factor, router=MoERouterConfig(top_k=top_k),
                shared_mlp=shared, lb_loss_weight=lb_loss_weight, z_loss_weight=z_loss_weight,
            ),
            **kwargs,
        )

    @classmethod
    def ngpt_like(cls, *, d_model: int, vocab_size: int, n_layers: int, n_heads: int, n_kv_heads: Optional[int] = None,
                  qk_norm: bool = True, rope_theta: int = 500_000, hidden_size_multiple_of: int = 256,
                  hidden_size_multiplier: Optional[float] = None, use_flash: bool = False, dtype: DType = DType.float32,
                  **kwargs) -> "TransformerConfig":
        hidden = int(8 * d_model / 3)
        if hidden_size_multiplier is not None:
            hidden = int(hidden_size_multiplier * hidden)
        hidden = ensure_multiple_of(hidden, hidden_size_multiple_of)
        block = TransformerBlockConfig(
            name=TransformerBlockType.normalized,
            sequence_mixer=AttentionConfig(
                name=AttentionType.normalized, n_heads=n_heads, n_kv_heads=n_kv_heads,
                qk_norm=LayerNormConfig(name=LayerNormType.l2_norm) if qk_norm else None,
                rope=RoPEConfig(name=RoPEType.default, theta=rope_theta), use_flash=use_flash, dtype=dtype,
            ),
            feed_forward=FeedForwardConfig(name=FeedForwardType.normalized, hidden_size=hidden, dtype=dtype),
        )
        return cls(name=TransformerType.normalized, d_model=d_model, vocab_size=vocab_size, n_layers=n_layers, block=block,
                   lm_head=LMHeadConfig(name=LMHeadType.normalized, dtype=dtype), dtype=dtype,
                   init_method=InitMethod.normalized, **kwargs)

    @classmethod
    def gemma3_like(cls, *, d_model: int, vocab_size: int, n_layers: int, n_heads: int, n_kv_heads: int, hidden_size: int,
                    head_dim: Optional[int] = None, gate: Optional[GateConfig] = None,
                    activation: ActivationFunction = ActivationFunction.gelu_tanh, local_window_size: int = 1024,
                    local_rope_theta: int = 10_000, global_rope_theta: int = 1_000_000, global_layer_interval: int = 6,
                    layer_norm_eps: float = 1e-6, fused_ops: bool = False, use_flash: Optional[bool] = None,
                    attn_backend: Optional[AttentionBackendName] = None, dtype: DType = DType.float32,
                    **kwargs) -> "TransformerConfig":
        """Gemma-3: five sliding-window layers (RoPE base 10k) per global layer (base 1M), peri-norm, GeGLU."""
        norm = LayerNormConfig(name=LayerNormType.fused_rms if fused_ops else LayerNormType.rms, eps=layer_norm_eps,
                               bias=False, dtype=dtype)

        def make_block(theta: int, window: Optional[int]) -> TransformerBlockConfig:
            sw = None
            if window is not None:
                sw = SlidingWindowAttentionConfig(pattern=[window], force_full_attention_on_first_layer=False,
                                                  force_full_attention_on_last_layer=False)
            return TransformerBlockConfig(
                name=TransformerBlockType.peri_norm,
                sequence_mixer=AttentionConfig(
                    name=AttentionType.default, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, bias=False,
                    rope=RoPEConfig(name=RoPEType.default, theta=theta), gate=gate, qk_norm=norm, use_head_qk_norm=True,
                    use_flash=use_flash, backend=attn_backend, sliding_window=sw, dtype=dtype,
                ),
                feed_forward=FeedForwardConfig(hidden_size=hidden_size, bias=False, dtype=dtype, activation=activation),
                layer_norm=norm,
            )

        return cls(
            d_model=d_model, vocab_size=vocab_size, n_layers=n_layers,
            block={"local": make_block(local_rope_theta, local_window_size), "global": make_block(global_rope_theta, None)},
            block_pattern=["local"] * (global_layer_interval - 1) + ["global"],
            lm_head=LMHeadConfig(layer_norm=norm, bias=False, dtype=dtype), dtype=dtype, embed_scale=math.sqrt(d_model),
            **kwargs,
        )

    @classmethod
    def qwen3_5_like(cls, *, d_model: int, vocab_size: int, n_layers: int, n_heads: int, n_kv_heads: int, head_dim: int,
                     intermediate_size: int, linear_num_key_heads: int = 16, linear_num_value_heads: int = 32,
                     linear_key_head_dim: int = 128, linear_value_head_dim: int = 128, linear_conv_kernel_dim: int = 4,
                     rope_theta: int = 10_000_000, partial_rotary_factor: float = 0.25, layer_norm_eps: float = 1e-6,
                     fused_ops: bool = False, use_flash: Optional[bool] = None,
                     attn_backend: Optional[AttentionBackendName] = None, dtype: DType = DType.float32,
                     **kwargs) -> "TransformerConfig":
        """Qwen-3.5 hybrid: three gated-delta-net (linear attention) layers per full-attention layer."""
        from ..attention.recurrent import GatedDeltaNetConfig

        norm = LayerNormConfig(name=LayerNormType.qwen_rms, eps=layer_norm_eps, bias=False, dtype=dtype)
        ffn = FeedForwardConfig(hidden_size=intermediate_size, bias=False, dtype=dtype)
        gdn = TransformerBlockConfig(
            name=TransformerBlockType.default,
            sequence_mixer=GatedDeltaNetConfig(
                n_heads=linear_num_key_heads, n_v_heads=linear_num_value_heads, head_dim=linear_key_head_dim,
                expand_v=linear_value_head_dim / linear_key_head_dim, allow_neg_eigval=False,
                conv_size=linear_conv_kernel_dim, norm_eps=layer_norm_eps, dtype=dtype,
            ),
            feed_forward=ffn, layer_norm=norm,
        )
        attn = TransformerBlockConfig(
            name=TransformerBlockType.default,
            sequence_mixer=AttentionConfig(
                name=AttentionType.default, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, bias=False,
                rope=RoPEConfig(name=RoPEType.default, theta=rope_theta,
                                full_precision=kwargs.pop("rope_full_precision", False),
                                partial_rotary_factor=partial_rotary_factor),
                gate=GateConfig(granularity=GateGranularity.elementwise), qk_norm=norm, use_head_qk_norm=True,
                use_flash=use_flash, backend=attn_backend, dtype=dtype,
            ),
            feed_forward=ffn, layer_norm=norm,
        )
        return cls(d_model=d_model, vocab_size=vocab_size, n_layers=n_layers, block={"gdn": gdn, "attn": attn},
                   block_pattern=["gdn", "gdn", "gdn", "attn"], lm_head=LMHeadConfig(layer_norm=norm, bias=False, dtype=dtype),
                   dtype=dtype, tie_word_embeddings=kwargs.pop("tie_word_embeddings", True), **kwargs)

    def with_rope_scaling(self, rope_scaling: RoPEScalingConfig, full_attn_layers_only: bool = True) -> "TransformerConfig":
        """Copy of this config with RoPE scaling on every layer, or only on the full-attention layers."""
        new = self.copy()
        if isinstance(new.block, dict):
            raise OLMoConfigurationError("Cannot use `with_rope_scaling` with a hybrid model with named blocks.")
        mixer = new.block.sequence_mixer
        if not isinstance(mixer, AttentionConfig) or mixer.rope is None:
            raise ValueError("Cannot apply RoPE scaling to a model without RoPE.")
        if new.block_overrides:
            raise ValueError("Cannot apply RoPE scaling when block_overrides are already set.")

        def scaled(block_cfg: TransformerBlockConfig) -> TransformerBlockConfig:
            out = block_cfg.copy()
            rope = out.sequence_mixer.rope.copy()
            rope.scaling = rope_scaling
            out.sequence_mixer.rope = rope
            return out

        if not full_attn_layers_only:
            new.block = scaled(new.block)
            return new
        sw = mixer.sliding_window
        overrides = {i: scaled(new.block) for i in range(new.n_layers) if not (sw and sw.should_use_swa(i, new.n_layers))}
        new.block_overrides = overrides or None
        return new


# ----------------------------------------------------------------------------------------------------------
# Attach one classmethod per named size.
# ----------------------------------------------------------------------------------------------------------


def _llama_size(name: str, spec: Dict[str, Any]):
    def factory(cls, vocab_size: int, **kwargs) -> TransformerConfig:
        args = dict(spec["fixed"])
        for key, default in spec["defaults"].items():
            args[key] = kwargs.pop(key, default)
        ffn = args.pop("ffn", None)
        if ffn is not None:  # Qwen-3: explicit MLP width, Qwen RMSNorm, eps 1e-6
            args.update(feed_forward=FeedForwardConfig(hidden_size=ffn, bias=False, dtype=kwargs.get("dtype", DType.float32)),
                        layer_norm_name=LayerNormType.qwen_rms, layer_norm_eps=1e-6)
        return cls.llama_like(vocab_size=vocab_size, **args, **kwargs)

    factory.__name__ = name
    factory.__doc__ = f"The ``{name}`` configuration (see :data:`MODEL_SIZES`)."
    return classmethod(factory)


def _olmo3_size(name: str, base: str):
    def factory(cls, vocab_size: int, **kwargs) -> TransformerConfig:
        kwargs.setdefault("sliding_window", _sliding_window_default())
        kwargs.setdefault("attn_backend", AttentionBackendName.flash_2)
        if name == "olmo3_600M":
            kwargs.setdefault("d_model", 1280)
        return getattr(cls, base)(vocab_size, **kwargs)

    factory.__name__ = name
    factory.__doc__ = f"``{base}`` with sliding-window attention (4096) in three of every four layers."
    return classmethod(factory)


def _gemma3_size(name: str, dims):
    d_model, n_layers, n_heads, n_kv_heads, hidden = dims

    def factory(cls, vocab_size: int = 262208, **kwargs) -> TransformerConfig:
        return cls.gemma3_like(d_model=d_model, vocab_size=vocab_size, n_layers=kwargs.pop("n_layers", n_layers),
                               n_heads=kwargs.pop("n_heads", n_heads), n_kv_heads=kwargs.pop("n_kv_heads", n_kv_heads),
                               hidden_size=kwargs.pop("hidden_size", hidden), **kwargs)

    factory.__name__ = name
    return classmethod(factory)


def _qwen3_5_size(name: str, dims):
    d_model, n_layers, n_heads, n_kv_heads, inter, lk, lv = dims

    def factory(cls, vocab_size: int, **kwargs) -> TransformerConfig:
        return cls.qwen3_5_like(
            d_model=d_model, vocab_size=vocab_size, n_layers=kwargs.pop("n_layers", n_layers),
            n_heads=kwargs.pop("n_heads", n_heads), n_kv_heads=kwargs.pop("n_kv_heads", n_kv_heads),
            head_dim=kwargs.pop("head_dim", 256), intermediate_size=kwargs.pop("intermediate_size", inter),
            linear_num_key_heads=kwargs.pop("linear_num_key_heads", lk),
            linear_num_value_heads=kwargs.pop("linear_num_value_heads", lv), **kwargs)

    factory.__name__ = name
    return classmethod(factory)


def _moe_size(name: str, spec: Dict[str, Any]):
    def factory(cls, vocab_size: int, **kwargs) -> TransformerConfig:
        d_model = kwargs.pop("d_model", spec["d_model"])
        moe = MoEConfig(
            name=spec["moe"], num_experts=spec["experts"], hidden_size=int(0.5 * d_model),
            router=MoERouterConfig(top_k=spec["top_k"]),
            shared_mlp=FeedForwardConfig(hidden_size=d_model * 2) if spec["shared"] else None,
            lb_loss_weight=0.01, z_loss_weight=0.001,
        )
        extra = dict(feed_forward=FeedForwardConfig(hidden_size=d_model * 2, bias=False)) if spec["dense"] else {}
        return cls.llama_like(
            d_model=d_model, vocab_size=vocab_size, n_layers=kwargs.pop("n_layers", spec["n_layers"]),
            n_heads=kwargs.pop("n_heads", spec["n_heads"]), name=kwargs.pop("name", TransformerType.moe),
            block_name=kwargs.pop("block_name", spec["block"]), qk_norm=kwargs.pop("qk_norm", True),
            rope_theta=kwargs.pop("rope_theta", 500_000), layer_norm_eps=1e-6, feed_forward_moe=moe, **extra, **kwargs)

    factory.__name__ = name
    return classmethod(factory)


def _ngpt_size(name: str, d_model: int, n_layers: int, n_heads: int):
    def factory(cls, vocab_size: int, **kwargs) -> TransformerConfig:
        return cls.ngpt_like(d_model=d_model, vocab_size=vocab_size, n_layers=kwargs.pop("n_layers", n_layers),
                             n_heads=kwargs.pop("n_heads", n_heads), **kwargs)

    factory.__name__ = name
    return classmethod(factory)


for _name, _spec in MODEL_SIZES.items():
    setattr(TransformerConfig, _name, _llama_size(_name, _spec))
for _name, _base in _OLMO3_BASE.items():
    setattr(TransformerConfig, _name, _olmo3_size(_name, _base))
for _name, _dims in _GEMMA3.items():
    setattr(TransformerConfig, _name, _gemma3_size(_name, _dims))
for _name, _dims in _QWEN3_5.items():
    setattr(TransformerConfig, _name, _qwen3_5_size(_name, _dims))
for _name, _spec in _MOE.items():
    setattr(TransformerConfig, _name, _moe_size(_name, _spec))
setattr(TransformerConfig, "ngpt_271M", _ngpt_size("ngpt_271M", 1024, 16, 16))
setattr(TransformerConfig, "ngpt_1B", _ngpt_size("ngpt_1B", 2048, 18, 16))
