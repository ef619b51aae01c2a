"""
Transformer blocks (class names and forward semantics of src/olmo_core/nn/transformer/block.py:96-1095).

Nine variants: pre-norm (``default``), pre-norm with LayerNorm scaling, OLMo-2's ``reordered_norm`` (norm on
the *output* of attention / MLP), ``peri_norm`` (norm on both sides), nGPT ``normalized``, and the MoE
versions (``moe``, ``moe_reordered_norm``, ``moe_hybrid``, ``moe_hybrid_reordered_norm``).

For the reordered-norm block the residual add is fused into the RMSNorm kernel
(``h = x + norm(f(x))`` is one pass over memory), which is the hot configuration of the OLMo-2/3 models.
"""

from __future__ import annotations

import math
from abc import abstractmethod
from typing import Dict, Optional, Tuple, Union

import torch
import torch.nn as nn

from ...doc_utils import beta_feature
from ..attention import RingContextParallelStyle, SequenceMixerConfig, UlyssesContextParallelStyle
from ..buffer_cache import BufferCache
from ..feed_forward import FeedForwardConfig
from ..layer_norm import LayerNormConfig, RMSNorm, l2_normalize
from ..moe import MoEConfig
from ..residual_stream import ResidualStream

__all__ = [
    "TransformerBlockBase",
    "TransformerBlock",
    "LayerNormScaledTransformerBlock",
    "ReorderedNormTransformerBlock",
    "PeriNormTransformerBlock",
    "NormalizedTransformerBlock",
    "MoETransformerBlock",
    "MoEReorderedNormTransformerBlock",
    "MoEHybridTransformerBlockBase",
    "MoEHybridTransformerBlock",
    "MoEHybridReorderedNormTransformerBlock",
]


def _post_norm_residual(norm: nn.Module, y: torch.Tensor, x: torch.Tensor, stream: Optional[ResidualStream],
                        training: bool) -> torch.Tensor:
    """``x + norm(y)`` using the fused kernel when the norm and the residual stream allow it."""
    plain = stream is None or (stream.alpha == 1.0 and (stream.dropout == 0.0 or not training))
    if plain and isinstance(norm, RMSNorm) and type(norm).forward is RMSNorm.forward:
        return norm(y, residual=x)
    normed = norm(y)
    return x + normed if stream is None else stream(x, normed)


class TransformerBlockBase(nn.Module):
    """Common interface of all block types."""

    def __init__(self, *, n_layers: int):
        super().__init__()
        self.n_layers = n_layers
        self.block_idx = 0

    @abstractmethod
    def forward(self, x: torch.Tensor, *, loss_div_factor: Optional[Union[torch.Tensor, float]] = None, **kwargs) -> torch.Tensor:
        raise NotImplementedError

    def apply_pp(self, pp_mesh) -> None:
        """A block has nothing of its own to set up for pipeline parallelism
        (src/olmo_core/nn/transformer/block.py:60-61)."""
        del pp_mesh

    def apply_tp(self, tp_mesh, *, input_layout=None, float8_enabled: bool = False) -> None:
        from ...parallel.tensor import shard_block_

        shard_block_(self, tp_mesh)

    def apply_cp(self, cp_mesh, ring: Optional[RingContextParallelStyle] = None,
                 uly: Optional[UlyssesContextParallelStyle] = None) -> None:
        self.attention.apply_cp(cp_mesh, ring=ring, uly=uly)  # type: ignore[attr-defined]

    def apply_fsdp(self, *args, **kwargs) -> None:
        """Parameter sharding is applied to the whole model by ``olmo_core_b200.parallel.fsdp``."""

    def apply_compile(self) -> None:
        """No tracing compiler on the GPU path: fusions are explicit kernels."""

    def num_flops_per_token(self, seq_len: int) -> int:
        n = self.attention.num_flops_per_token(seq_len)  # type: ignore[attr-defined]
        for name in ("feed_forward", "feed_forward_moe"):
            m = getattr(self, name, None)
            if m is not None:
                n += m.num_flops_per_token(seq_len)
        return n

    @property
    def is_moe(self) -> bool:
        return False


class TransformerBlock(TransformerBlockBase):
    """Pre-norm block: ``h = x + attn(norm(x)); out = h + mlp(norm(h))``."""

    def __init__(
        self,
        *,
        d_model: int,
        block_idx: int,
        n_layers: int,
        sequence_mixer: SequenceMixerConfig,
        feed_forward: FeedForwardConfig,
        layer_norm: LayerNormConfig,
        dropout: float = 0.0,
        attention_residual_alpha: float = 1.0,
        feed_forward_residual_alpha: float = 1.0,
        init_device: str = "cpu",
        cache: Optional[BufferCache] = None,
    ):
        super().__init__(n_layers=n_layers)
        self.d_model = d_model
        self.block_idx = block_idx
        # The attribute keeps the name ``attention`` whatever the mixer type, so checkpoint keys are stable.
        self.attention = sequence_mixer.build(d_model, layer_idx=block_idx, n_layers=n_layers, init_device=init_device,
                                              cache=cache)
        self.attention_norm = layer_norm.build(d_model, init_device=init_device)
        self.attention_residual_stream = ResidualStream(alpha=attention_residual_alpha, dropout=dropout)
        self.feed_forward = feed_forward.build(d_model=d_model, init_device=init_device)
        self.feed_forward_norm = layer_norm.build(d_model, init_device=init_device)
        self.feed_forward_residual_stream = ResidualStream(alpha=feed_forward_residual_alpha, dropout=dropout)

    def forward(self, x, *, loss_div_factor=None, **kwargs):
        h = self.attention_residual_stream(x, self.attention(self.attention_norm(x), **kwargs))
        return self.feed_forward_residual_stream(h, self.feed_forward(self.feed_forward_norm(h)))


class LayerNormScaledTransformerBlock(TransformerBlock):
    """Pre-norm block whose norm outputs are scaled by ``1/sqrt(layer index + 1)`` (LayerNorm Scaling)."""

    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self.register_buffer("ln_scale", torch.tensor(1.0 / math.sqrt(self.block_idx + 1), dtype=torch.float32))

    def forward(self, x, *, loss_div_factor=None, **kwargs):
        s = self.ln_scale.to(dtype=x.dtype, device=x.device)
        h = self.attention_residual_stream(x, self.attention(self.attention_norm(x) * s, **kwargs))
        return self.feed_forward_residual_stream(h, self.feed_forward(self.feed_forward_norm(h) * s))


class ReorderedNormTransformerBlock(TransformerBlock):
    """OLMo-2 block: ``h = x + norm(attn(x)); out = h + norm(mlp(h))``."""

    def forward(self, x, *, loss_div_factor=None, **kwargs):
        h = _post_norm_residual(self.attention_norm, self.attention(x, **kwargs), x, self.attention_residual_stream,
                                self.training)
        return _post_norm_residual(self.feed_forward_norm, self.feed_forward(h), h, self.feed_forward_residual_stream,
                                   self.training)


class PeriNormTransformerBlock(TransformerBlock):
    """Peri-LN: norms on both the input and the output of each sub-layer (Gemma-3 style)."""

    def __init__(self, *, d_model: int, layer_norm: LayerNormConfig, init_device: str = "cpu", **kwargs):
        super().__init__(d_model=d_model, layer_norm=layer_norm, init_device=init_device, **kwargs)
        self.post_attention_norm = layer_norm.build(d_model, init_device=init_device)
        self.post_feed_forward_norm = layer_norm.build(d_model, init_device=init_device)

    def forward(self, x, *, loss_div_factor=None, **kwargs):
        h = _post_norm_residual(self.post_attention_norm, self.attention(self.attention_norm(x), **kwargs), x,
                                self.attention_residual_stream, self.training)
        return _post_norm_residual(self.post_feed_forward_norm, self.feed_forward(self.feed_forward_norm(h)), h,
                                   self.feed_forward_residual_stream, self.training)


@beta_feature
class NormalizedTransformerBlock(TransformerBlockBase):
    """nGPT block: hidden states stay on the unit sphere; sub-layer outputs are blended in with learned rates."""

    def __init__(self, *, d_model: int, block_idx: int, n_layers: int, sequence_mixer: SequenceMixerConfig,
                 feed_forward: FeedForwardConfig, init_device: str = "cpu", cache: Optional[BufferCache] = None):
        super().__init__(n_layers=n_layers)
        self.d_model = d_model
        self.block_idx = block_idx
        self.attention = sequence_mixer.build(d_model, layer_idx=block_idx, n_layers=n_layers, init_device=init_device,
                                              cache=cache)
        self.feed_forward = feed_forward.build(d_model=d_model, init_device=init_device)
        self.attn_alpha_init_value = 0.05
        self.attn_alpha_init_scaling = 1.0 / math.sqrt(d_model)
        self.attn_alpha = nn.Parameter(torch.empty(d_model, dtype=torch.float32, device=init_device))
        self.mlp_alpha_init_value = 0.05
        self.mlp_alpha_init_scaling = 1.0 / math.sqrt(d_model)
        self.mlp_alpha = nn.Parameter(torch.empty(d_model, dtype=torch.float32, device=init_device))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.attn_alpha.device.type != "meta":
            with torch.no_grad():
                self.attn_alpha.fill_(self.attn_alpha_init_scaling)
                self.mlp_alpha.fill_(self.mlp_alpha_init_scaling)

    def forward(self, x, *, loss_div_factor=None, **kwargs):
        a = (self.attn_alpha * (self.attn_alpha_init_value / self.attn_alpha_init_scaling)).abs().to(x.dtype)
        h = l2_normalize(torch.lerp(x, l2_normalize(self.attention(x, **kwargs)), a))
        m = (self.mlp_alpha * (self.mlp_alpha_init_value / self.mlp_alpha_init_scaling)).abs().to(x.dtype)
        return l2_normalize(torch.lerp(h, l2_normalize(self.feed_forward(h)), m))

    def apply_tp(self, tp_mesh, **kwargs) -> None:
        raise NotImplementedError("TP is not implemented yet for the normalized transformer block variant")

    @torch.no_grad()
    def normalize_matrices(self) -> None:
        for m in (self.attention, self.feed_forward):
            if hasattr(m, "normalize_matrices"):
                m.normalize_matrices()


@beta_feature
class MoETransformerBlock(TransformerBlockBase):
    """Pre-norm block with a mixture-of-experts feed-forward."""

    def __init__(self, *, d_model: int, block_idx: int, n_layers: int, sequence_mixer: SequenceMixerConfig,
                 feed_forward_moe: MoEConfig, layer_norm: LayerNormConfig, dropout: float = 0.0,
                 init_device: str = "cpu", cache: Optional[BufferCache] = None):
        super().__init__(n_layers=n_layers)
        self.d_model = d_model
        self.block_idx = block_idx
        self.attention = sequence_mixer.build(d_model, layer_idx=block_idx, n_layers=n_layers, init_device=init_device,
                                              cache=cache)
        self.attention_norm = layer_norm.build(d_model, init_device=init_device)
        self.feed_forward_moe = feed_forward_moe.build(d_model=d_model, n_layers=n_layers, init_device=init_device,
                                                       cache=cache)
        self.feed_forward_norm = layer_norm.build(d_model, init_device=init_device)
        self.dropout = nn.Dropout(dropout) if dropout > 0.0 else nn.Identity()
        self._ep_enabled = False
        self._tp_enabled = False

    @property
    def is_moe(self) -> bool:
        return True

    @property
    def router(self):
        return self.feed_forward_moe.router

    @property
    def shared_mlp(self):
        return self.feed_forward_moe.shared_mlp

    @property
    def experts(self):
        return self.feed_forward_moe.experts

    @property
    def top_k(self) -> int:
        return self.feed_forward_moe.top_k

    @property
    def ep_enabled(self) -> bool:
        return self._ep_enabled

    @property
    def tp_enabled(self) -> bool:
        return self._tp_enabled

    def compute_metrics(self, reset: bool = True) -> Dict[str, Tuple[torch.Tensor, Optional[object]]]:
        return self.feed_forward_moe.compute_metrics(reset=reset)

    def reset_metrics(self) -> None:
        self.feed_forward_moe.reset_metrics()

    def post_batch(self, dry_run: bool = False) -> None:
        self.feed_forward_moe.post_batch(dry_run=dry_run)

    def forward(self, x, *, loss_div_factor=None, **kwargs):
        h = x + self.dropout(self.attention(self.attention_norm(x), **kwargs))
        return h + self.dropout(self.feed_forward_moe(self.feed_forward_norm(h), loss_div_factor=loss_div_factor))

    def apply_pp(self, pp_mesh) -> None:
        self.feed_forward_moe.apply_pp(pp_mesh)

    def apply_ep(self, ep_mesh, **kwargs) -> None:
        self.feed_forward_moe.apply_ep(ep_mesh, **kwargs)
        self._ep_enabled = True

    def apply_tp(self, tp_mesh, **kwargs) -> None:
        super().apply_tp(tp_mesh, **kwargs)
        self._tp_enabled = True

    def apply_cp(self, cp_mesh, ring=None, uly=None) -> None:
        self.attention.apply_cp(cp_mesh, ring=ring, uly=uly)
        self.feed_forward_moe.apply_cp(cp_mesh)


@beta_feature
class MoEReorderedNormTransformerBlock(MoETransformerBlock):
    """OLMoE block: norms on the outputs of attention and of the MoE."""

    def forward(self, x, *, loss_div_factor=None, **kwargs):
        drop = isinstance(self.dropout, nn.Dropout) and self.training
        att = self.attention(x, **kwargs)
        if drop:
            h = x + self.dropout(self.attention_norm(att))
            return h + self.dropout(self.feed_forward_norm(self.feed_forward_moe(h, loss_div_factor=loss_div_factor)))
        h = _post_norm_residual(self.attention_norm, att, x, None, self.training)
        return _post_norm_residual(self.feed_forward_norm, self.feed_forward_moe(h, loss_div_factor=loss_div_factor), h,
                                   None, self.training)


@beta_feature
class MoEHybridTransformerBlockBase(MoETransformerBlock):
    """Blocks that run a dense MLP and an MoE side by side: ``out = dense(x) + sparse(x)``."""

    def __init__(self, *, d_model: int, block_idx: int, n_layers: int, sequence_mixer: SequenceMixerConfig,
                 feed_forward_moe: MoEConfig, feed_forward: FeedForwardConfig, layer_norm: LayerNormConfig,
                 dropout: float = 0.0, init_device: str = "cpu", cache: Optional[BufferCache] = None):
        super().__init__(d_model=d_model, block_idx=block_idx, n_layers=n_layers, sequence_mixer=sequence_mixer,
                         feed_forward_moe=feed_forward_moe, layer_norm=layer_norm, dropout=dropout,
                         init_device=init_device, cache=cache)
        self.feed_forward = feed_forward.build(d_model=d_model, init_device=init_device)
        self.feed_forward_moe_norm = layer_norm.build(d_model, init_device=init_device)
        self._use_combined_forward: Optional[bool] = None

    @property
    def use_combined_forward(self) -> bool:
        """Whether the sparse branch runs on a side stream beside the dense branch. Unless set, it follows whether
        the experts are partitioned over ranks (src/olmo_core/nn/transformer/block.py:744-759)."""
        if self._use_combined_forward is not None:
            return self._use_combined_forward
        return bool(getattr(self, "_ep_enabled", False) or getattr(self, "_tp_enabled", False))

    @use_combined_forward.setter
    def use_combined_forward(self, should_use: bool) -> None:
        if should_use and not (getattr(self, "_ep_enabled", False) or getattr(self, "_tp_enabled", False)):
            raise RuntimeError("combined forward can only be used when expert parallelism is enabled")
        self._use_combined_forward = should_use

    @abstractmethod
    def dense_forward(self, x: torch.Tensor, **kwargs) -> torch.Tensor:
        raise NotImplementedError

    @abstractmethod
    def sparse_forward(self, x: torch.Tensor, *, loss_div_factor=None) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, x, *, loss_div_factor=None, **kwargs):
        if self.use_combined_forward and x.is_cuda:
            return self.combined_forward(x, loss_div_factor=loss_div_factor, **kwargs)
        return self.sparse_forward(x, loss_div_factor=loss_div_factor) + self.dense_forward(x, **kwargs)

    def combined_forward(self, x, *, loss_div_factor=None, **kwargs):
        """Run the sparse branch on a side stream so its all-to-alls overlap the dense branch."""
        from ...utils import get_or_init_stream

        side = get_or_init_stream("moe_sparse")
        cur = torch.cuda.current_stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            sparse = self.sparse_forward(x, loss_div_factor=loss_div_factor)
        dense = self.dense_forward(x, **kwargs)
        cur.wait_stream(side)
        sparse.record_stream(cur)
        return sparse + dense

@beta_feature
class MoEHybridTransformerBlock(MoEHybridTransformerBlockBase):
    def dense_forward(self, x, **kwargs):
        h = x + self.dropout(self.attention(self.attention_norm(x), **kwargs))
        return h + self.dropout(self.feed_forward(self.feed_forward_norm(h)))

    def sparse_forward(self, x, *, loss_div_factor=None):
        return self.dropout(self.feed_forward_moe(self.feed_forward_moe_norm(x), loss_div_factor=loss_div_factor))


@beta_feature
class MoEHybridReorderedNormTransformerBlock(MoEHybridTransformerBlockBase):
    def dense_forward(self, x, **kwargs):
        h = x + self.dropout(self.attention_norm(self.attention(x, **kwargs)))
        return h + self.dropout(self.feed_forward_norm(self.feed_forward(h)))

    def sparse_forward(self, x, *, loss_div_factor=None):
        return self.dropout(self.feed_forward_moe_norm(self.feed_forward_moe(x, loss_div_factor=loss_div_factor)))
