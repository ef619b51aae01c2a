"""
Attention modules and their config (API of src/olmo_core/nn/attention/__init__.py:55-1159).

Data flow of :class:`Attention` on CUDA: three tcgen05 GEMMs (``w_q``, ``w_k``, ``w_v``) -> one fused
kernel per tensor that applies the QK-norm and the rotary embedding in a single pass -> the flash
attention kernel on ``[B, T, H, D]`` views (no transposes) -> optional sigmoid gate -> ``w_out`` GEMM.
On CPU the same module runs the PyTorch statements of each step.
"""

from __future__ import annotations

import logging
import math
from abc import abstractmethod
from dataclasses import dataclass
from typing import Generic, List, Optional, Tuple, TypeVar

import torch
import torch.nn as nn

from ...config import Config, DType, Registrable, StrEnum
from ...exceptions import OLMoConfigurationError
from ...ops.elementwise import NORM_FULL, NORM_HEAD, NORM_NONE, norm_rope
from ...ops.gemm import multi_linear
from ..buffer_cache import BufferCache
from ..config import ModuleConfig
from ..feed_forward import Linear
from ..layer_norm import LayerNorm, LayerNormConfig, RMSNorm, QwenRMSNorm, l2_normalize
from ..rope import ComplexRotaryEmbedding, RoPEConfig, RotaryEmbedding, RotaryEmbeddingBase
from .backend import (
    AttentionBackend,
    AttentionBackendName,
    FlashAttention2Backend,
    FlashAttention3Backend,
    FlashAttention4Backend,
    KernelAttentionBackend,
    TEAttentionBackend,
    TorchAttentionBackend,
)
from .base import SeqMixer, SequenceMixer, SequenceMixerConfig
from .kv_cache import KVCacheManager
from .recurrent import GatedDeltaNet, GatedDeltaNetConfig
from .ring import (
    RingAttentionLlama3LoadBalancer,
    RingAttentionLoadBalancer,
    RingAttentionLoadBalancerType,
    RingAttentionZigZagLoadBalancer,
    RingContextParallelStyle,
    UlyssesContextParallelStyle,
    UlyssesLoadBalancer,
)

__all__ = [
    "GatedDeltaNet",
    "GatedDeltaNetConfig",
    "SequenceMixer",
    "SequenceMixerConfig",
    "SlidingWindowAttentionConfig",
    "GateGranularity",
    "GateConfig",
    "AttentionType",
    "AttentionBackendName",
    "AttentionBackend",
    "TorchAttentionBackend",
    "KernelAttentionBackend",
    "FlashAttention2Backend",
    "FlashAttention3Backend",
    "FlashAttention4Backend",
    "TEAttentionBackend",
    "AttentionConfig",
    "Attention",
    "FusedAttention",
    "NormalizedAttention",
    "KVCacheManager",
    "RingAttentionLoadBalancerType",
    "RingAttentionLoadBalancer",
    "RingAttentionZigZagLoadBalancer",
    "RingAttentionLlama3LoadBalancer",
    "UlyssesLoadBalancer",
    "RingContextParallelStyle",
    "UlyssesContextParallelStyle",
]

log = logging.getLogger(__name__)


class GateGranularity(StrEnum):
    headwise = "headwise"
    elementwise = "elementwise"


@dataclass
class GateConfig(Config):
    granularity: GateGranularity = GateGranularity.headwise
    full_precision: bool = True


@dataclass
class SlidingWindowAttentionConfig(Config):
    """``pattern`` of window sizes repeated over the layers; -1 means full attention."""

    pattern: List[int]
    force_full_attention_on_first_layer: bool = True
    force_full_attention_on_last_layer: bool = True

    def _get_window_size(self, layer_idx: int, n_layers: int) -> int:
        if self.force_full_attention_on_first_layer and layer_idx == 0:
            return -1
        if self.force_full_attention_on_last_layer and layer_idx == n_layers - 1:
            return -1
        idx = layer_idx - 1 if self.force_full_attention_on_first_layer else layer_idx
        w = self.pattern[idx % len(self.pattern)]
        if w <= 0 and w != -1:
            raise OLMoConfigurationError(f"Sliding window size must be positive or -1 (got {w})")
        return w

    def should_use_swa(self, layer_idx: int, n_layers: int) -> bool:
        return self._get_window_size(layer_idx, n_layers) != -1

    def get_window_size(self, layer_idx: int, n_layers: int) -> int:
        w = self._get_window_size(layer_idx, n_layers)
        if w == -1:
            raise ValueError(f"Layer {layer_idx} is not configured for sliding window attention.")
        return w


class AttentionType(StrEnum):
    default = "default"
    fused = "fused"
    normalized = "normalized"


@SequenceMixerConfig.register("attention")
@dataclass
class AttentionConfig(SequenceMixerConfig["SequenceMixer"]):
    name: AttentionType = AttentionType.default
    n_heads: int = 16
    n_kv_heads: Optional[int] = None
    head_dim: Optional[int] = None
    bias: Optional[bool] = None
    gate: Optional[GateConfig] = None
    rope: Optional[RoPEConfig] = None
    clip_qkv: Optional[float] = None
    qk_norm: Optional[LayerNormConfig] = None
    dropout: Optional[float] = None
    use_flash: Optional[bool] = None
    backend: Optional[AttentionBackendName] = None
    dtype: DType = DType.float32
    sliding_window: Optional[SlidingWindowAttentionConfig] = None
    use_head_qk_norm: Optional[bool] = None

    def num_params(self, d_model: int) -> int:
        H = self.n_heads
        Hkv = self.n_kv_heads or H
        hd = self.head_dim or d_model // H
        bias = self.bias if self.bias is not None else self.name != AttentionType.normalized
        n = d_model * H * hd + 2 * d_model * Hkv * hd + H * hd * d_model
        if bias:
            n += H * hd + 2 * Hkv * hd + d_model
        if self.qk_norm is not None:
            if self.use_head_qk_norm:
                n += 2 * self.qk_norm.num_params(hd)
            else:
                n += self.qk_norm.num_params(H * hd) + self.qk_norm.num_params(Hkv * hd)
        if self.gate is not None:
            width = H if self.gate.granularity == GateGranularity.headwise else H * hd
            n += d_model * width + (width if bias else 0)
        if self.name == AttentionType.normalized:
            n += H * hd + Hkv * hd
        return n

    def build(self, d_model: int, *, layer_idx: int, n_layers: int, init_device: str = "cpu",
              cache: Optional[BufferCache] = None) -> "SequenceMixer":
        kwargs = self.as_dict(exclude_none=True, recurse=False)
        kwargs.pop("name")
        sw: Optional[SlidingWindowAttentionConfig] = kwargs.pop("sliding_window", None)
        if sw is not None and sw.should_use_swa(layer_idx, n_layers):
            kwargs["window_size"] = sw.get_window_size(layer_idx, n_layers)
        else:
            rope_cfg = kwargs.get("rope")
            if rope_cfg is not None and rope_cfg.no_global_rope:
                kwargs["rope"] = None
        kwargs.update(dtype=DType(kwargs.pop("dtype")).as_pt(), d_model=d_model, init_device=init_device, cache=cache)
        try:
            if self.name == AttentionType.default:
                return Attention(**kwargs)
            if self.name == AttentionType.fused:
                kwargs.pop("use_flash", None)
                if "window_size" in kwargs:
                    raise OLMoConfigurationError("'window_size' is not supported with fused attention")
                return FusedAttention(**kwargs)
            if self.name == AttentionType.normalized:
                if "window_size" in kwargs:
                    raise OLMoConfigurationError("'window_size' is not supported with normalized attention")
                return NormalizedAttention(**kwargs)
            raise NotImplementedError(self.name)
        except TypeError as e:
            raise OLMoConfigurationError(f"invalid options for '{self.name}' {self.__class__.__name__}, {e}") from e


def _pick_backend(backend: Optional[AttentionBackendName], use_flash: Optional[bool]) -> AttentionBackendName:
    if backend is not None:
        return AttentionBackendName(backend)
    if use_flash:
        return AttentionBackendName.flash_2
    # The kernel backend handles CPU tensors through the reference math, so it is a safe default.
    return AttentionBackendName.flash_2 if torch.cuda.is_available() else AttentionBackendName.torch


class Attention(SequenceMixer):
    """Multi-head / grouped-query self-attention with optional QK-norm, RoPE, sliding window and gate."""

    def __init__(
        self,
        *,
        d_model: int,
        n_heads: int,
        n_kv_heads: Optional[int] = None,
        head_dim: Optional[int] = None,
        bias: bool = True,
        gate: Optional[GateConfig] = None,
        rope: Optional[RoPEConfig] = None,
        clip_qkv: Optional[float] = None,
        qk_norm: Optional[LayerNormConfig] = None,
        dropout: float = 0.0,
        softmax_scale: Optional[float] = None,
        use_flash: Optional[bool] = None,
        backend: Optional[AttentionBackendName] = None,
        window_size: Optional[int] = None,
        dtype: torch.dtype = torch.float32,
        init_device: str = "cpu",
        cache: Optional[BufferCache] = None,
        use_head_qk_norm: bool = False,
    ):
        super().__init__()
        self.d_model = d_model
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads or n_heads
        self.head_dim = head_dim if head_dim is not None else d_model // n_heads
        hd = self.head_dim
        self.w_q = Linear(d_model, n_heads * hd, bias, dtype, init_device)
        self.w_k = Linear(d_model, self.n_kv_heads * hd, bias, dtype, init_device)
        self.w_v = Linear(d_model, self.n_kv_heads * hd, bias, dtype, init_device)
        self.w_out = Linear(n_heads * hd, d_model, bias, dtype, init_device)
        self.gate = gate
        self.w_g: Optional[Linear] = None
        if gate is not None:
            width = n_heads if gate.granularity == GateGranularity.headwise else n_heads * hd
            self.w_g = Linear(d_model, width, bias, dtype, init_device)
        self.clip_qkv = clip_qkv
        self.use_head_qk_norm = use_head_qk_norm
        self.q_norm: Optional[LayerNorm] = None
        self.k_norm: Optional[LayerNorm] = None
        if qk_norm is not None:
            if use_head_qk_norm:
                self.q_norm = qk_norm.build(size=hd, init_device=init_device)
                self.k_norm = qk_norm.build(size=hd, init_device=init_device)
            else:
                self.q_norm = qk_norm.build(size=n_heads * hd, init_device=init_device)
                self.k_norm = qk_norm.build(size=self.n_kv_heads * hd, init_device=init_device)
        self.rope: Optional[RotaryEmbeddingBase] = None
        if rope is not None:
            if rope.name == "fused":
                raise OLMoConfigurationError("fused RoPE is only meant for the fused attention module")
            self.rope = rope.build(hd, cache=cache)
        self.dropout_p = dropout
        self.window_size = window_size
        if window_size is not None and window_size <= 0:
            raise OLMoConfigurationError(f"'window_size' must be positive (got {window_size})")
        self.backend_name = _pick_backend(backend, use_flash)
        self.backend = self.backend_name.build(
            head_dim=hd,
            n_heads=n_heads,
            n_kv_heads=self.n_kv_heads,
            scale=softmax_scale,
            dropout_p=dropout,
            window_size=(window_size - 1, 0) if window_size is not None else (-1, -1),
        )
        self.kv_cache_manager: Optional[KVCacheManager] = None
        self.tp_group = None
        self._cp_enabled = False

    # -- properties ----------------------------------------------------------------------------------
    @property
    def cp_enabled(self) -> bool:
        return self._cp_enabled

    @property
    def tp_enabled(self) -> bool:
        return self.tp_group is not None

    # -- fused QK-norm + RoPE -------------------------------------------------------------------------
    def _fusable(self, x: torch.Tensor, start_pos, freqs_cis) -> bool:
        if not x.is_cuda or freqs_cis is not None or self.clip_qkv is not None or self.tp_enabled:
            return False
        if self.rope is None or not isinstance(self.rope, RotaryEmbedding) or self.rope.rotary_dim != self.head_dim:
            return False
        if not self.rope.full_precision:
            return False
        for n in (self.q_norm, self.k_norm):
            if n is not None and (not isinstance(n, RMSNorm) or isinstance(n, QwenRMSNorm) or n.bias is not None
                                  or n.weight is None or not n.full_precision):
                return False
        return (self.q_norm is None) == (self.k_norm is None)

    def _norm_rope_fused(self, q, k, T, start_pos, pos_sin, pos_cos, cu_doc_lens, rope_pos_ids=None):
        assert isinstance(self.rope, RotaryEmbedding)
        offset = int(start_pos) if start_pos is not None else 0
        if pos_sin is None or pos_cos is None:
            need = offset + T if rope_pos_ids is None else int(getattr(self, "_rope_table_len", None) or offset + T)
            bufs = self.rope.get_buffers(need, q.device)
            pos_sin, pos_cos = bufs.pos_sin, bufs.pos_cos
        pos_ids = None
        if rope_pos_ids is not None:
            pos_ids = rope_pos_ids.reshape(-1).to(device=q.device, dtype=torch.int32)
        elif cu_doc_lens is not None:
            flat = torch.arange(q.shape[0] * T, device=q.device, dtype=cu_doc_lens.dtype)
            doc = torch.bucketize(flat, cu_doc_lens[1:], right=True)
            pos_ids = (flat - cu_doc_lens[doc]).to(torch.int32)
        mode = NORM_NONE if self.q_norm is None else (NORM_HEAD if self.use_head_qk_norm else NORM_FULL)
        eps = self.q_norm.eps if self.q_norm is not None else 0.0
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        q = norm_rope(q, qw, pos_sin, pos_cos, q.shape[-1] // self.head_dim, eps, mode, pos_ids, offset)
        k = norm_rope(k, kw, pos_sin, pos_cos, k.shape[-1] // self.head_dim, eps, mode, pos_ids, offset)
        return q, k

    def forward(
        self,
        x: torch.Tensor,
        cu_doc_lens: Optional[torch.Tensor] = None,
        cu_doc_lens_q: Optional[torch.Tensor] = None,
        cu_doc_lens_k: Optional[torch.Tensor] = None,
        max_doc_len: Optional[int] = None,
        max_doc_len_q: Optional[int] = None,
        max_doc_len_k: Optional[int] = None,
        local_k_slice: Optional[slice] = None,
        pos_sin: Optional[torch.Tensor] = None,
        pos_cos: Optional[torch.Tensor] = None,
        freqs_cis: Optional[torch.Tensor] = None,
        cache_leftpad: Optional[torch.Tensor] = None,
        rope_pos_ids: Optional[torch.Tensor] = None,
        rope_table_len: Optional[int] = None,
    ) -> torch.Tensor:
        """
        ``rope_pos_ids`` (int ``[B, T]``) gives the rotary position of every token explicitly; a context-parallel shard of
        packed documents needs it (positions restart per document and the shard is not a contiguous range), together
        with ``rope_table_len``, the length of the whole sequence.
        """
        B, T, _ = x.shape
        hd = self.head_dim
        tp_fused = getattr(self, "_tp_fused_call", False)
        if tp_fused:
            # x is this rank's SEQUENCE shard: the projections gather the other shards inside their GEMMs
            q, k, v = self._tp_project_in(x)
            T = q.shape[1]
        else:
            q, k, v = multi_linear(x, (self.w_q, self.w_k, self.w_v))
        start_pos = self.kv_cache_manager.current_position() if self.kv_cache_manager is not None else None
        if (self.cp_enabled and self.rope is not None and pos_sin is None and pos_cos is None and freqs_cis is None
                and rope_pos_ids is None):
            raise RuntimeError("RoPE buffers must be passed to attention after being sharded by the context-parallel load balancer")
        self._rope_table_len = rope_table_len

        if self._fusable(x, start_pos, freqs_cis):
            q, k = self._norm_rope_fused(q, k, T, start_pos, pos_sin, pos_cos, cu_doc_lens, rope_pos_ids)
            q, k, v = q.view(B, T, -1, hd), k.view(B, T, -1, hd), v.view(B, T, -1, hd)
        else:
            if self.clip_qkv is not None:
                q, k, v = (t.clamp(min=-self.clip_qkv, max=self.clip_qkv) for t in (q, k, v))
            if not self.use_head_qk_norm:
                if self.q_norm is not None:
                    q = self._full_width_norm(self.q_norm, q)
                if self.k_norm is not None:
                    k = self._full_width_norm(self.k_norm, k)
            q, k, v = q.view(B, T, -1, hd), k.view(B, T, -1, hd), v.view(B, T, -1, hd)
            if self.use_head_qk_norm:
                if self.q_norm is not None:
                    q = self.q_norm(q)
                if self.k_norm is not None:
                    k = self.k_norm(k)
            if self.rope is not None:
                if rope_pos_ids is not None:
                    q, k = self.rope(q, k, head_first=False, pos_ids=rope_pos_ids, table_len=rope_table_len)
                else:
                    q, k = self.rope(q, k, head_first=False, start_pos=start_pos, pos_sin=pos_sin, pos_cos=pos_cos,
                                     freqs_cis=freqs_cis, cu_doc_lens=cu_doc_lens)

        att = self.backend(
            (q, k, v),
            cu_doc_lens=cu_doc_lens,
            cu_doc_lens_q=cu_doc_lens_q,
            cu_doc_lens_k=cu_doc_lens_k,
            max_doc_len=max_doc_len,
            max_doc_len_q=max_doc_len_q,
            max_doc_len_k=max_doc_len_k,
            local_k_slice=local_k_slice,
            kv_cache=self.kv_cache_manager,
            cache_leftpad=cache_leftpad,
        )
        if self.w_g is not None:
            assert self.gate is not None
            g = self.w_g(x)
            g = torch.sigmoid(g.float()) if self.gate.full_precision else torch.sigmoid(g)
            if self.gate.granularity == GateGranularity.headwise:
                att = att * g.to(att.dtype).unsqueeze(-1)
            else:
                att = att * g.to(att.dtype).view(B, T, -1, hd)
        att = att.reshape(B, T, -1)
        if tp_fused:
            return self._tp_project_out(att)
        return self._project_out(att)

    def _tp_project_in(self, x: torch.Tensor):
        """
        Column-parallel q / k / v of a sequence-sharded ``x [B, T/tp, D]``: each GEMM loads the peers' rows from their
        memory tile by tile (no gathered copy of ``x`` exists). The kernels return rows in rank-major order
        ``[tp, B, T/tp]``; for one sequence per batch that already is sequence order, otherwise one permuting copy
        restores ``[B, T]``.
        """
        from ...parallel.tp_fused import gather_linear_multi

        B, Tl, _ = x.shape
        ws = torch.distributed.get_world_size(self.tp_group)
        outs = []
        for y in gather_linear_multi(x, (self.w_q.weight, self.w_k.weight, self.w_v.weight), self.tp_group, "attn-qkv"):
            y = y.view(ws, B, Tl, -1)  # rows come back as [ws * B * Tl, F_local]
            outs.append(y.view(1, ws * Tl, -1) if B == 1 else y.permute(1, 0, 2, 3).reshape(B, ws * Tl, -1))
        return outs

    def _tp_project_out(self, att: torch.Tensor) -> torch.Tensor:
        """Row-parallel output projection: partial products leave the GEMM epilogue as reductions into the owners' rows."""
        from ...parallel.tp_fused import linear_reduce_scatter

        B, T, F = att.shape
        ws = torch.distributed.get_world_size(self.tp_group)
        Tl = T // ws
        rows = att if B == 1 else att.view(B, ws, Tl, F).permute(1, 0, 2, 3)
        y = linear_reduce_scatter(rows.reshape(ws * B * Tl, F), self.w_out.weight, self.tp_group, "attn-out")
        return y.view(B, Tl, -1)

    def sdpa(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_doc_lens: Optional[torch.Tensor] = None,
             cu_doc_lens_q: Optional[torch.Tensor] = None, cu_doc_lens_k: Optional[torch.Tensor] = None,
             max_doc_len: Optional[int] = None, max_doc_len_q: Optional[int] = None, max_doc_len_k: Optional[int] = None,
             local_k_slice: Optional[slice] = None, cache_leftpad: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Scaled dot-product attention of ``[B, T, heads, head_dim]`` tensors through this layer's backend (and KV cache)."""
        return self.backend((q, k, v), cu_doc_lens=cu_doc_lens, cu_doc_lens_q=cu_doc_lens_q, cu_doc_lens_k=cu_doc_lens_k,
                            max_doc_len=max_doc_len, max_doc_len_q=max_doc_len_q, max_doc_len_k=max_doc_len_k,
                            local_k_slice=local_k_slice, kv_cache=self.kv_cache_manager, cache_leftpad=cache_leftpad)

    def _full_width_norm(self, norm: nn.Module, t: torch.Tensor) -> torch.Tensor:
        if self.tp_enabled:
            from ...parallel.tensor import tp_full_width_rms_norm

            return tp_full_width_rms_norm(norm, t, self.tp_group)
        return norm(t)

    def _project_out(self, att: torch.Tensor) -> torch.Tensor:
        return self.w_out(att)

    # -- parallelism ----------------------------------------------------------------------------------
    def apply_tp(self, tp_mesh, input_layout=None, output_layout=None, use_local_output: bool = True,
                 float8_enabled: bool = False):
        from ...parallel.tensor import shard_attention_

        shard_attention_(self, tp_mesh)

    def apply_cp(self, cp_mesh, ring: Optional[RingContextParallelStyle] = None,
                 uly: Optional[UlyssesContextParallelStyle] = None):
        self.backend.apply_cp(cp_mesh, ring=ring, uly=uly)
        self._cp_enabled = True

    # -- bookkeeping -----------------------------------------------------------------------------------
    def init_kv_cache_manager(self, batch_size: int, max_seq_len: int, dtype: torch.dtype = torch.bfloat16) -> None:
        self.backend.assert_supports_kv_cache()
        device = self.w_q.weight.device
        if self.kv_cache_manager is not None and self.kv_cache_manager.is_reusable(batch_size, max_seq_len):
            self.kv_cache_manager.zero_cache()
        else:
            self.kv_cache_manager = KVCacheManager(batch_size, max_seq_len, self.n_kv_heads, self.head_dim, device, dtype)

    def reset_kv_cache_manager(self) -> None:
        self.kv_cache_manager = None

    def num_flops_per_token(self, seq_len: int) -> int:
        """``6 * params`` for the projections plus ``12 * H * Dh * visible keys`` for the score/value products."""
        n_params = sum(p.numel() for p in self.parameters())
        visible = min(self.window_size, seq_len) if self.window_size is not None else seq_len
        return 6 * n_params + 12 * self.n_heads * self.head_dim * visible

    def init_weights(self, *, init_method, d_model: int, block_idx: int, num_blocks: int, std: float = 0.02,
                     generator: Optional[torch.Generator] = None) -> None:
        from ..transformer.init import init_linear

        s_in, s_out = init_method.attention_stds(
            d_model=d_model, in_features=self.w_q.in_features, out_in_features=self.w_out.in_features,
            block_idx=block_idx, num_blocks=num_blocks, std=std,
        )
        for w in (self.w_q, self.w_k, self.w_v):
            init_linear(w, std=s_in, generator=generator)
        if self.w_g is not None:
            init_linear(self.w_g, std=s_in, generator=generator)
        init_linear(self.w_out, std=s_out, generator=generator)


class FusedAttention(Attention):
    """
    Variant with a single packed ``w_qkv`` projection (MHA only). The GPU data flow is the same as
    :class:`Attention`: one GEMM writes the packed buffer and q/k/v are column views of it.
    """

    def __init__(self, *, d_model: int, n_heads: int, bias: bool = True, rope: Optional[RoPEConfig] = None,
                 clip_qkv: Optional[float] = None, dropout: float = 0.0, dtype: torch.dtype = torch.float32,
                 init_device: str = "cpu", cache: Optional[BufferCache] = None, backend: Optional[AttentionBackendName] = None,
                 n_kv_heads: Optional[int] = None, **unused):
        if n_kv_heads is not None and n_kv_heads != n_heads:
            raise OLMoConfigurationError("fused attention does not support MQA/GQA")
        nn.Module.__init__(self)
        self.d_model, self.n_heads, self.n_kv_heads = d_model, n_heads, n_heads
        self.head_dim = d_model // n_heads
        self.w_qkv = Linear(d_model, 3 * d_model, bias, dtype, init_device)
        self.w_out = Linear(d_model, d_model, bias, dtype, init_device)
        self.clip_qkv = clip_qkv
        self.dropout_p = dropout
        self.rope = None
        if rope is not None:
            self.rope = RoPEConfig(name="default", theta=rope.theta, full_precision=rope.full_precision,
                                   scaling=rope.scaling).build(self.head_dim, cache=cache)
        self.q_norm = self.k_norm = None
        self.use_head_qk_norm = False
        self.w_g = None
        self.gate = None
        self.window_size = None
        self.backend_name = _pick_backend(backend, True)
        self.backend = self.backend_name.build(head_dim=self.head_dim, n_heads=n_heads, dropout_p=dropout)
        self.kv_cache_manager = None
        self.tp_group = None
        self._cp_enabled = False

    def forward(self, x: torch.Tensor, max_doc_len: Optional[int] = None, cu_doc_lens: Optional[torch.Tensor] = None,
                pos_sin: Optional[torch.Tensor] = None, pos_cos: Optional[torch.Tensor] = None,
                freqs_cis: Optional[torch.Tensor] = None, cache_leftpad: Optional[torch.Tensor] = None, **kwargs) -> torch.Tensor:
        B, T, _ = x.shape
        qkv = self.w_qkv(x)
        if self.clip_qkv is not None:
            qkv = qkv.clamp(min=-self.clip_qkv, max=self.clip_qkv)
        q, k, v = qkv.split(self.d_model, dim=-1)
        if self._fusable(x, None, freqs_cis):
            q, k = self._norm_rope_fused(q, k, T, None, pos_sin, pos_cos, cu_doc_lens)
            q, k, v = (t.reshape(B, T, self.n_heads, self.head_dim) for t in (q, k, v))
        else:
            q, k, v = (t.reshape(B, T, self.n_heads, self.head_dim) for t in (q, k, v))
            if self.rope is not None:
                q, k = self.rope(q, k, head_first=False, pos_sin=pos_sin, pos_cos=pos_cos, cu_doc_lens=cu_doc_lens)
        att = self.backend((q, k, v), cu_doc_lens=cu_doc_lens, max_doc_len=max_doc_len)
        return self.w_out(att.reshape(B, T, -1))

    def apply_tp(self, *args, **kwargs):
        raise NotImplementedError("tensor parallelism is not implemented for the fused attention variant")

    def init_weights(self, *, init_method, d_model: int, block_idx: int, num_blocks: int, std: float = 0.02,
                     generator: Optional[torch.Generator] = None) -> None:
        from ..transformer.init import init_linear

        s_in, s_out = init_method.attention_stds(d_model=d_model, in_features=d_model, out_in_features=d_model,
                                                 block_idx=block_idx, num_blocks=num_blocks, std=std)
        init_linear(self.w_qkv, std=s_in, generator=generator)
        init_linear(self.w_out, std=s_out, generator=generator)


class NormalizedAttention(Attention):
    """nGPT attention: unit-norm q/k with learned scales ``sq``/``sk`` and softmax scale ``sqrt(head_dim)``."""

    def __init__(self, *, d_model: int, n_heads: int, n_kv_heads: Optional[int] = None, rope: Optional[RoPEConfig] = None,
                 qk_norm: Optional[LayerNormConfig] = None, use_flash: Optional[bool] = None,
                 backend: Optional[AttentionBackendName] = None, dtype: torch.dtype = torch.float32, init_device: str = "cpu",
                 cache: Optional[BufferCache] = None, **unused):
        super().__init__(d_model=d_model, n_heads=n_heads, n_kv_heads=n_kv_heads, bias=False, rope=rope, qk_norm=qk_norm,
                         use_flash=use_flash, backend=backend, dtype=dtype, init_device=init_device, cache=cache,
                         softmax_scale=math.sqrt(d_model // n_heads))
        self.sq_init_value = 1.0
        self.sq_init_scaling = 1.0 / math.sqrt(d_model)
        self.sq = nn.Parameter(torch.empty(self.head_dim * n_heads, dtype=dtype, device=init_device))
        self.sk_init_value = 1.0
        self.sk_init_scaling = 1.0 / math.sqrt(d_model)
        self.sk = nn.Parameter(torch.empty(self.head_dim * self.n_kv_heads, dtype=dtype, device=init_device))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.sq.device.type != "meta":
            nn.init.constant_(self.sq, self.sq_init_scaling)
            nn.init.constant_(self.sk, self.sk_init_scaling)

    def forward(self, x: torch.Tensor, cu_doc_lens: Optional[torch.Tensor] = None, max_doc_len: Optional[int] = None,
                pos_sin: Optional[torch.Tensor] = None, pos_cos: Optional[torch.Tensor] = None,
                freqs_cis: Optional[torch.Tensor] = None, cache_leftpad: Optional[torch.Tensor] = None, **kwargs) -> torch.Tensor:
        if cache_leftpad is not None:
            raise NotImplementedError("cache_leftpad is not supported for the normalized attention variant")
        B, T, _ = x.shape
        q, k, v = multi_linear(x, (self.w_q, self.w_k, self.w_v))
        if self.q_norm is not None and self.k_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        q = (self.sq * (self.sq_init_value / self.sq_init_scaling)).to(q.dtype).view(1, 1, -1) * q
        k = (self.sk * (self.sk_init_value / self.sk_init_scaling)).to(k.dtype).view(1, 1, -1) * k
        q = q.view(B, T, self.n_heads, self.head_dim)
        k = k.view(B, T, self.n_kv_heads, self.head_dim)
        v = v.view(B, T, self.n_kv_heads, self.head_dim)
        if self.rope is not None:
            q, k = self.rope(q, k, head_first=False, pos_sin=pos_sin, pos_cos=pos_cos, freqs_cis=freqs_cis,
                             cu_doc_lens=cu_doc_lens)
        att = self.backend((q, k, v), cu_doc_lens=cu_doc_lens, max_doc_len=max_doc_len)
        return self.w_out(att.reshape(B, T, -1))

    def apply_tp(self, *args, **kwargs):
        raise NotImplementedError("tensor parallelism is not implemented for the normalized attention variant")

    @torch.no_grad()
    def normalize_matrices(self) -> None:
        for w, dim in ((self.w_q.weight, -1), (self.w_k.weight, -1), (self.w_v.weight, -1), (self.w_out.weight, 0)):
            w.copy_(l2_normalize(w, dim=dim))
