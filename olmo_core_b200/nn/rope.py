"""
Rotary positional embeddings: config, frequency-scaling strategies and modules
(API of src/olmo_core/nn/rope.py:29-867).

The sin/cos tables are ``[seq_len, rotary_dim]`` fp32, built as ``cat(freqs, freqs)`` with
``freqs = outer(positions, theta^(-2i/d))``, and shared between layers through a :class:`BufferCache`.
On CUDA the attention module does not call :meth:`RotaryEmbedding.forward`; it hands the tables to the
fused QK-norm + RoPE kernel (``ops.elementwise.norm_rope``). ``forward`` is the PyTorch statement of the
same math used on CPU, for KV-cache decoding and as the test oracle.
"""

from __future__ import annotations

import math
from abc import abstractmethod
from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

import torch
import torch.nn as nn

from ..config import Config, Registrable, StrEnum
from ..exceptions import OLMoConfigurationError
from .buffer_cache import BufferCache
from .config import ModuleConfig

__all__ = [
    "RoPEType",
    "RoPEConfig",
    "RoPEScalingConfig",
    "ABFRoPEScalingConfig",
    "PIRoPEScalingConfig",
    "StepwiseRoPEScalingConfig",
    "YaRNRoPEScalingConfig",
    "RoPEBuffers",
    "RotaryEmbeddingBase",
    "RotaryEmbedding",
    "FusedRotaryEmbedding",
    "ComplexRotaryEmbedding",
    "compute_inv_freqs",
]


class RoPEType(StrEnum):
    default = "default"
    fused = "fused"
    complex = "complex"


def compute_inv_freqs(theta: float, dim: int, device: Optional[torch.device] = None) -> torch.Tensor:
    """``theta^(-2i/dim)`` for ``i`` in ``[0, dim/2)``, fp32."""
    return 1.0 / (theta ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))


@dataclass
class RoPEScalingConfig(Config, Registrable):
    """Strategy for stretching RoPE to longer contexts: returns scaled inverse frequencies and a factor
    folded into the sin/cos tables (which rescales attention logits)."""

    @abstractmethod
    def compute_scaled_inv_freq(self, theta: int, dim: int, device: torch.device) -> Tuple[torch.Tensor, float]:
        raise NotImplementedError

    @abstractmethod
    def to_hf_config(self) -> dict:
        raise NotImplementedError


@RoPEScalingConfig.register("abf")
@dataclass
class ABFRoPEScalingConfig(RoPEScalingConfig):
    """Adjusted base frequency: simply a different ``theta``."""

    attention_rescale_factor: float = 1.0
    new_theta: int = 8_000_000

    def compute_scaled_inv_freq(self, theta: int, dim: int, device: torch.device) -> Tuple[torch.Tensor, float]:
        return compute_inv_freqs(self.new_theta, dim, device), self.attention_rescale_factor

    def to_hf_config(self) -> dict:
        return {"rope_type": "default", "rope_theta": self.new_theta}


@RoPEScalingConfig.register("pi")
@dataclass
class PIRoPEScalingConfig(RoPEScalingConfig):
    """Position interpolation: all frequencies divided by ``factor``."""

    attention_rescale_factor: float = 1.0
    factor: float = 2.0

    def compute_scaled_inv_freq(self, theta: int, dim: int, device: torch.device) -> Tuple[torch.Tensor, float]:
        inv = compute_inv_freqs(theta, dim, device)
        return (inv / self.factor if self.factor != 1.0 else inv), self.attention_rescale_factor

    def to_hf_config(self) -> dict:
        return {"rope_type": "linear", "factor": self.factor}


@RoPEScalingConfig.register("stepwise")
@dataclass
class StepwiseRoPEScalingConfig(RoPEScalingConfig):
    """Llama-3.1 per-frequency scaling: long wavelengths divided by ``factor``, short ones kept,
    a linear blend in between."""

    attention_rescale_factor: float = 1.0
    factor: float = 32.0
    low_freq_proportion: float = 0.0
    high_freq_proportion: float = 0.25
    old_context_len: int = 8192

    def compute_scaled_inv_freq(self, theta: int, dim: int, device: torch.device) -> Tuple[torch.Tensor, float]:
        inv = compute_inv_freqs(theta, dim, device)
        low_f = 1.0 / (1.0 - self.low_freq_proportion)
        high_f = 1.0 / self.high_freq_proportion
        wavelen = 2.0 * math.pi / inv
        long_wave = wavelen > self.old_context_len / low_f
        short_wave = wavelen < self.old_context_len / high_f
        blend = (self.old_context_len / wavelen - low_f) / (high_f - low_f)
        mid = (1.0 - blend) * inv / self.factor + blend * inv
        out = torch.where(long_wave, inv / self.factor, torch.where(short_wave, inv, mid))
        return out, self.attention_rescale_factor

    def to_hf_config(self) -> dict:
        return {
            "rope_type": "llama3",
            "factor": self.factor,
            "original_max_position_embeddings": self.old_context_len,
            "low_freq_factor": 1.0 / (1 - self.low_freq_proportion),
            "high_freq_factor": 1.0 / self.high_freq_proportion,
        }


@RoPEScalingConfig.register("yarn")
@dataclass
class YaRNRoPEScalingConfig(RoPEScalingConfig):
    """YaRN: ramp between interpolated (``/factor``) and original frequencies; tables scaled by
    ``0.1 ln(factor) + 1``."""

    factor: float = 8.0
    beta_fast: int = 32
    beta_slow: int = 1
    old_context_len: int = 8192

    _IGNORE_FIELDS: ClassVar[Tuple[str, ...]] = ("attention_rescale_factor",)

    def _dim_of_rotations(self, n_rot: float, theta: float, dim: int) -> float:
        return dim * math.log(self.old_context_len / (n_rot * 2.0 * math.pi)) / (2.0 * math.log(theta))

    def compute_scaled_inv_freq(self, theta: int, dim: int, device: torch.device) -> Tuple[torch.Tensor, float]:
        extrap = compute_inv_freqs(theta, dim, device)
        interp = extrap / self.factor
        half = extrap.shape[0]
        lo = max(int(math.floor(self._dim_of_rotations(self.beta_fast, theta, dim))), 0)
        hi = min(int(math.ceil(self._dim_of_rotations(self.beta_slow, theta, dim))), half - 1)
        ramp = ((torch.arange(half, device=device, dtype=torch.float32) - lo) / max(hi - lo, 1e-3)).clamp_(0, 1)
        return interp * ramp + extrap * (1.0 - ramp), self.get_attention_rescale_factor()

    def get_attention_rescale_factor(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0

    def to_hf_config(self) -> dict:
        return {
            "rope_type": "yarn",
            "factor": self.factor,
            "original_max_position_embeddings": self.old_context_len,
            "beta_fast": self.beta_fast,
            "beta_slow": self.beta_slow,
            "attention_factor": self.get_attention_rescale_factor(),
        }


@dataclass
class RoPEConfig(ModuleConfig):
    name: RoPEType = RoPEType.default
    theta: int = 500_000
    full_precision: bool = True
    no_global_rope: bool = False
    scaling: Optional[RoPEScalingConfig] = None
    partial_rotary_factor: float = 1.0

    def build(self, head_size: int, cache: Optional[BufferCache] = None) -> "RotaryEmbeddingBase":
        kwargs = self.as_dict(exclude_none=True, recurse=False)
        kwargs.pop("name")
        kwargs.pop("no_global_rope")
        kwargs.update(head_size=head_size, cache=cache)
        try:
            if self.name == RoPEType.default:
                return RotaryEmbedding(**kwargs)
            if self.name == RoPEType.fused:
                return FusedRotaryEmbedding(**kwargs)
            if self.name == RoPEType.complex:
                return ComplexRotaryEmbedding(**kwargs)
            raise NotImplementedError(self.name)
        except TypeError as e:
            raise OLMoConfigurationError(f"invalid options for '{self.name}' {self.__class__.__name__}, {e}") from e


@dataclass
class RoPEBuffers:
    pos_sin: Optional[torch.Tensor] = None
    pos_cos: Optional[torch.Tensor] = None
    freqs_cis: Optional[torch.Tensor] = None


class RotaryEmbeddingBase(nn.Module):
    def __init__(
        self,
        *,
        head_size: int,
        theta: int = 500_000,
        full_precision: bool = True,
        cache: Optional[BufferCache] = None,
        scaling: Optional[RoPEScalingConfig] = None,
        partial_rotary_factor: float = 1.0,
    ):
        super().__init__()
        self.dim = head_size
        self.rotary_dim = int(head_size * partial_rotary_factor)
        if self.rotary_dim % 2 != 0:
            raise OLMoConfigurationError("the rotary dimension must be even")
        self.theta = theta
        self.full_precision = full_precision
        self.scaling = scaling
        self._cache = (cache or BufferCache()).with_namespace(
            f"rope-{self.__class__.__name__}-{theta}-{self.rotary_dim}-{id(scaling) if scaling is not None else 0}"
        )

    def warmup_cache(self, max_seq_len: int, device: torch.device) -> None:
        self.get_buffers(max_seq_len, device)

    @abstractmethod
    def get_buffers(self, max_seq_len: int, device: torch.device) -> RoPEBuffers:
        raise NotImplementedError

    def _inv_freq(self, device: torch.device) -> Tuple[torch.Tensor, float]:
        if self.scaling is None:
            return compute_inv_freqs(self.theta, self.rotary_dim, device), 1.0
        return self.scaling.compute_scaled_inv_freq(self.theta, self.rotary_dim, device)


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


class RotaryEmbedding(RotaryEmbeddingBase):
    """Rotate-half RoPE with cached fp32 sin/cos tables."""

    def _tables(self, seq_len: int, device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
        sin = self._cache.get("sin")
        cos = self._cache.get("cos")
        if sin is not None and cos is not None and sin.shape[0] >= seq_len and sin.device == device:
            return sin, cos
        with torch.autocast(device.type, enabled=False):
            inv_freq, rescale = self._inv_freq(device)
            pos = torch.arange(seq_len, device=device, dtype=torch.float32)
            freqs = torch.outer(pos, inv_freq)
            ang = torch.cat((freqs, freqs), dim=-1)
            sin, cos = ang.sin() * rescale, ang.cos() * rescale
        self._cache["sin"], self._cache["cos"] = sin, cos
        return sin, cos

    def get_buffers(self, max_seq_len: int, device: torch.device) -> RoPEBuffers:
        sin, cos = self._tables(max_seq_len, device)
        return RoPEBuffers(pos_sin=sin, pos_cos=cos)

    def _rotate(self, t: torch.Tensor, sin: torch.Tensor, cos: torch.Tensor) -> torch.Tensor:
        rd = sin.shape[-1]
        if rd == t.shape[-1]:
            return t * cos + _rotate_half(t) * sin
        rot, rest = t[..., :rd], t[..., rd:]
        return torch.cat((rot * cos + _rotate_half(rot) * sin, rest), dim=-1)

    def forward(
        self,
        q: torch.Tensor,
        k: torch.Tensor,
        head_first: bool = True,
        start_pos: Optional[int] = None,
        pos_sin: Optional[torch.Tensor] = None,
        pos_cos: Optional[torch.Tensor] = None,
        freqs_cis: Optional[torch.Tensor] = None,
        cu_doc_lens: Optional[torch.Tensor] = None,
        pos_ids: Optional[torch.Tensor] = None,
        table_len: Optional[int] = None,
    ) -> Tuple[torch.Tensor, torch.Tensor]:
        """
        ``q``/``k``: ``[B, H, T, D]`` when ``head_first`` else ``[B, T, H, D]``. ``start_pos`` is the absolute
        position of the first token (decoding); ``cu_doc_lens`` restarts positions at each packed document;
        ``pos_ids`` (int ``[B, T]``) names every token's position outright (tables of ``table_len`` rows).
        """
        if pos_ids is not None:
            seq_dim = 2 if head_first else 1
            qf, kf = (q.float(), k.float()) if self.full_precision else (q, k)
            with torch.autocast(q.device.type, enabled=False):
                ids = pos_ids.to(q.device).long()
                ps, pc = self._tables(int(table_len or (int(ids.max()) + 1)), q.device)
                s_, c_ = ps.type_as(qf)[ids], pc.type_as(qf)[ids]  # [B, T, D]
                s_, c_ = (s_.unsqueeze(1), c_.unsqueeze(1)) if head_first else (s_.unsqueeze(2), c_.unsqueeze(2))
                qf, kf = self._rotate(qf, s_, c_), self._rotate(kf, s_, c_)
            return qf.type_as(q), kf.type_as(k)
        if freqs_cis is not None:
            raise RuntimeError(f"'freqs_cis' is invalid for {self.__class__.__name__}")
        if cu_doc_lens is not None and start_pos is not None:
            raise RuntimeError("'cu_doc_lens' and 'start_pos' are mutually exclusive")
        seq_dim = 2 if head_first else 1
        q_len, k_len = q.size(seq_dim), k.size(seq_dim)
        qf, kf = (q.float(), k.float()) if self.full_precision else (q, k)
        with torch.autocast(q.device.type, enabled=False):
            need = (start_pos + k_len) if start_pos is not None else k_len
            if pos_sin is None or pos_cos is None:
                pos_sin, pos_cos = self._tables(need, q.device)
            if pos_sin.size(-2) < need:
                raise RuntimeError(f"RoPE buffers shorter than required: need {need}, have {pos_sin.size(-2)}.")
            pos_sin, pos_cos = pos_sin.type_as(qf), pos_cos.type_as(qf)
            if cu_doc_lens is not None:
                if q_len != k_len:
                    raise RuntimeError("'cu_doc_lens' requires q_len == k_len (no kv-cache packed mode)")
                B = q.size(0)
                flat = torch.arange(B * k_len, device=q.device, dtype=cu_doc_lens.dtype)
                doc = torch.bucketize(flat, cu_doc_lens[1:], right=True)
                idx = (flat - cu_doc_lens[doc]).long()
                s = pos_sin.index_select(0, idx).view(B, k_len, -1)
                c = pos_cos.index_select(0, idx).view(B, k_len, -1)
                s, c = (s.unsqueeze(1), c.unsqueeze(1)) if head_first else (s.unsqueeze(2), c.unsqueeze(2))
                qf, kf = self._rotate(qf, s, c), self._rotate(kf, s, c)
            else:
                q0 = start_pos if start_pos is not None else k_len - q_len
                k0 = start_pos if start_pos is not None else 0

                def view(t: torch.Tensor, start: int, n: int) -> torch.Tensor:
                    t = t[start : start + n]
                    return t[None, None] if head_first else t[None, :, None]

                qf = self._rotate(qf, view(pos_sin, q0, q_len), view(pos_cos, q0, q_len))
                kf = self._rotate(kf, view(pos_sin, k0, k_len), view(pos_cos, k0, k_len))
        return qf.type_as(q), kf.type_as(k)


class FusedRotaryEmbedding(RotaryEmbedding):
    """
    The rotary embedding under its "fused" name. Called with one packed ``qkv`` tensor
    ``[batch, seq, 3, heads, head_size]`` it rotates the query and key planes and returns the packed tensor
    (the calling convention of src/olmo_core/nn/rope.py:668-705); called with ``(q, k, ...)`` it behaves like
    :class:`RotaryEmbedding`. On CUDA both forms run the package's rotary kernel.
    """

    def forward(self, q: torch.Tensor, k: Optional[torch.Tensor] = None, *args, **kwargs):  # type: ignore[override]
        if k is not None:
            return super().forward(q, k, *args, **kwargs)
        qkv = q
        if qkv.dim() != 5 or qkv.shape[2] != 3:
            raise ValueError("expected a packed qkv tensor of shape (batch, seq, 3, heads, head_size)")
        if kwargs.get("freqs_cis") is not None:
            raise RuntimeError(f"'freqs_cis' is invalid for {type(self).__name__}")
        q_rot, k_rot = super().forward(qkv[:, :, 0], qkv[:, :, 1], head_first=False, *args, **kwargs)
        return torch.stack([q_rot.to(qkv.dtype), k_rot.to(qkv.dtype), qkv[:, :, 2]], dim=2)


class ComplexRotaryEmbedding(RotaryEmbeddingBase):
    """RoPE as a complex rotation of adjacent channel pairs (Llama-style interleaved layout)."""

    def _freqs_cis(self, seq_len: int, device: torch.device) -> torch.Tensor:
        f = self._cache.get("freqs_cis")
        if f is not None and f.shape[0] >= seq_len and f.device == device:
            return f
        with torch.autocast(device.type, enabled=False):
            inv_freq, rescale = self._inv_freq(device)
            pos = torch.arange(seq_len, device=device, dtype=torch.float32)
            f = torch.polar(torch.full((seq_len, inv_freq.shape[0]), rescale, device=device), torch.outer(pos, inv_freq))
        self._cache["freqs_cis"] = f
        return f

    def get_buffers(self, max_seq_len: int, device: torch.device) -> RoPEBuffers:
        return RoPEBuffers(freqs_cis=self._freqs_cis(max_seq_len, device))

    def forward(
        self,
        q: torch.Tensor,
        k: torch.Tensor,
        head_first: bool = True,
        start_pos: Optional[int] = None,
        pos_sin: Optional[torch.Tensor] = None,
        pos_cos: Optional[torch.Tensor] = None,
        freqs_cis: Optional[torch.Tensor] = None,
        cu_doc_lens: Optional[torch.Tensor] = None,
    ) -> Tuple[torch.Tensor, torch.Tensor]:
        if pos_sin is not None or pos_cos is not None:
            raise RuntimeError(f"'pos_sin'/'pos_cos' are invalid for {self.__class__.__name__}")
        if cu_doc_lens is not None:
            raise RuntimeError("intra-document positions are not supported by the complex variant")
        seq_dim = 2 if head_first else 1
        q_len, k_len = q.size(seq_dim), k.size(seq_dim)
        need = (start_pos + k_len) if start_pos is not None else k_len
        if freqs_cis is None:
            freqs_cis = self._freqs_cis(need, q.device)
        q0 = start_pos if start_pos is not None else k_len - q_len
        k0 = start_pos if start_pos is not None else 0

        def rot(t: torch.Tensor, start: int, n: int) -> torch.Tensor:
            rd = self.rotary_dim
            tr, rest = t[..., :rd], t[..., rd:]
            tc = torch.view_as_complex(tr.float().reshape(*tr.shape[:-1], -1, 2))
            f = freqs_cis[start : start + n]
            f = f[None, None] if head_first else f[None, :, None]
            out = torch.view_as_real(tc * f).flatten(-2)
            return torch.cat((out.type_as(t), rest), dim=-1) if rest.numel() else out.type_as(t)

        return rot(q, q0, q_len), rot(k, k0, k_len)
