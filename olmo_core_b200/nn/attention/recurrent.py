"""
Gated DeltaNet: a linear-attention sequence mixer with a per-head matrix state updated by the gated delta rule
(parameters and forward semantics of src/olmo_core/nn/attention/recurrent.py:34-453; used by the Qwen-3.5-style hybrids).

Per value head, with L2-normalised ``q_t, k_t`` (``q`` scaled by ``d_k^-1/2``), decay ``a_t = exp(g_t)`` and write
strength ``beta_t``::

    S_t = a_t * S_{t-1} + k_t (beta_t * (v_t - a_t * S_{t-1}^T k_t))^T        S in R^{d_k x d_v}
    o_t = S_t^T q_t

The recurrence is evaluated chunk-wise: inside a chunk of ``C`` tokens the dependence of the corrected values on one
another is a unit-lower-triangular system, solved once per chunk, so the sequential part is ``T / C`` matrix products
instead of ``T`` rank-one updates. Everything is plain PyTorch in fp32 (also the oracle for a future kernel).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...config import DType
from ..convolution import CausalConv1d
from .base import SequenceMixerConfig

__all__ = ["GatedDeltaNet", "GatedDeltaNetConfig", "gated_delta_rule", "gated_delta_rule_recurrent"]


def gated_delta_rule_recurrent(q, k, v, g, beta, scale: Optional[float] = None):
    """Token-by-token reference. q,k: [B,T,H,dk], v: [B,T,H,dv], g,beta: [B,T,H] -> [B,T,H,dv]."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    q = F.normalize(q, dim=-1) * scale
    k = F.normalize(k, dim=-1)
    S = q.new_zeros(B, H, dk, dv)
    out = q.new_empty(B, T, H, dv)
    for t in range(T):
        S = S * g[:, t].exp()[..., None, None]
        delta = (v[:, t] - torch.einsum("bhkv,bhk->bhv", S, k[:, t])) * beta[:, t][..., None]
        S = S + torch.einsum("bhk,bhv->bhkv", k[:, t], delta)
        out[:, t] = torch.einsum("bhkv,bhk->bhv", S, q[:, t])
    return out


def gated_delta_rule(q, k, v, g, beta, scale: Optional[float] = None, chunk_size: int = 64):
    """Chunk-parallel evaluation of the same recurrence (identical result up to fp32 rounding)."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    in_dtype = v.dtype
    q, k, v, g, beta = (t.float().transpose(1, 2) for t in (q, k, v, g, beta))  # [B,H,T,...]
    q = F.normalize(q, dim=-1) * scale
    k = F.normalize(k, dim=-1)
    pad = (-T) % chunk_size
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
        g, beta = F.pad(g, (0, pad)), F.pad(beta, (0, pad))
    n = q.shape[2] // chunk_size
    C = chunk_size
    q, k, v = (t.reshape(B, H, n, C, -1) for t in (q, k, v))
    g, beta = g.reshape(B, H, n, C), beta.reshape(B, H, n, C)
    gc = g.cumsum(-1)  # log decay from the chunk start up to and including token i
    decay = (gc[..., :, None] - gc[..., None, :]).tril().exp().tril()  # exp(gc_i - gc_j) for j <= i
    kb = k * beta[..., None]
    # (I + A) u = beta * v - beta * exp(gc) * (k S0), with A_ij = beta_i exp(gc_i - gc_j) k_i.k_j for j < i
    A = (kb @ k.transpose(-1, -2)) * decay
    A = A.tril(-1)
    eye = torch.eye(C, device=q.device, dtype=q.dtype)
    T_inv = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False)
    u_rhs = T_inv @ (v * beta[..., None])             # part of the corrected values that does not depend on S0
    w = T_inv @ (kb * gc.exp()[..., None])            # multiplies S0: u = u_rhs - w S0
    S = q.new_zeros(B, H, dk, dv)
    out = q.new_empty(B, H, n, C, dv)
    attn = (q @ k.transpose(-1, -2)) * decay          # intra-chunk scores (causal, inclusive)
    for c in range(n):
        u = u_rhs[:, :, c] - w[:, :, c] @ S
        out[:, :, c] = (q[:, :, c] * gc[:, :, c].exp()[..., None]) @ S + attn[:, :, c] @ u
        last = gc[:, :, c, -1]
        S = S * last.exp()[..., None, None] + (k[:, :, c] * (last[..., None] - gc[:, :, c]).exp()[..., None]).transpose(-1, -2) @ u
    out = out.reshape(B, H, n * C, dv)[:, :, :T]
    return out.transpose(1, 2).to(in_dtype)


class _GatedRMSNorm(nn.Module):
    """``rmsnorm(x) * weight * silu(gate)`` over the last dimension."""

    def __init__(self, size: int, eps: float, device: str):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(size, device=device))

    def forward(self, x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()
        return (y * F.silu(gate.float())).to(x.dtype)


class GatedDeltaNet(nn.Module):
    def __init__(self, *, d_model: int, n_heads: int, n_v_heads: Optional[int] = None, head_dim: Optional[int] = None,
                 expand_v: float = 2.0, allow_neg_eigval: bool = True, conv_size: int = 4, conv_bias: bool = False,
                 norm_eps: float = 1e-5, dtype: torch.dtype = torch.float32, init_device: str = "cpu"):
        super().__init__()
        self.d_model = d_model
        self.n_heads = n_heads
        self.n_v_heads = n_v_heads if n_v_heads is not None else n_heads
        self.head_dim = head_dim if head_dim is not None else d_model // n_heads
        self.expand_v = expand_v
        self.allow_neg_eigval = allow_neg_eigval
        self.conv_size = conv_size
        self.head_k_dim = self.head_dim
        self.head_v_dim = int(self.head_dim * expand_v)
        self.key_dim = self.n_heads * self.head_k_dim
        self.value_dim = self.n_v_heads * self.head_v_dim
        assert self.n_v_heads >= self.n_heads and self.n_v_heads % self.n_heads == 0
        lin = dict(bias=False, dtype=dtype, device=init_device)
        self.w_q = nn.Linear(d_model, self.key_dim, **lin)
        self.w_k = nn.Linear(d_model, self.key_dim, **lin)
        self.w_v = nn.Linear(d_model, self.value_dim, **lin)
        self.w_a = nn.Linear(d_model, self.n_v_heads, **lin)
        self.w_b = nn.Linear(d_model, self.n_v_heads, **lin)
        self.A_log = nn.Parameter(torch.empty(self.n_v_heads, dtype=dtype, device=init_device))
        self.dt_bias = nn.Parameter(torch.empty(self.n_v_heads, dtype=dtype, device=init_device))
        conv = dict(kernel_size=conv_size, bias=conv_bias, activation="silu", dtype=dtype, init_device=init_device)
        self.q_conv1d = CausalConv1d(hidden_size=self.key_dim, **conv)
        self.k_conv1d = CausalConv1d(hidden_size=self.key_dim, **conv)
        self.v_conv1d = CausalConv1d(hidden_size=self.value_dim, **conv)
        self.w_g = nn.Linear(d_model, self.value_dim, **lin)
        self.o_norm = _GatedRMSNorm(self.head_v_dim, norm_eps, init_device)
        self.w_out = nn.Linear(self.value_dim, d_model, **lin)
        self.cp_enabled = False

    def _forward_ulysses(self, x: torch.Tensor, cu_doc_lens: Optional[torch.Tensor]) -> torch.Tensor:
        """
        Context parallelism for a recurrent mixer: the state runs along the whole sequence, so instead of the sequence
        the HEADS are split. Projections act on this rank's tokens; one sequence<->head exchange hands every rank all
        tokens of its heads (the depth-wise convolutions use the matching channel slice of their weights), the delta rule
        runs per head over the full sequence, and a second exchange brings the outputs back to the local tokens
        (reference: src/olmo_core/nn/attention/recurrent.py:164-238).
        """
        from ...distributed.parallel.context_parallel import (
            all_to_all_cp2hp,
            all_to_all_single_cp2hp,
            all_to_all_single_hp2cp,
        )

        B, Tl, _ = x.shape
        cp, rank = self._cp_size, self._cp_rank
        q = self.w_q(x).view(B, Tl, self.n_heads, self.head_k_dim)
        k = self.w_k(x).view(B, Tl, self.n_heads, self.head_k_dim)
        v = self.w_v(x).view(B, Tl, self.n_v_heads, self.head_v_dim)
        ab = torch.stack([self.w_a(x).float(), self.w_b(x).float()], dim=-1)  # [B, Tl, Hv, 2]
        q, k = all_to_all_cp2hp([q, k], self._cp_pg)  # [B, T, H / cp, hk]
        v = all_to_all_single_cp2hp(v, self._cp_pg)
        ab = all_to_all_single_cp2hp(ab, self._cp_pg)  # [B, T, Hv / cp, 2]
        T = q.shape[1]
        hv = slice(rank * self.n_v_heads // cp, (rank + 1) * self.n_v_heads // cp)
        beta = ab[..., 1].sigmoid().to(x.dtype)
        if self.allow_neg_eigval:
            beta = beta * 2.0
        g = -self.A_log.float()[hv].exp() * F.softplus(ab[..., 0] + self.dt_bias[hv])
        q = self.q_conv1d(q.reshape(B, T, -1), cu_seqlens=cu_doc_lens).view(B, T, -1, self.head_k_dim)
        k = self.k_conv1d(k.reshape(B, T, -1), cu_seqlens=cu_doc_lens).view(B, T, -1, self.head_k_dim)
        v = self.v_conv1d(v.reshape(B, T, -1), cu_seqlens=cu_doc_lens).view(B, T, -1, self.head_v_dim)
        if self.n_v_heads > self.n_heads:
            r = self.n_v_heads // self.n_heads
            q, k = q.repeat_interleave(r, dim=-2), k.repeat_interleave(r, dim=-2)
        if cu_doc_lens is None:
            o = gated_delta_rule(q, k, v, g, beta)
        else:
            bounds = cu_doc_lens.tolist()
            o = torch.cat([gated_delta_rule(q[:, a:b], k[:, a:b], v[:, a:b], g[:, a:b], beta[:, a:b])
                           for a, b in zip(bounds[:-1], bounds[1:])], dim=1)
        o = all_to_all_single_hp2cp(o.contiguous(), self._cp_pg)  # [B, Tl, Hv, hv]
        gate = self.w_g(x).view(B, Tl, -1, self.head_v_dim)
        return self.w_out(self.o_norm(o, gate).reshape(B, Tl, -1))

    def forward(self, x: torch.Tensor, cu_doc_lens: Optional[torch.Tensor] = None, **kwargs) -> torch.Tensor:
        del kwargs  # the block passes attention-only arguments (RoPE buffers, ...) to every mixer
        if self.cp_enabled:
            return self._forward_ulysses(x, cu_doc_lens)
        B, T, _ = x.shape
        q, k, v = self.w_q(x), self.w_k(x), self.w_v(x)
        beta = self.w_b(x).sigmoid()
        if self.allow_neg_eigval:
            beta = beta * 2.0
        g = -self.A_log.float().exp() * F.softplus(self.w_a(x).float() + self.dt_bias)
        q = self.q_conv1d(q, cu_seqlens=cu_doc_lens).view(B, T, -1, self.head_k_dim)
        k = self.k_conv1d(k, cu_seqlens=cu_doc_lens).view(B, T, -1, self.head_k_dim)
        v = self.v_conv1d(v, cu_seqlens=cu_doc_lens).view(B, T, -1, self.head_v_dim)
        if self.n_v_heads > self.n_heads:
            r = self.n_v_heads // self.n_heads
            q, k = q.repeat_interleave(r, dim=-2), k.repeat_interleave(r, dim=-2)
        if cu_doc_lens is None:
            o = gated_delta_rule(q, k, v, g, beta)
        else:  # the state restarts at every document boundary
            bounds = cu_doc_lens.tolist()
            o = torch.cat([gated_delta_rule(q[:, a:b], k[:, a:b], v[:, a:b], g[:, a:b], beta[:, a:b])
                           for a, b in zip(bounds[:-1], bounds[1:])], dim=1)
        gate = self.w_g(x).view(B, T, -1, self.head_v_dim)
        return self.w_out(self.o_norm(o, gate).reshape(B, T, -1))

    def apply_tp(self, tp_mesh, **kwargs) -> None:
        raise NotImplementedError("tensor parallelism is not implemented for GatedDeltaNet")

    def apply_cp(self, cp_mesh, ring=None, uly=None, **kwargs) -> None:
        """Ulysses (head-split) context parallelism; a ring over the sequence cannot carry the recurrent state."""
        del kwargs
        if ring is not None or uly is None:
            raise NotImplementedError("GatedDeltaNet supports Ulysses context parallelism only: its state runs along the "
                                      "whole sequence, so the heads are split, not the sequence")
        cp = cp_mesh.size()
        if self.n_heads % cp != 0 or self.n_v_heads % cp != 0:
            raise ValueError(f"the number of key heads ({self.n_heads}) and value heads ({self.n_v_heads}) must be "
                             f"multiples of the context-parallel degree ({cp})")
        self._cp_pg, self._cp_size, self._cp_rank = cp_mesh.get_group(), cp, cp_mesh.get_local_rank()
        for conv in (self.q_conv1d, self.k_conv1d, self.v_conv1d):
            conv.apply_cp(cp_mesh)
        self.cp_enabled = cp > 1

    @torch.no_grad()
    def init_weights(self, *, init_method=None, d_model: Optional[int] = None, block_idx: int = 0, num_blocks: int = 1,
                     std: float = 0.02, generator: Optional[torch.Generator] = None) -> None:
        del init_method, d_model, block_idx, num_blocks
        for lin in (self.w_q, self.w_k, self.w_v, self.w_a, self.w_b, self.w_g, self.w_out):
            nn.init.trunc_normal_(lin.weight, mean=0.0, std=std, a=-3 * std, b=3 * std, generator=generator)
        for conv in (self.q_conv1d, self.k_conv1d, self.v_conv1d):
            bound = 1.0 / math.sqrt(conv.weight.shape[-1])
            conv.weight.uniform_(-bound, bound, generator=generator)
            if conv.bias is not None:
                conv.bias.zero_()
        # decay rates and time-step biases as in Mamba-style mixers: A in [0, 16), dt in [1e-3, 1e-1] (log-uniform)
        self.A_log.copy_(torch.empty_like(self.A_log).uniform_(0, 16, generator=generator).clamp_(min=1e-4).log())
        dt = torch.exp(torch.empty_like(self.dt_bias).uniform_(0, 1, generator=generator) * (math.log(0.1) - math.log(1e-3))
                       + math.log(1e-3)).clamp_(min=1e-4)
        self.dt_bias.copy_(dt + torch.log(-torch.expm1(-dt)))  # inverse softplus
        self.o_norm.weight.fill_(1.0)

    def num_flops_per_token(self, seq_len: int) -> int:
        del seq_len
        proj = 2 * self.d_model * (2 * self.key_dim + 2 * self.value_dim + 2 * self.n_v_heads) + 2 * self.value_dim * self.d_model
        state = 2 * 3 * self.n_v_heads * self.head_k_dim * self.head_v_dim  # decay/update/read of the state per token
        return 3 * (proj + state)


@SequenceMixerConfig.register("gated_delta_net")
@dataclass
class GatedDeltaNetConfig(SequenceMixerConfig["GatedDeltaNet"]):
    n_heads: int = 16
    n_v_heads: Optional[int] = None
    head_dim: Optional[int] = None
    expand_v: float = 2.0
    allow_neg_eigval: bool = True
    conv_size: int = 4
    conv_bias: bool = False
    norm_eps: float = 1e-5
    dtype: DType = DType.float32

    def num_params(self, d_model: int) -> int:
        n_v = self.n_v_heads if self.n_v_heads is not None else self.n_heads
        hd = self.head_dim if self.head_dim is not None else d_model // self.n_heads
        key_dim, value_dim = self.n_heads * hd, n_v * int(hd * self.expand_v)
        n = d_model * (2 * key_dim + 2 * value_dim + 2 * n_v) + value_dim * d_model  # projections
        n += 2 * n_v  # A_log, dt_bias
        n += self.conv_size * (2 * key_dim + value_dim) + (2 * key_dim + value_dim if self.conv_bias else 0)
        n += int(hd * self.expand_v)  # output norm
        return n

    def num_active_params(self, d_model: int) -> int:
        return self.num_params(d_model)

    def build(self, d_model: int, *, layer_idx: int = 0, n_layers: int = 1, init_device: str = "cpu", cache=None) -> GatedDeltaNet:
        del layer_idx, n_layers, cache
        kwargs = self.as_dict(exclude_none=True, recurse=False)
        kwargs["dtype"] = DType(kwargs.pop("dtype")).as_pt()
        return GatedDeltaNet(d_model=d_model, init_device=init_device, **kwargs)
