"""
Language-model head: final norm, output projection and (when labels are given) the loss
(API of src/olmo_core/nn/lm_head.py:30-562).

Two loss implementations exist: ``default`` materialises the logits with the tcgen05 GEMM and runs the
cross-entropy kernel over them; ``fused_linear`` streams row chunks through GEMM -> loss kernel -> dgrad /
wgrad GEMMs and never holds ``[N, V]`` logits (3.3 GB in fp32 for 8192 tokens of a 100k vocabulary).
With ``fused_linear`` the ``loss_div_factor`` is folded into the gradient inside the kernel.
"""

from __future__ import annotations

import logging
import math
from dataclasses import dataclass
from typing import Literal, NamedTuple, Optional, Union

import torch
import torch.nn as nn

from ..config import DType, StrEnum
from ..exceptions import OLMoConfigurationError
from .config import ModuleConfig
from .feed_forward import Linear
from .functional import cross_entropy_loss, fused_linear_cross_entropy_loss
from .layer_norm import LayerNormConfig, l2_normalize

__all__ = ["LMHeadType", "LMLossImplementation", "LMHeadConfig", "LMHead", "NormalizedLMHead", "LMOutputWithLoss"]

log = logging.getLogger(__name__)


class LMHeadType(StrEnum):
    default = "default"
    normalized = "normalized"


class LMLossImplementation(StrEnum):
    default = "default"
    fused_linear = "fused_linear"


class LMOutputWithLoss(NamedTuple):
    logits: Optional[torch.Tensor]
    loss: torch.Tensor
    ce_loss: torch.Tensor
    z_loss: Optional[torch.Tensor]


@dataclass
class LMHeadConfig(ModuleConfig):
    name: LMHeadType = LMHeadType.default
    layer_norm: Optional[LayerNormConfig] = None
    bias: Optional[bool] = None
    dtype: DType = DType.float32
    loss_implementation: LMLossImplementation = LMLossImplementation.default

    def num_params(self, d_model: int, vocab_size: int) -> int:
        bias = self.bias if self.bias is not None else self.name != LMHeadType.normalized
        n = d_model * vocab_size
        if self.layer_norm is not None:
            n += self.layer_norm.num_params(d_model)
        if bias:
            n += vocab_size
        if self.name == LMHeadType.normalized:
            n += vocab_size
        return n

    def build(self, *, d_model: int, vocab_size: int, init_device: str = "cpu") -> "LMHead":
        kwargs = self.as_dict(exclude_none=True, recurse=False)
        kwargs.pop("name")
        kwargs.update(d_model=d_model, vocab_size=vocab_size, init_device=init_device,
                      dtype=DType(kwargs.pop("dtype")).as_pt())
        try:
            if self.name == LMHeadType.default:
                return LMHead(**kwargs)
            if self.name == LMHeadType.normalized:
                return NormalizedLMHead(**kwargs)
            raise NotImplementedError(self.name)
        except TypeError as e:
            raise OLMoConfigurationError(f"invalid options for '{self.name}' {self.__class__.__name__}, {e}") from e


class LMHead(nn.Module):
    def __init__(
        self,
        *,
        d_model: int,
        vocab_size: int,
        layer_norm: Optional[LayerNormConfig] = None,
        dtype: torch.dtype = torch.float32,
        bias: bool = True,
        init_device: str = "cpu",
        loss_implementation: LMLossImplementation = LMLossImplementation.default,
    ):
        super().__init__()
        self.d_model = d_model
        self.vocab_size = vocab_size
        self.norm = layer_norm.build(d_model, init_device=init_device) if layer_norm is not None else None
        self.w_out = Linear(d_model, vocab_size, bias, dtype, init_device)
        self.loss_implementation = LMLossImplementation(loss_implementation)
        self.tp_group = None
        self.cp_group = None

    @property
    def tp_enabled(self) -> bool:
        return self.tp_group is not None

    @property
    def cp_enabled(self) -> bool:
        return self.cp_group is not None

    def forward(
        self,
        x: torch.Tensor,
        *,
        labels: Optional[torch.Tensor] = None,
        ignore_index: int = -100,
        loss_reduction: Literal["mean", "sum", "none"] = "mean",
        z_loss_multiplier: Optional[float] = None,
        loss_div_factor: Optional[Union[torch.Tensor, float]] = None,
        return_logits: Optional[bool] = None,
        logits_to_keep: Union[int, torch.Tensor] = 0,
        tp_sequence_sharded: bool = False,
    ) -> Union[torch.Tensor, LMOutputWithLoss]:
        """
        Without ``labels`` returns logits ``[B, T, V]``. With ``labels`` returns
        :class:`LMOutputWithLoss`; ``loss_div_factor`` divides the (sum- or none-reduced) losses.
        ``tp_sequence_sharded``: ``x`` is this tensor-parallel rank's ``[B, T / tp, d]`` part of the sequence (``labels``
        are whole); what is returned covers the whole sequence.
        """
        if tp_sequence_sharded and self.tp_enabled:
            return self._forward_sequence_parallel(
                x, labels=labels, ignore_index=ignore_index, loss_reduction=loss_reduction,
                z_loss_multiplier=z_loss_multiplier, loss_div_factor=loss_div_factor, return_logits=return_logits,
                logits_to_keep=logits_to_keep)
        B = x.shape[0]
        h = self.norm(x) if self.norm is not None else x
        if isinstance(logits_to_keep, int):
            if logits_to_keep != 0:
                h = h[:, -logits_to_keep:, :]
                if labels is not None:
                    labels = labels[:, -logits_to_keep:]
        else:
            h = h.gather(1, logits_to_keep.unsqueeze(-1).expand(-1, -1, h.size(-1)))
            if labels is not None:
                labels = labels.gather(1, logits_to_keep)

        if labels is None:
            if return_logits is False:
                raise RuntimeError("'return_logits=False' is only valid when 'labels' is provided")
            return self._project(h)

        if loss_div_factor is not None and loss_reduction == "mean":
            raise RuntimeError("'loss_div_factor' only makes sense with 'sum' or 'none' loss reduction")
        div = self._effective_div_factor(loss_div_factor)

        logits: Optional[torch.Tensor] = None
        fused = (
            self.loss_implementation == LMLossImplementation.fused_linear
            and self.w_out.bias is None
            and loss_reduction in ("sum", "mean")
            and not return_logits
        )
        if fused:
            scale = None
            if div is not None:
                scale = (1.0 / div) if torch.is_tensor(div) else torch.tensor(1.0 / div, dtype=torch.float32, device=h.device)
            loss, z_loss = fused_linear_cross_entropy_loss(
                h.reshape(-1, self.d_model), self.w_out.weight, labels.reshape(-1), ignore_index=ignore_index,
                reduction=loss_reduction, compute_z_loss=z_loss_multiplier is not None,
                z_loss_multiplier=z_loss_multiplier or 1e-4, loss_scale=scale,
            )
            ce_loss = loss - z_loss if z_loss is not None else loss
        else:
            logits = self._project(h)
            ce_loss, z_loss = cross_entropy_loss(
                logits.reshape(-1, logits.shape[-1]), labels.reshape(-1), ignore_index=ignore_index,
                reduction=loss_reduction, compute_z_loss=z_loss_multiplier is not None,
                z_loss_multiplier=z_loss_multiplier or 1e-4,
            )
            if loss_reduction == "none":
                ce_loss = ce_loss.view(B, -1)
                z_loss = z_loss.view(B, -1) if z_loss is not None else None
            if div is not None:
                ce_loss = ce_loss / div
                z_loss = z_loss / div if z_loss is not None else None
            loss = ce_loss + z_loss if z_loss is not None else ce_loss
        if return_logits is False:
            logits = None
        return LMOutputWithLoss(logits=logits, loss=loss, ce_loss=ce_loss.detach(),
                                z_loss=z_loss.detach() if z_loss is not None else None)

    def _forward_sequence_parallel(self, x, *, labels, ignore_index, loss_reduction, z_loss_multiplier, loss_div_factor,
                                   return_logits, logits_to_keep):
        """
        Tensor parallelism: norm, projection and loss run on this rank's ``T / tp`` tokens with whole weights (what the
        reference's sequence-parallel plan does, src/olmo_core/nn/lm_head.py:366-417); loss sums are added over the
        group, logits and per-token losses are gathered along the sequence. The head's parameters get partial gradients.
        """
        from ..parallel.tensor import gather_from_sequence_parallel, local_sequence_shard, sum_partials

        group = self.tp_group
        if not (isinstance(logits_to_keep, int) and logits_to_keep == 0):
            # "the last n positions" live on the last ranks only: evaluate on the gathered sequence (inference path;
            # every rank repeats the work, so this form is not meant for training)
            full = gather_from_sequence_parallel(x, group)
            return self.forward(full, labels=labels, ignore_index=ignore_index, loss_reduction=loss_reduction,
                                z_loss_multiplier=z_loss_multiplier, loss_div_factor=loss_div_factor,
                                return_logits=return_logits, logits_to_keep=logits_to_keep)
        B = x.shape[0]
        h = self.norm(x) if self.norm is not None else x
        if labels is None:
            if return_logits is False:
                raise RuntimeError("'return_logits=False' is only valid when 'labels' is provided")
            return gather_from_sequence_parallel(self._project(h), group)
        if loss_div_factor is not None and loss_reduction == "mean":
            raise RuntimeError("'loss_div_factor' only makes sense with 'sum' or 'none' loss reduction")
        div = self._effective_div_factor(loss_div_factor)
        local_labels = local_sequence_shard(labels, group)
        with_z = z_loss_multiplier is not None
        logits: Optional[torch.Tensor] = None
        if loss_reduction == "none":
            local_logits = self._project(h)
            ce, z = cross_entropy_loss(local_logits.reshape(-1, local_logits.shape[-1]), local_labels.reshape(-1),
                                       ignore_index=ignore_index, reduction="none", compute_z_loss=with_z,
                                       z_loss_multiplier=z_loss_multiplier or 1e-4)
            ce_loss = gather_from_sequence_parallel(ce.view(B, -1), group)
            z_loss = gather_from_sequence_parallel(z.view(B, -1), group) if z is not None else None
            if return_logits:
                logits = gather_from_sequence_parallel(local_logits, group)
            if div is not None:
                ce_loss = ce_loss / div
                z_loss = z_loss / div if z_loss is not None else None
        else:
            # The scale is applied to the local sums BEFORE they are added: the fused loss forms its gradients during
            # the forward pass, which is only right when the gradient that later arrives at its output is one.
            scale: Optional[torch.Tensor] = None
            if loss_reduction == "mean":
                import torch.distributed as dist

                count = (local_labels != ignore_index).sum().float()
                dist.all_reduce(count, group=group)
                scale = 1.0 / count.clamp(min=1.0)
            elif div is not None:
                scale = (1.0 / div) if torch.is_tensor(div) else torch.tensor(1.0 / div, dtype=torch.float32, device=h.device)
            fused = (self.loss_implementation == LMLossImplementation.fused_linear and self.w_out.bias is None
                     and not return_logits)
            if fused:
                total, z = fused_linear_cross_entropy_loss(
                    h.reshape(-1, self.d_model), self.w_out.weight, local_labels.reshape(-1), ignore_index=ignore_index,
                    reduction="sum", compute_z_loss=with_z, z_loss_multiplier=z_loss_multiplier or 1e-4, loss_scale=scale)
                ce = total - z if z is not None else total
            else:
                local_logits = self._project(h)
                ce, z = cross_entropy_loss(local_logits.reshape(-1, local_logits.shape[-1]), local_labels.reshape(-1),
                                           ignore_index=ignore_index, reduction="sum", compute_z_loss=with_z,
                                           z_loss_multiplier=z_loss_multiplier or 1e-4)
                if scale is not None:
                    ce = ce * scale
                    z = z * scale if z is not None else None
                if return_logits:
                    logits = gather_from_sequence_parallel(local_logits, group)
            parts = [ce.float().reshape(1)] + ([z.float().reshape(1)] if z is not None else [])
            totals = sum_partials(torch.cat(parts), group)  # one exchange for both sums
            ce_loss = totals[0]
            z_loss = totals[1] if z is not None else None
        loss = ce_loss + z_loss if z_loss is not None else ce_loss
        if return_logits is False:
            logits = None
        return LMOutputWithLoss(logits=logits, loss=loss, ce_loss=ce_loss.detach(),
                                z_loss=z_loss.detach() if z_loss is not None else None)

    def _project(self, h: torch.Tensor) -> torch.Tensor:
        return self.w_out(h)

    def _effective_div_factor(self, div):
        """
        Context-parallel ranks each see ``1/CP`` of a sequence while gradients are *averaged* over the
        combined data x context group, so each rank's partial loss is scaled up by CP.
        """
        if div is None:
            return None
        if self.cp_enabled:
            import torch.distributed as dist

            div = div / dist.get_world_size(self.cp_group)
        return div

    def apply_tp(self, tp_mesh, **kwargs) -> None:
        from ..parallel.tensor import shard_lm_head_

        shard_lm_head_(self, tp_mesh)

    def apply_cp(self, cp_mesh) -> None:
        self.cp_group = cp_mesh.get_group()

    def num_flops_per_token(self, seq_len: int) -> int:
        return 6 * sum(p.numel() for p in self.parameters())


class NormalizedLMHead(LMHead):
    """nGPT head: logits scaled per vocabulary entry by the learned ``sz``."""

    def __init__(self, *, d_model: int, vocab_size: int, dtype: torch.dtype = torch.float32, init_device: str = "cpu",
                 loss_implementation: LMLossImplementation = LMLossImplementation.default, **unused):
        super().__init__(d_model=d_model, vocab_size=vocab_size, layer_norm=None, bias=False, dtype=dtype,
                         init_device=init_device, loss_implementation=LMLossImplementation.default)
        self.sz_init_value = 1.0
        self.sz_init_scaling = 1.0 / math.sqrt(d_model)
        self.sz = nn.Parameter(torch.empty(vocab_size, dtype=dtype, device=init_device))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.sz.device.type != "meta":
            nn.init.constant_(self.sz, self.sz_init_scaling)

    def _project(self, h: torch.Tensor) -> torch.Tensor:
        sz = self.sz * (self.sz_init_value / self.sz_init_scaling)
        return sz.to(h.dtype) * self.w_out(h)

    @torch.no_grad()
    def normalize_matrices(self) -> None:
        self.w_out.weight.copy_(l2_normalize(self.w_out.weight, dim=-1))
