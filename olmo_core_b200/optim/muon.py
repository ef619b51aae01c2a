"""
Muon / NorMuon (role of src/olmo_core/optim/muon.py:43-237, which wraps the external ``dion`` package).
Implemented in-tree: matrices are updated with the Newton-Schulz orthogonalised momentum, all other
parameters (embeddings, LM head, vectors) with AdamW.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Type

import torch
import torch.nn as nn
from torch.optim.optimizer import Optimizer

from ..config import StrEnum
from .config import MatrixAwareOptimConfig, OptimConfig

__all__ = ["Muon", "MuonConfig", "NorMuonConfig", "MuonAdjustLRStrategy", "newton_schulz"]


def newton_schulz(g: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Quintic Newton-Schulz iteration that drives the singular values of ``g`` towards one."""
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g.to(torch.bfloat16 if g.is_cuda else torch.float32)
    transposed = x.shape[-2] > x.shape[-1]
    if transposed:
        x = x.transpose(-2, -1)
    x = x / (x.norm(dim=(-2, -1), keepdim=True) + eps)
    for _ in range(steps):
        xxT = x @ x.transpose(-2, -1)
        x = a * x + (b * xxT + c * (xxT @ xxT)) @ x
    if transposed:
        x = x.transpose(-2, -1)
    return x.to(g.dtype)


class MuonAdjustLRStrategy(StrEnum):
    """How the step of an orthogonalised ``[rows, cols]`` update is scaled (src/olmo_core/optim/muon.py:35-40)."""

    spectral_norm = "spectral_norm"
    """``sqrt(max(1, rows / cols))``: keeps the update's spectral norm comparable across widths (learning-rate transfer)."""
    rms_norm = "rms_norm"
    """``0.2 * sqrt(max(rows, cols))``: the update's RMS matches AdamW's, so AdamW learning rates carry over."""

    def scale(self, rows: int, cols: int) -> float:
        if self == MuonAdjustLRStrategy.spectral_norm:
            return max(1.0, rows / cols) ** 0.5
        return 0.2 * max(rows, cols) ** 0.5


class Muon(Optimizer):
    def __init__(self, params, lr: float = 0.02, mu: float = 0.95, betas: Tuple[float, float] = (0.9, 0.95),
                 weight_decay: float = 0.01, eps: float = 1e-8, nesterov: bool = True, ns_steps: int = 5,
                 normalize: bool = False, adjust_lr: Optional[str] = "spectral_norm", cautious_wd: bool = False):
        super().__init__(params, dict(lr=lr, mu=mu, betas=betas, weight_decay=weight_decay, eps=eps, nesterov=nesterov,
                                      ns_steps=ns_steps, normalize=normalize, algorithm="muon", adjust_lr=adjust_lr,
                                      cautious_wd=cautious_wd))

    @torch.no_grad()
    def step(self, closure=None) -> None:
        if closure is not None:
            with torch.enable_grad():
                closure()
        for group in self.param_groups:
            algo = group.get("algorithm", "muon")
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad
                state = self.state[p]
                if algo == "muon" and p.ndim >= 2:
                    if not state:
                        state["momentum"] = torch.zeros_like(p)
                        if group["normalize"]:
                            state["row_var"] = torch.zeros(p.shape[0], 1, device=p.device, dtype=p.dtype)
                    buf = state["momentum"].mul_(group["mu"]).add_(g)
                    upd = g.add(buf, alpha=group["mu"]) if group["nesterov"] else buf
                    upd = newton_schulz(upd.reshape(upd.shape[0], -1), group["ns_steps"]).view_as(p)
                    if group["normalize"]:  # NorMuon: per-row second-moment normalisation of the orthogonal update
                        v = state["row_var"].mul_(group["betas"][1]).add_(upd.pow(2).mean(dim=-1, keepdim=True), alpha=1 - group["betas"][1])
                        upd = upd / (v.sqrt() + group["eps"])
                        upd = upd * (upd.numel() ** 0.5 / (upd.norm() + group["eps"])) * 0.2
                    elif group.get("adjust_lr") is not None:
                        upd = upd * MuonAdjustLRStrategy(group["adjust_lr"]).scale(p.shape[0], p[0].numel())
                    if group.get("cautious_wd"):  # decay only the entries that the update is already shrinking
                        p.addcmul_(p, (upd * p > 0).to(p.dtype), value=-group["lr"] * group["weight_decay"])
                    else:
                        p.mul_(1 - group["lr"] * group["weight_decay"])
                    p.add_(upd, alpha=-group["lr"])
                else:
                    if not state:
                        state["step"] = 0
                        state["exp_avg"] = torch.zeros_like(p)
                        state["exp_avg_sq"] = torch.zeros_like(p)
                    state["step"] += 1
                    b1, b2 = group["betas"]
                    state["exp_avg"].lerp_(g, 1 - b1)
                    state["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                    bc1, bc2 = 1 - b1 ** state["step"], 1 - b2 ** state["step"]
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                    p.addcdiv_(state["exp_avg"], (state["exp_avg_sq"] / bc2).sqrt().add_(group["eps"]), value=-group["lr"] / bc1)


@OptimConfig.register("muon")
@dataclass
class MuonConfig(MatrixAwareOptimConfig[Muon]):
    # defaults of src/olmo_core/optim/muon.py:60-90
    lr: float = 0.01
    mu: float = 0.95
    betas: Tuple[float, float] = (0.9, 0.95)
    weight_decay: float = 0.1
    eps: float = 1e-8
    nesterov: bool = False
    ns_steps: int = 5
    scalar_lr: Optional[float] = None
    normalize: bool = False
    adjust_lr: Optional[MuonAdjustLRStrategy] = MuonAdjustLRStrategy.rms_norm
    cautious_wd: bool = False
    flatten: bool = True
    """Tensors with more than two dimensions are always treated as ``[shape[0], -1]`` matrices."""
    use_triton: bool = False
    """Accepted for compatibility; the orthogonalisation runs on the in-tree GEMM path either way."""

    @classmethod
    def optimizer(cls) -> Type[Muon]:
        return Muon

    def build_groups(self, model: nn.Module, strict: bool = True) -> List[Dict[str, Any]]:
        cats = self.categorize(model)
        named = dict(model.named_parameters())
        adam_lr = self.scalar_lr if self.scalar_lr is not None else self.lr
        groups = []
        if cats["matrix"]:
            groups.append({"params": [named[n] for n in cats["matrix"]], "algorithm": "muon"})
        for cat, lr in (("embed", self.embedding_lr), ("lm_head", self.lm_head_lr), ("vector", self.vector_lr)):
            if cats[cat]:
                groups.append({"params": [named[n] for n in cats[cat]], "algorithm": "adamw", "lr": lr if lr is not None else adam_lr})
        return groups

    def build(self, model: nn.Module, strict: bool = True) -> Muon:
        kwargs = self.as_dict()
        for k in ("group_overrides", "compile", "fixed_fields", "embedding_lr", "lm_head_lr", "vector_lr", "scalar_lr",
                  "flatten", "use_triton"):
            kwargs.pop(k)
        optim = Muon(self.build_groups(model, strict), **kwargs)
        for g in optim.param_groups:
            g.setdefault("initial_lr", g["lr"])
        return optim


@OptimConfig.register("normuon")
@dataclass
class NorMuonConfig(MuonConfig):
    normalize: bool = True
