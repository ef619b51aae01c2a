"""
Dion: distributed orthonormalised updates through a rank-``r`` power iteration
(role of src/olmo_core/optim/dion.py:36-164, which wraps the external ``dion`` package).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Type

import torch
from torch.optim.optimizer import Optimizer

from .config import OptimConfig
from .muon import MuonConfig

__all__ = ["Dion", "DionConfig"]


class Dion(Optimizer):
    def __init__(self, params, lr: float = 0.01, mu: float = 0.95, betas: Tuple[float, float] = (0.9, 0.95),
                 weight_decay: float = 0.01, eps: float = 1e-8, rank_fraction: float = 0.25, rank_multiple_of: int = 1,
                 **unused):
        super().__init__(params, dict(lr=lr, mu=mu, betas=betas, weight_decay=weight_decay, eps=eps,
                                      rank_fraction=rank_fraction, rank_multiple_of=rank_multiple_of, algorithm="dion"))

    @torch.no_grad()
    def step(self, closure=None) -> None:
        if closure is not None:
            with torch.enable_grad():
                closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                g, state = p.grad, self.state[p]
                if group.get("algorithm", "dion") == "dion" and p.ndim == 2:
                    m, n = p.shape
                    r = max(1, int(min(m, n) * group["rank_fraction"]))
                    mult = max(1, int(group.get("rank_multiple_of", 1)))
                    r = min(min(m, n), -(-r // mult) * mult)  # rounded up to the multiple, never above full rank
                    if not state:
                        state["momentum"] = torch.zeros_like(p)
                        state["Q"] = torch.linalg.qr(torch.randn(n, r, device=p.device, dtype=torch.float32))[0].to(p.dtype)
                    M = state["momentum"].add_(g)
                    P = torch.linalg.qr((M @ state["Q"]).float())[0].to(p.dtype)  # [m, r] orthonormal
                    R = M.t() @ P  # [n, r]
                    M.sub_(P @ R.t(), alpha=1 - group["mu"])  # error feedback
                    Q = R / (R.norm(dim=0, keepdim=True) + group["eps"])
                    state["Q"] = Q
                    p.mul_(1 - group["lr"] * group["weight_decay"]).add_(P @ Q.t(), alpha=-group["lr"] * (m / n) ** 0.5)
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


@OptimConfig.register("dion")
@dataclass
class DionConfig(MuonConfig):
    lr: float = 0.01
    rank_fraction: float = 0.25
    rank_multiple_of: int = 1
    """Round the low-rank dimension up to a multiple of this number (useful for even sharding)."""

    @classmethod
    def optimizer(cls) -> Type[Dion]:
        return Dion

    def build(self, model, strict: bool = True) -> Dion:
        groups = self.build_groups(model, strict)
        for g in groups:
            if g.get("algorithm") == "muon":
                g["algorithm"] = "dion"
        optim = Dion(groups, lr=self.lr, mu=self.mu, betas=self.betas, weight_decay=self.weight_decay, eps=self.eps,
                     rank_fraction=self.rank_fraction, rank_multiple_of=self.rank_multiple_of)
        for g in optim.param_groups:
            g.setdefault("initial_lr", g["lr"])
        return optim
