"""Config of torch's plain Adam (counterpart of src/olmo_core/optim/adam.py:9-24).

Adam without decoupled weight decay is only used for small experiments; the training recipes use ``AdamWConfig`` or
``SkipStepAdamWConfig``, whose update runs in this package's fused kernels.
"""

from dataclasses import dataclass
from typing import Optional, Tuple, Type

from torch.optim import Adam

from .config import OptimConfig

__all__ = ["AdamConfig"]


@OptimConfig.register("adam")
@dataclass
class AdamConfig(OptimConfig[Adam]):
    lr: float = 1e-3
    betas: Tuple[float, float] = (0.9, 0.999)  # decay of the first / second moment
    eps: float = 1e-8
    foreach: Optional[bool] = None  # None lets torch pick per device
    fused: Optional[bool] = None

    @classmethod
    def optimizer(cls) -> Type[Adam]:
        return Adam
