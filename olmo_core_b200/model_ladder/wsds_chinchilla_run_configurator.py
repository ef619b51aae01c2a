"""
Run recipe based on Chinchilla-style scaling rules and the WSD-S schedule
(behaviour of src/olmo_core/model_ladder/wsds_chinchilla_run_configurator.py:25-255).

For ``N`` non-embedding parameters (relative to a 108M-parameter anchor):

* batch size (tokens)  ``2048 * 160 * (N / 108e6)^(2/3)``
* peak learning rate   ``0.0047 * (N / 108e6)^(-1/3) / 2 * lr_multiplier``; AdamW ``beta2`` 0.95 from 512Ki tokens, else 0.99
* duration             ``chinchilla_multiple * tokens_per_param * N`` tokens, rounded to whole batches
* schedule             warm-up of ``N`` tokens, then one warmup-stable-decay period ending at each of 0.5xC, 1xC, 2xC ...
                       so that every period end is a usable (decayed) checkpoint.
"""

from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass
from pathlib import Path
from typing import List, Optional, Tuple

from ..aliases import PathOrStr
from ..exceptions import OLMoConfigurationError
from ..optim import WSDS, OptimConfig, OptimGroupOverride, Scheduler, SchedulerUnits, SkipStepAdamWConfig
from ..train import Duration
from .base import RunConfigurator
from .utils import format_count, format_tokens

__all__ = ["WSDSChinchillaRunConfigurator"]

_ANCHOR_PARAMS = 108_000_000


@dataclass(kw_only=True)
class WSDSChinchillaRunConfigurator(RunConfigurator):
    chinchilla_multiple: float  # total duration as a multiple of Chinchilla-optimal; a power of two >= 0.5
    decay_fraction: float = 0.1  # share of each period spent decaying
    tokens_per_param: int = 20
    lr_multiplier: float = 1.0
    stepped_schedule: bool = False  # scale the peak LR of the period that ends at DxC by 1/sqrt(D)

    def __post_init__(self):
        if self.chinchilla_multiple < 0.5 or not math.log2(self.chinchilla_multiple).is_integer():
            raise OLMoConfigurationError("'chinchilla_multiple' must be at least 0.5 and a power of 2")
        if not 0 < self.decay_fraction < 0.5:
            raise OLMoConfigurationError("'decay_fraction' must be greater than 0.0 and less than 0.5")

    # -- scaling rules -------------------------------------------------------------------------------------
    def configure_target_batch_size(self, num_params: int) -> int:
        return round(2048 * 160 * (num_params / _ANCHOR_PARAMS) ** (2 / 3))

    def configure_duration(self, num_params: int, batch_size: int) -> Duration:
        return self._chinchilla_duration(num_params, batch_size, self.chinchilla_multiple)

    def configure_optimizer(self, num_params: int, batch_size: int) -> OptimConfig:
        lr = 0.0047 * (num_params / _ANCHOR_PARAMS) ** (-1 / 3) / 2.0 * self.lr_multiplier
        return SkipStepAdamWConfig(
            lr=lr, weight_decay=0.1, betas=(0.9, 0.95 if batch_size >= 524_288 else 0.99),
            group_overrides=[OptimGroupOverride(params=["embeddings.weight"], opts=dict(weight_decay=0.0))])

    def configure_chinchilla_periods(self, num_params: int) -> Tuple[int, List[float]]:
        """(warm-up tokens, the multiples of Chinchilla-optimal at which a period ends)."""
        top = int(math.log2(self.chinchilla_multiple))
        return num_params, [2.0 ** p for p in range(-1, top + 1)]

    def _period_ends(self, num_params: int, batch_size: int) -> List[Tuple[float, int, int]]:
        """(multiple, end in tokens, length in tokens) of every period."""
        _, multiples = self.configure_chinchilla_periods(num_params)
        out, previous = [], 0
        for c in multiples:
            end = self._chinchilla_duration(num_params, batch_size, c).value
            out.append((c, end, end - previous))
            previous = end
        return out

    def configure_lr_scheduler(self, num_params: int, batch_size: int) -> Scheduler:
        warmup, _ = self.configure_chinchilla_periods(num_params)
        periods = self._period_ends(num_params, batch_size)
        return WSDS(units=SchedulerUnits.tokens, warmup=warmup, decay_fraction=self.decay_fraction,
                    period_lengths=[length for _, _, length in periods],
                    period_lr_multipliers=[1 / math.sqrt(c) for c, _, _ in periods] if self.stepped_schedule else None)

    def configure_checkpoint_intervals(self, num_params: int, batch_size: int) -> List[Tuple[Duration, str]]:
        """Two checkpoints per period: just before its decay starts and at its end."""
        out: List[Tuple[Duration, str]] = []
        for i, (c, end, length) in enumerate(self._period_ends(num_params, batch_size), start=1):
            label = f"period {i}, {c:g}xC" if float(c).is_integer() else f"period {i}, {c}xC"
            out.append((Duration.tokens(end - round(length * self.decay_fraction)), f"{label} pre-decay"))
            out.append((Duration.tokens(end), f"{label} post-decay"))
        return out

    def _chinchilla_duration(self, num_params: int, batch_size: int, c: float) -> Duration:
        d = Duration.chinchilla_tokens(c, model_params=num_params, _tok_per_param=self.tokens_per_param)
        return dataclasses.replace(d, value=batch_size * round(d.value / batch_size))

    # -- report ------------------------------------------------------------------------------------------------
    def lr_schedule_points(self, num_params: int, batch_size: int) -> Tuple[List[int], List[float]]:
        """(tokens seen, learning rate) after every batch of the run."""
        optim = self.configure_optimizer(num_params, batch_size)
        scheduler = self.configure_lr_scheduler(num_params, batch_size)
        t_max = self.configure_duration(num_params, batch_size).value
        tokens = list(range(batch_size, t_max + batch_size, batch_size))
        return tokens, [float(scheduler.get_lr(optim.lr, t, t_max)) for t in tokens]  # type: ignore[attr-defined]

    def plot_lr_schedule(self, num_params: int, batch_size: int, *, show: bool = True,
                         save_path: Optional[PathOrStr] = None) -> Optional[PathOrStr]:
        try:
            import matplotlib.pyplot as plt  # type: ignore
        except ImportError as e:
            raise ImportError("matplotlib is required to plot the learning-rate schedule") from e
        tokens, lrs = self.lr_schedule_points(num_params, batch_size)
        warmup, _ = self.configure_chinchilla_periods(num_params)
        t_max = tokens[-1]
        fig, ax = plt.subplots(figsize=(12, 6))
        ax.plot(tokens, lrs)
        ax.grid(True)
        for c, end, _ in self._period_ends(num_params, batch_size):
            ax.axvline(x=end, color="red", linestyle="--", alpha=0.5)
            ax.text(end, 0.0, f"{c}xC", color="red", alpha=0.5, rotation=45)
        marks = [batch_size * (d.value // batch_size) for d, _ in self.configure_checkpoint_intervals(num_params, batch_size)]
        lookup = dict(zip(tokens, lrs))
        ax.scatter(marks, [lookup.get(t, 0.0) for t in marks], color="green", label="Checkpoint")
        one_x = self._chinchilla_duration(num_params, batch_size, 1.0).value
        ax.set_title(f"Learning rate schedule for a {format_count(num_params)} model out to {self.chinchilla_multiple}xC")
        ax.set_xlabel(f"Tokens\n\npeak LR={max(lrs):.6f}, batch size={format_tokens(batch_size)}, "
                      f"1xC={format_tokens(one_x)}\nwarmup={format_tokens(warmup)} / {warmup // batch_size:,d} steps, "
                      f"duration={format_tokens(t_max)} / {t_max // batch_size:,d} steps")
        ax.legend(loc="upper right")
        fig.tight_layout()
        if save_path is not None:
            Path(save_path).parent.mkdir(parents=True, exist_ok=True)
            fig.savefig(save_path)
        if show:
            plt.show()
        return save_path
