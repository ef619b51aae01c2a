"""
Learning-rate schedulers (API of src/olmo_core/optim/scheduler.py:21-1131). A scheduler maps
``(initial_lr, current, t_max)`` -- in steps or tokens -- to a learning rate; :meth:`Scheduler.set_lr`
applies it to an optimizer param group using the trainer's progress.

The shapes are assembled from three primitives: a linear ramp up from ``warmup_min_lr``, a linear ramp down
to ``decay_min_lr`` and a generic interpolation (linear or half-cosine) between two rates.
"""

from __future__ import annotations

import logging
import warnings
from abc import ABCMeta, abstractmethod
from dataclasses import dataclass, field
from math import cos, pi, sqrt
from typing import TYPE_CHECKING, Any, Dict, List, Optional, Union

import torch

from ..config import Config, Registrable, StrEnum
from ..exceptions import OLMoConfigurationError
from .config import INITIAL_LR_FIELD, LR_FIELD

if TYPE_CHECKING:
    from ..train import Trainer

__all__ = [
    "SchedulerUnits",
    "Scheduler",
    "ConstantScheduler",
    "ConstantWithWarmup",
    "WSD",
    "PowerLR",
    "LinearWithWarmup",
    "InvSqrtWithWarmup",
    "CosWithWarmup",
    "HalfCosWithWarmup",
    "CosWithWarmupAndLinearDecay",
    "ComposableSchedulerStageType",
    "ComposableSchedulerStage",
    "OverrideDecay",
    "ComposableScheduler",
    "SequentialScheduler",
    "WSDS",
    "ExponentialScheduler",
]

log = logging.getLogger(__name__)
LR = Union[float, torch.Tensor]


class SchedulerUnits(StrEnum):
    steps = "steps"
    tokens = "tokens"


def _ramp_up(peak: LR, current: int, warmup: int, floor: float = 0.0) -> LR:
    if isinstance(peak, float):
        assert 0 <= floor < peak
    return floor + (peak - floor) * min(current, warmup) / warmup


def _ramp_down(peak: LR, remaining: int, decay: int, floor: float = 0.0) -> LR:
    if isinstance(peak, float):
        assert 0 <= floor < peak
    return floor + (peak - floor) * min(remaining, decay) / decay


# aliases used by other modules / tests
_linear_warmup = _ramp_up
_linear_decay = _ramp_down


@dataclass
class Scheduler(Config, Registrable, metaclass=ABCMeta):
    lr_field: str = LR_FIELD
    initial_lr_field: str = INITIAL_LR_FIELD
    units: SchedulerUnits = SchedulerUnits.steps

    @abstractmethod
    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        raise NotImplementedError

    def set_lr(self, group: Dict[str, Any], trainer: "Trainer") -> LR:
        if self.lr_field not in group and self.initial_lr_field not in group:
            shown = "\n - ".join(f"{k}: {v}" for k, v in group.items() if k != "params")
            raise RuntimeError(
                f"learning rate field '{self.lr_field}' and initial learning rate field '{self.initial_lr_field}' "
                f"not found in optimizer param group with {len(group['params'])} parameter(s):\n - {shown}"
            )
        if group.get(self.initial_lr_field) is None:
            group[self.initial_lr_field] = group[self.lr_field]
        if self.units == SchedulerUnits.steps:
            if trainer.max_steps is None:
                raise OLMoConfigurationError("'max_steps' must be known in the trainer for step-based scheduling.")
            new_lr = self.get_lr(group[self.initial_lr_field], trainer.global_step, trainer.max_steps)
        elif self.units == SchedulerUnits.tokens:
            if trainer.max_tokens is None:
                raise OLMoConfigurationError("'max_tokens' must be known in the trainer for token-based scheduling.")
            new_lr = self.get_lr(group[self.initial_lr_field], trainer.global_train_tokens_seen, trainer.max_tokens)
        else:
            raise NotImplementedError(self.units)
        current = group.get(self.lr_field)
        if isinstance(current, torch.Tensor):
            current.fill_(new_lr)
        else:
            group[self.lr_field] = new_lr
        return new_lr


@dataclass
class _WarmupMixin:
    """``warmup`` (absolute) or ``warmup_fraction`` (of ``t_max``); ``warmup_steps`` is the deprecated alias."""

    def _init_warmup(self, default_warmup: Optional[int] = 2000) -> None:
        if getattr(self, "warmup", None) is None and getattr(self, "warmup_steps", None) is not None:
            self.warmup = self.warmup_steps  # type: ignore[attr-defined]
            self.warmup_steps = None  # type: ignore[attr-defined]
            warnings.warn(f"'{type(self).__name__}.warmup_steps' is deprecated, please use '.warmup' instead.", DeprecationWarning)
        if (self.warmup is None) == (self.warmup_fraction is None):  # type: ignore[attr-defined]
            if self.warmup is None and default_warmup is not None:  # type: ignore[attr-defined]
                self.warmup = default_warmup  # type: ignore[attr-defined]
            else:
                raise OLMoConfigurationError("Either 'warmup' or 'warmup_fraction' must be specified.")
        wf = self.warmup_fraction  # type: ignore[attr-defined]
        if wf is not None and not 0 <= wf <= 1:
            raise OLMoConfigurationError("'warmup_fraction' must be between 0 and 1.")

    def _warmup_len(self, t_max: int) -> int:
        return self.warmup if self.warmup is not None else round(t_max * self.warmup_fraction)  # type: ignore[attr-defined]


@dataclass
class _DecayMixin:
    def _init_decay(self) -> None:
        if getattr(self, "decay", None) is None and getattr(self, "decay_steps", None) is not None:
            self.decay = self.decay_steps  # type: ignore[attr-defined]
            self.decay_steps = None  # type: ignore[attr-defined]
            warnings.warn(f"'{type(self).__name__}.decay_steps' is deprecated, please use '.decay' instead.", DeprecationWarning)
        if self.decay is not None and self.decay_fraction is not None:  # type: ignore[attr-defined]
            self.decay_fraction = None  # an explicit length wins over the default fraction
        if self.decay is None and self.decay_fraction is None:  # type: ignore[attr-defined]
            raise OLMoConfigurationError("Either 'decay' or 'decay_fraction' must be specified.")
        df = self.decay_fraction  # type: ignore[attr-defined]
        if df is not None and not 0 <= df <= 1:
            raise OLMoConfigurationError("'decay_fraction' must be between 0 and 1.")

    def _decay_len(self, t_max: int) -> int:
        return self.decay if self.decay is not None else round(t_max * self.decay_fraction)  # type: ignore[attr-defined]


@Scheduler.register("constant")
@dataclass
class ConstantScheduler(Scheduler):
    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        return initial_lr


@Scheduler.register("constant_with_warmup")
@dataclass
class ConstantWithWarmup(Scheduler, _WarmupMixin):
    warmup: Optional[int] = None
    warmup_steps: Optional[int] = None
    warmup_fraction: Optional[float] = None
    warmup_min_lr: float = 0.0

    def __post_init__(self):
        self._init_warmup()

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        w = self._warmup_len(t_max)
        return _ramp_up(initial_lr, current, w, self.warmup_min_lr) if current <= w else initial_lr


@Scheduler.register("wsd")
@dataclass
class WSD(Scheduler, _WarmupMixin, _DecayMixin):
    """Warm-up, stable, linear decay."""

    warmup: Optional[int] = None
    warmup_steps: Optional[int] = None
    warmup_fraction: Optional[float] = None
    decay: Optional[int] = None
    decay_steps: Optional[int] = None
    decay_fraction: Optional[float] = 0.1
    warmup_min_lr: float = 0.0
    decay_min_lr: float = 0.0

    def __post_init__(self):
        self._init_warmup()
        self._init_decay()

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        w = self._warmup_len(t_max)
        if current <= w:
            return _ramp_up(initial_lr, current, w, self.warmup_min_lr)
        d = self._decay_len(t_max)
        if current >= t_max - d:
            return _ramp_down(initial_lr, t_max - current, d, self.decay_min_lr)
        return initial_lr


@Scheduler.register("power_lr")
@dataclass
class PowerLR(Scheduler, _WarmupMixin, _DecayMixin):
    """Warm-up, then ``lr * (t / warmup)^b``, then a linear tail to ``decay_min_lr``."""

    b: float = -0.51
    warmup: Optional[int] = None
    warmup_steps: Optional[int] = None
    warmup_fraction: Optional[float] = None
    warmup_min_lr: float = 0.0
    decay: Optional[int] = None
    decay_steps: Optional[int] = None
    decay_fraction: Optional[float] = 0.1
    decay_min_lr: float = 0.0

    def __post_init__(self):
        self._init_warmup()
        self._init_decay()

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        w, d = self._warmup_len(t_max), self._decay_len(t_max)
        if current <= w:
            return _ramp_up(initial_lr, current, w, self.warmup_min_lr)
        if current >= t_max - d:
            return _ramp_down(initial_lr * ((t_max - d) / w) ** self.b, t_max - current, d, self.decay_min_lr)
        return initial_lr * (current / w) ** self.b


@Scheduler.register("linear_with_warmup")
@dataclass
class LinearWithWarmup(Scheduler, _WarmupMixin):
    alpha_f: float = 0.1
    t_max: Optional[int] = None
    warmup: Optional[int] = None
    warmup_steps: Optional[int] = None
    warmup_fraction: Optional[float] = None
    warmup_min_lr: float = 0.0

    def __post_init__(self):
        self._init_warmup()

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        t_max = t_max if self.t_max is None else self.t_max
        floor = initial_lr * self.alpha_f
        w = self._warmup_len(t_max)
        if current < w:
            return _ramp_up(initial_lr, current, w, self.warmup_min_lr)
        if current >= t_max:
            return floor
        return initial_lr - (initial_lr - floor) * ((current - w) / (t_max - w))


@Scheduler.register("inv_sqrt_with_warmup")
@dataclass
class InvSqrtWithWarmup(Scheduler, _WarmupMixin):
    alpha_f: float = 0.1
    warmup: Optional[int] = None
    warmup_steps: Optional[int] = None
    warmup_fraction: Optional[float] = None
    warmup_min_lr: float = 0.0

    def __post_init__(self):
        self._init_warmup()

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        w = self._warmup_len(t_max)
        if current < w:
            return _ramp_up(initial_lr, current, w, self.warmup_min_lr)
        floor = initial_lr * self.alpha_f
        return floor + (initial_lr - floor) * sqrt(w / current)


@Scheduler.register("cos_with_warmup")
@dataclass
class CosWithWarmup(Scheduler, _WarmupMixin):
    warmup: Optional[int] = None
    warmup_steps: Optional[int] = None
    warmup_fraction: Optional[float] = None
    alpha_f: float = 0.1
    t_max: Optional[int] = None
    warmup_min_lr: float = 0.0

    def __post_init__(self):
        self._init_warmup()

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        t_max = t_max if self.t_max is None else self.t_max
        floor = initial_lr * self.alpha_f
        w = self._warmup_len(t_max)
        if current < w:
            return _ramp_up(initial_lr, current, w, self.warmup_min_lr)
        if current >= t_max:
            return floor
        return floor + (initial_lr - floor) * (1 + cos(pi * (current - w) / (t_max - w))) / 2


@Scheduler.register("half_cos_with_warmup")
@dataclass
class HalfCosWithWarmup(Scheduler, _WarmupMixin):
    """Second half of a cosine: warms up to the cosine's midpoint, then follows its falling half."""

    warmup: Optional[int] = None
    warmup_steps: Optional[int] = None
    warmup_fraction: Optional[float] = None
    alpha_f: float = 0.1
    t_max: Optional[int] = None
    warmup_min_lr: float = 0.0

    def __post_init__(self):
        self._init_warmup()

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        t_max = t_max if self.t_max is None else self.t_max
        floor = initial_lr * self.alpha_f
        w = self._warmup_len(t_max)
        if current < w:
            return _ramp_up(floor + (initial_lr - floor) / 2, current, w, self.warmup_min_lr)
        if current >= t_max:
            return floor
        span = t_max - w
        return floor + (initial_lr - floor) * (1 + cos(pi * ((current - w) + span) / (2 * span))) / 2


@Scheduler.register("cos_with_warmup_and_linear_decay")
@dataclass
class CosWithWarmupAndLinearDecay(CosWithWarmup, _DecayMixin):
    decay: Optional[int] = None
    decay_steps: Optional[int] = None
    decay_fraction: Optional[float] = 0.1
    decay_min_lr: float = 0.0

    def __post_init__(self):
        super().__post_init__()
        self._init_decay()

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        d = self._decay_len(t_max)
        if current >= t_max - d:
            knee = CosWithWarmup.get_lr(self, initial_lr, t_max - d, t_max)
            return _ramp_down(knee, t_max - current, d, self.decay_min_lr)
        return CosWithWarmup.get_lr(self, initial_lr, current, t_max)


class ComposableSchedulerStageType(StrEnum):
    linear = "linear"
    cosine = "cosine"


def _interp(shape: ComposableSchedulerStageType, start: LR, end: LR, current: int, duration: int) -> LR:
    if shape == ComposableSchedulerStageType.linear:
        return start + (end - start) * current / duration
    if shape == ComposableSchedulerStageType.cosine:
        return end + (start - end) * (1 + cos(pi * current / duration)) / 2
    raise NotImplementedError(shape)


def _abs_or_fraction(initial_lr: LR, value: Optional[float], fraction: Optional[float]) -> LR:
    return value if value is not None else initial_lr * fraction  # type: ignore[operator]


def _check_nonneg(**values: Optional[float]) -> None:
    for k, v in values.items():
        if v is not None and v < 0:
            raise OLMoConfigurationError(f"'{k}' must be >= 0.")


@dataclass
class ComposableSchedulerStage(Config):
    duration: int
    shape: ComposableSchedulerStageType = ComposableSchedulerStageType.linear
    start_lr: Optional[float] = None
    start_lr_fraction: Optional[float] = None
    end_lr: Optional[float] = None
    end_lr_fraction: Optional[float] = None

    def __post_init__(self):
        if self.duration <= 0:
            raise OLMoConfigurationError("'duration' must be > 0 for every stage.")
        if self.start_lr is not None and self.start_lr_fraction is not None:
            raise OLMoConfigurationError("Specify at most one of 'start_lr' or 'start_lr_fraction' for a stage.")
        if (self.end_lr is None) == (self.end_lr_fraction is None):
            raise OLMoConfigurationError("Specify exactly one of 'end_lr' or 'end_lr_fraction' for each stage.")
        _check_nonneg(start_lr=self.start_lr, start_lr_fraction=self.start_lr_fraction, end_lr=self.end_lr,
                      end_lr_fraction=self.end_lr_fraction)


@dataclass
class OverrideDecay(Config):
    """From ``start`` on, ignore the main schedule and decay from its value at ``start`` to the end rate."""

    start: int
    duration: int
    shape: ComposableSchedulerStageType = ComposableSchedulerStageType.linear
    end_lr: Optional[float] = None
    end_lr_fraction: Optional[float] = None

    def __post_init__(self):
        if self.start < 0:
            raise OLMoConfigurationError("'start' must be >= 0 for override decay.")
        if self.duration <= 0:
            raise OLMoConfigurationError("'duration' must be > 0 for override decay.")
        if (self.end_lr is None) == (self.end_lr_fraction is None):
            raise OLMoConfigurationError("Specify exactly one of 'end_lr' or 'end_lr_fraction' for override decay.")
        _check_nonneg(end_lr=self.end_lr, end_lr_fraction=self.end_lr_fraction)

    def lr_at(self, main_lr_at, initial_lr: LR, current: int) -> LR:
        """Rate at ``current`` (>= ``start``), given the main schedule as a function of the step."""
        start_lr = main_lr_at(self.start)
        end_lr = _abs_or_fraction(initial_lr, self.end_lr, self.end_lr_fraction)
        t = current - self.start
        return _interp(self.shape, start_lr, end_lr, t, self.duration) if t < self.duration else end_lr


@Scheduler.register("composable")
@dataclass
class ComposableScheduler(Scheduler):
    """Piecewise schedule in absolute units; ``t_max`` is ignored. After the last stage the rate stays constant."""

    stages: List[ComposableSchedulerStage] = field(default_factory=list)
    override_decay: Optional[OverrideDecay] = None
    _warned_t_max_ignored: bool = field(default=False, init=False, repr=False)

    def __post_init__(self, *args):
        if not self.stages:
            raise OLMoConfigurationError("'stages' must be specified and non-empty.")

    def _main_schedule_lr(self, initial_lr: LR, current: int) -> LR:
        current = max(current, 0)
        begin = 0
        prev_end: LR = initial_lr
        for st in self.stages:
            start = prev_end if st.start_lr is None and st.start_lr_fraction is None else _abs_or_fraction(
                initial_lr, st.start_lr, st.start_lr_fraction)
            end = _abs_or_fraction(initial_lr, st.end_lr, st.end_lr_fraction)
            if current < begin + st.duration:
                return _interp(st.shape, start, end, current - begin, st.duration)
            prev_end, begin = end, begin + st.duration
        return prev_end

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        if not self._warned_t_max_ignored:
            total = sum(s.duration for s in self.stages)
            warnings.warn(f"'{type(self).__name__}' ignores 't_max'; the schedule is defined absolutely by stage "
                          f"durations (total={total}, t_max={t_max}).", UserWarning, stacklevel=2)
            self._warned_t_max_ignored = True
        current = max(current, 0)
        if self.override_decay is None or current < self.override_decay.start:
            return self._main_schedule_lr(initial_lr, current)
        return self.override_decay.lr_at(lambda t: self._main_schedule_lr(initial_lr, t), initial_lr, current)


@Scheduler.register("sequential")
@dataclass
class SequentialScheduler(Scheduler):
    """Chain schedulers: scheduler ``i`` runs for ``schedulers_max[i]`` units, the last until the end."""

    schedulers: List[Scheduler] = field(default_factory=lambda: [ConstantWithWarmup()])
    schedulers_max: Optional[List[int]] = None
    schedulers_max_steps: Optional[List[int]] = None
    override_decay: Optional[OverrideDecay] = None
    _warned_t_max_ignored: bool = field(default=False, init=False, repr=False)

    def __post_init__(self, *args):
        if self.schedulers_max is None and self.schedulers_max_steps is not None:
            self.schedulers_max, self.schedulers_max_steps = self.schedulers_max_steps, None
            warnings.warn(f"'{type(self).__name__}.schedulers_max_steps' is deprecated, please use '.schedulers_max' instead.",
                          DeprecationWarning)
        if self.schedulers_max is None:
            raise OLMoConfigurationError("'schedulers_max' must be specified")
        if len(self.schedulers_max) == len(self.schedulers):
            self.schedulers_max = list(self.schedulers_max[:-1])  # the last scheduler runs to the end
        if len(self.schedulers_max) + 1 != len(self.schedulers):
            raise OLMoConfigurationError(
                f"Max steps must be set for all schedulers except the last when using '{type(self).__name__}'")

    def _sequential_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        assert self.schedulers_max is not None
        for sched, span in zip(self.schedulers[:-1], self.schedulers_max):
            if current <= span:
                return sched.get_lr(initial_lr, current, min(t_max, span))
            initial_lr = sched.get_lr(initial_lr, span, span)  # the next scheduler starts where this one ended
            current -= span
            t_max -= span
        assert t_max > 0
        return self.schedulers[-1].get_lr(initial_lr, current, t_max)

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        assert 0 <= current <= t_max
        if self.override_decay is None or current < self.override_decay.start:
            return self._sequential_lr(initial_lr, current, t_max)
        if not self._warned_t_max_ignored:
            warnings.warn(f"'{type(self).__name__}' ignores 't_max' once 'override_decay' is active (t_max={t_max}).",
                          UserWarning, stacklevel=2)
            self._warned_t_max_ignored = True
        return self.override_decay.lr_at(lambda t: self._sequential_lr(initial_lr, t, t_max), initial_lr, current)


@Scheduler.register("wsds")
@dataclass
class WSDS(Scheduler):
    """
    Warm-up, then repeated stable + decay periods (each period ends with a linear decay to ``decay_min_lr`` and
    the next one jumps back to its peak). The warm-up is carved out of the first period.
    """

    period_lengths: List[int] = field(default_factory=list)
    period_lr_multipliers: Optional[List[float]] = None
    warmup: Optional[int] = None
    warmup_fraction: Optional[float] = None
    decay: Optional[int] = None
    decay_fraction: Optional[float] = None
    warmup_min_lr: float = 0.0
    decay_min_lr: float = 0.0
    _cum_period_end: List[int] = field(default_factory=list, init=False, repr=False)
    _warmup_steps: int = field(default=0, init=False, repr=False)
    _adjusted_period_lengths: List[int] = field(default_factory=list, init=False, repr=False)

    def __post_init__(self, *args):
        if not self.period_lengths or any(p <= 0 for p in self.period_lengths):
            raise OLMoConfigurationError("'period_lengths' must be non-empty with positive entries.")
        if self.period_lr_multipliers is not None:
            if len(self.period_lr_multipliers) != len(self.period_lengths):
                raise OLMoConfigurationError("'period_lr_multipliers' length must match 'period_lengths' length.")
            if any(m <= 0.0 for m in self.period_lr_multipliers):
                raise OLMoConfigurationError("All entries in 'period_lr_multipliers' must be > 0.")
        if (self.warmup is None) == (self.warmup_fraction is None):
            raise OLMoConfigurationError("Exactly one of 'warmup' or 'warmup_fraction' must be specified.")
        if (self.decay is None) == (self.decay_fraction is None):
            raise OLMoConfigurationError("Exactly one of 'decay' or 'decay_fraction' must be specified.")
        for name in ("warmup_fraction", "decay_fraction"):
            v = getattr(self, name)
            if v is not None and not 0.0 <= v <= 1.0:
                raise OLMoConfigurationError(f"'{name}' must be in [0, 1].")
        if self.decay_min_lr < 0.0:
            raise OLMoConfigurationError("'decay_min_lr' must be >= 0.")
        first = self.period_lengths[0]
        self._warmup_steps = int(self.warmup) if self.warmup is not None else int(round(self.warmup_fraction * first))
        if self._warmup_steps + self._resolve_decay(first) > first:
            raise OLMoConfigurationError("First period: warmup + decay exceeds the period length.")
        for i, length in enumerate(self.period_lengths[1:], start=1):
            if self._resolve_decay(length) > length:
                raise OLMoConfigurationError(f"Period {i}: decay exceeds period length ({length}).")
        self._adjusted_period_lengths = [first - self._warmup_steps] + list(self.period_lengths[1:])
        total = 0
        self._cum_period_end = []
        for length in self._adjusted_period_lengths:
            total += length
            self._cum_period_end.append(total)

    def _resolve_decay(self, length: int) -> int:
        return int(self.decay) if self.decay is not None else int(round(self.decay_fraction * length))

    def _find_period(self, x: int) -> int:
        for idx, end in enumerate(self._cum_period_end):
            if x <= end:
                return idx
        return len(self._cum_period_end) - 1

    def _get_peak_lr(self, initial_lr: LR, pidx: int) -> LR:
        return initial_lr if self.period_lr_multipliers is None else initial_lr * self.period_lr_multipliers[pidx]

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        if current < self._warmup_steps:
            return _ramp_up(self._get_peak_lr(initial_lr, 0), current, self._warmup_steps, self.warmup_min_lr)
        t = current - self._warmup_steps
        if t >= self._cum_period_end[-1]:
            return self.decay_min_lr
        p = self._find_period(t)
        begin = 0 if p == 0 else self._cum_period_end[p - 1]
        length = self._adjusted_period_lengths[p]
        pos = min(max(t - begin, 0), length)
        d = self._resolve_decay(self.period_lengths[p])
        stable = length - d
        peak = self._get_peak_lr(initial_lr, p)
        return peak if pos < stable else _ramp_down(peak, d - (pos - stable), d, self.decay_min_lr)


@Scheduler.register("exponential")
@dataclass
class ExponentialScheduler(Scheduler):
    """Exponential *increase* from ``lr_min`` at 0 to the initial LR at ``t_max`` (for LR range tests)."""

    lr_min: float = 1e-9

    def __post_init__(self, *args):
        if self.lr_min <= 0:
            raise OLMoConfigurationError("'lr_min' must be positive.")

    def get_lr(self, initial_lr: LR, current: int, t_max: int) -> LR:
        if current >= t_max:
            return initial_lr
        if current == 0:
            return self.lr_min
        ratio = current / t_max
        growth = torch.pow(initial_lr / self.lr_min, ratio) if isinstance(initial_lr, torch.Tensor) else (initial_lr / self.lr_min) ** ratio
        return self.lr_min * growth
