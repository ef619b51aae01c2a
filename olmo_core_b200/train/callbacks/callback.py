"""
Callback interface of the trainer (hook names and order of src/olmo_core/train/callbacks/callback.py:71-185):
``post_attach`` -> (``post_checkpoint_loaded``) -> ``pre_train`` -> per epoch ``pre_epoch`` -> per step
``pre_load_batch`` -> ``pre_step`` -> ``pre_optim_step`` -> ``post_train_batch`` -> ``post_step`` ->
(``pre_log_metrics`` -> ``log_metrics``) -> (``post_checkpoint_saved``) -> ``post_epoch`` -> ``post_train``;
plus ``on_error`` and ``close``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import TYPE_CHECKING, Any, ClassVar, Dict, Optional

from ...aliases import PathOrStr
from ...config import Config

if TYPE_CHECKING:
    from ..trainer import Trainer

__all__ = ["Callback", "CallbackConfig"]


@dataclass
class Callback:
    """Base class; subclasses are dataclasses so that they serialise with the trainer config."""

    priority: ClassVar[int] = 0
    """Callbacks with a higher priority run first within each hook."""

    _trainer = None

    @property
    def trainer(self) -> "Trainer":
        assert self._trainer is not None, "callback has not been attached to a trainer"
        return self._trainer

    @trainer.setter
    def trainer(self, trainer: "Trainer") -> None:
        self._trainer = trainer

    @property
    def step(self) -> int:
        return self.trainer.global_step

    # -- state ---------------------------------------------------------------------------------------
    def state_dict(self) -> Dict[str, Any]:
        return {}

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        del state_dict

    def block_ephemeral_checkpoints(self) -> None:
        """Hold back ephemeral checkpoints for as long as at least one callback asks for it."""
        self.trainer._blocking_ephemeral_checkpoints.add(self.trainer.get_callback_name(self))

    def unblock_ephemeral_checkpoints(self) -> None:
        self.trainer._blocking_ephemeral_checkpoints.discard(self.trainer.get_callback_name(self))

    # -- hooks ---------------------------------------------------------------------------------------
    def post_attach(self) -> None:
        pass

    def post_checkpoint_loaded(self, path: PathOrStr) -> None:
        del path

    def pre_train(self) -> None:
        pass

    def pre_epoch(self) -> None:
        pass

    def pre_load_batch(self) -> None:
        pass

    def pre_step(self, batch: Dict[str, Any]) -> None:
        del batch

    def pre_optim_step(self) -> None:
        pass

    def post_train_batch(self) -> None:
        pass

    def post_step(self) -> None:
        pass

    def post_checkpoint_saved(self, path: PathOrStr) -> None:
        del path

    def pre_log_metrics(self, step: int, metrics: Dict[str, float]) -> None:
        del step, metrics

    def log_metrics(self, step: int, metrics: Dict[str, float]) -> None:
        del step, metrics

    def post_epoch(self) -> None:
        pass

    def post_train(self) -> None:
        pass

    def on_error(self, exc: BaseException) -> None:
        del exc

    def close(self) -> None:
        pass


@dataclass
class CallbackConfig(Callback, Config):
    """For callbacks whose runtime object cannot be serialised: ``build`` returns the real callback (or None)."""

    def build(self, trainer: "Trainer") -> Optional[Callback]:
        raise NotImplementedError
