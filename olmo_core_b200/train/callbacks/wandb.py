"""
Weights & Biases logging (options of src/olmo_core/train/callbacks/wandb.py:21-185). Rank 0 owns the run; a run
that gets one of ``cancel_tags`` attached in the W&B UI is canceled at the next check.
"""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ...distributed.utils import get_rank
from ...exceptions import OLMoEnvironmentError
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["WandBCallback"]

WANDB_API_KEY_ENV_VAR = "WANDB_API_KEY"


@dataclass
class WandBCallback(Callback):
    priority = 0  # type: ignore[assignment]

    enabled: bool = True
    name: Optional[str] = None
    project: Optional[str] = None
    entity: Optional[str] = None
    group: Optional[str] = None
    tags: Optional[List[str]] = None
    notes: Optional[str] = None
    config: Optional[Dict[str, Any]] = None
    cancel_tags: Optional[List[str]] = field(default_factory=lambda: ["cancel", "canceled", "cancelled"])
    cancel_check_interval: Optional[int] = None

    _wandb = None
    _run_path: Optional[str] = None
    _finalized: bool = False

    @property
    def wandb(self):
        if self._wandb is None:
            import wandb  # deferred: optional dependency

            self._wandb = wandb
        return self._wandb

    @property
    def run(self):
        return self.wandb.run

    @property
    def run_path(self) -> Optional[str]:
        return self._run_path

    @property
    def finalized(self) -> bool:
        return self._finalized

    def _active(self) -> bool:
        return self.enabled and get_rank() == 0

    def finalize(self, exit_code: int = 0) -> None:
        if not self._finalized and self._active() and self._wandb is not None and self.run is not None:
            self.wandb.finish(exit_code=exit_code, quiet=True)
        self._finalized = True

    def pre_train(self) -> None:
        if not self._active():
            return
        if WANDB_API_KEY_ENV_VAR not in os.environ:
            raise OLMoEnvironmentError(f"missing env var '{WANDB_API_KEY_ENV_VAR}'")
        wandb_dir = self.trainer.work_dir / "wandb"
        wandb_dir.mkdir(parents=True, exist_ok=True)
        self.wandb.init(dir=wandb_dir, project=self.project, entity=self.entity, group=self.group, name=self.name,
                        tags=self.tags, notes=self.notes, config=self.config)
        self._run_path = self.run.path
        self._finalized = False

    def log_metrics(self, step: int, metrics: Dict[str, float]) -> None:
        if self._active() and not self._finalized:
            self.wandb.log(metrics, step=step)

    def post_step(self) -> None:
        interval = self.cancel_check_interval or self.trainer.cancel_check_interval
        if self._active() and self.step % interval == 0:
            self.trainer.run_bookkeeping_op(self.check_if_canceled, op_name="wandb-cancel-check", distributed=False,
                                            allow_multiple=False)

    def on_error(self, exc: BaseException) -> None:
        del exc
        self.finalize(exit_code=1)

    def close(self) -> None:
        self.finalize()

    def check_if_canceled(self) -> None:
        if not self._active() or not self.cancel_tags or self._run_path is None:
            return
        try:
            run = self.wandb.Api(api_key=os.environ[WANDB_API_KEY_ENV_VAR]).run(self._run_path)
            hit = next((t for t in run.tags or [] if t.lower() in self.cancel_tags), None)
            if hit is not None:
                self.trainer.cancel_run(f"canceled from W&B tag '{hit}'")
        except Exception as e:  # network hiccups must not take the run down
            log.warning(f"Failed to check W&B cancellation tags: {e}")
