"""
Comet.ml logging (options of src/olmo_core/train/callbacks/comet.py:21-260). Rank 0 owns the experiment; with
``auto_resume`` the experiment key travels in the trainer checkpoint so that a restarted run keeps logging to
the same experiment.
"""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ...config import StrEnum
from ...distributed.utils import get_rank
from ...exceptions import OLMoEnvironmentError
from ...utils import set_env_var
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["CometCallback", "CometNotificationSetting", "COMET_API_KEY_ENV_VAR"]

COMET_API_KEY_ENV_VAR = "COMET_API_KEY"


class CometNotificationSetting(StrEnum):
    all = "all"
    end_only = "end_only"
    failure_only = "failure_only"
    none = "none"


@dataclass
class CometCallback(Callback):
    priority = 0  # type: ignore[assignment]

    enabled: bool = True
    name: Optional[str] = None
    project: Optional[str] = None
    workspace: Optional[str] = None
    tags: Optional[List[str]] = None
    config: Optional[Dict[str, Any]] = None
    cancel_tags: Optional[List[str]] = field(default_factory=lambda: ["cancel", "canceled", "cancelled"])
    cancel_check_interval: Optional[int] = None
    notifications: CometNotificationSetting = CometNotificationSetting.none
    failure_tag: str = "failed"
    auto_resume: bool = False

    _exp = None
    _exp_key: Optional[str] = None
    _finalized: bool = False

    @property
    def exp(self):
        return self._exp

    @exp.setter
    def exp(self, exp) -> None:
        self._exp = exp

    @property
    def finalized(self) -> bool:
        return self._finalized

    def _active(self) -> bool:
        return self.enabled and get_rank() == 0

    def state_dict(self) -> Dict[str, Any]:
        return {"exp_key": self._exp_key}

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        self._exp_key = state_dict.get("exp_key")

    def finalize(self) -> None:
        if not self._finalized and self._exp is not None:
            self._exp.end()
        self._finalized = True

    def _notify(self, status: str, *levels: CometNotificationSetting) -> None:
        if self.notifications in levels and self._exp is not None:
            self._exp.send_notification(f"Experiment {self._exp.get_name()} ({self._exp.get_key()})", status=status)

    def pre_train(self) -> None:
        if not self._active():
            return
        set_env_var("COMET_DISABLE_AUTO_LOGGING", "1")
        import comet_ml as comet  # deferred: optional dependency

        if COMET_API_KEY_ENV_VAR not in os.environ:
            raise OLMoEnvironmentError(f"missing env var '{COMET_API_KEY_ENV_VAR}'")
        key = os.environ[COMET_API_KEY_ENV_VAR]
        if self.auto_resume and self._exp_key is not None:
            log.info(f"Resuming Comet logging from existing experiment '{self._exp_key}'")
            self._exp = comet.start(api_key=key, mode="get", experiment_key=self._exp_key,
                                    experiment_config=comet.ExperimentConfig(auto_output_logging="simple",
                                                                             display_summary_level=0))
        else:
            self._exp = comet.Experiment(api_key=key, project_name=self.project, workspace=self.workspace,
                                         auto_output_logging="simple", display_summary_level=0)
            self._exp_key = self._exp.get_key()
            if self.name is not None:
                self._exp.set_name(self.name)
            if self.tags:
                self._exp.add_tags(self.tags)
            if self.config is not None:
                self._exp.log_parameters(self.config)
        self._finalized = False
        self._notify("started", CometNotificationSetting.all)

    def log_metrics(self, step: int, metrics: Dict[str, float]) -> None:
        if self._active() and self._exp is not None:
            self._exp.log_metrics(metrics, step=step)

    def post_step(self) -> None:
        interval = self.cancel_check_interval or self.trainer.cancel_check_interval
        if self._active() and self.step % interval == 0:
            self.trainer.run_bookkeeping_op(self.check_if_canceled, op_name="comet-cancel-check", distributed=False,
                                            allow_multiple=False)

    def post_train(self) -> None:
        if self._active():
            self._notify("completed successfully", CometNotificationSetting.all, CometNotificationSetting.end_only)

    def on_error(self, exc: BaseException) -> None:
        del exc
        if self._active() and self._exp is not None:
            self._exp.add_tag(self.failure_tag)
            self._notify("failed", CometNotificationSetting.all, CometNotificationSetting.end_only,
                         CometNotificationSetting.failure_only)

    def close(self) -> None:
        if self._active():
            self.finalize()

    def check_if_canceled(self) -> None:
        if not self._active() or self._finalized or not self.cancel_tags or self._exp is None:
            return
        try:
            from comet_ml.api import API

            remote = API(api_key=os.environ[COMET_API_KEY_ENV_VAR]).get_experiment_by_key(self._exp.get_key())
            tags = remote.get_tags() if remote is not None else []
        except Exception as e:
            log.warning(f"Failed to check Comet cancellation tags: {e}")
            return
        if any(t.lower() in self.cancel_tags for t in tags or []):
            self.trainer.cancel_run("canceled from Comet.ml tag")
