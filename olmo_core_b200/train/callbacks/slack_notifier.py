"""Slack webhook notifications (options of src/olmo_core/train/callbacks/slack_notifier.py:22-140)."""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Optional

from ...aliases import PathOrStr
from ...config import StrEnum
from ...distributed.utils import get_rank
from ...exceptions import OLMoEnvironmentError
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["SlackNotifierCallback", "SlackNotificationSetting", "SLACK_WEBHOOK_URL_ENV_VAR"]

SLACK_WEBHOOK_URL_ENV_VAR = "SLACK_WEBHOOK_URL"


class SlackNotificationSetting(StrEnum):
    all = "all"
    """Start, checkpoints, epochs, end and failures."""
    end_only = "end_only"
    """Successful end and failures."""
    failure_only = "failure_only"
    none = "none"


@dataclass
class SlackNotifierCallback(Callback):
    name: Optional[str] = None
    notifications: SlackNotificationSetting = SlackNotificationSetting.end_only
    enabled: bool = True
    webhook_url: Optional[str] = None

    def _on(self, *levels: SlackNotificationSetting) -> bool:
        return self.enabled and get_rank() == 0 and self.notifications in levels

    def post_attach(self) -> None:
        if self.enabled and get_rank() == 0 and not (self.webhook_url or os.environ.get(SLACK_WEBHOOK_URL_ENV_VAR)):
            raise OLMoEnvironmentError(f"missing env var '{SLACK_WEBHOOK_URL_ENV_VAR}'")

    def pre_train(self) -> None:
        if self._on(SlackNotificationSetting.all):
            self._post_message("started")

    def post_checkpoint_saved(self, path: PathOrStr) -> None:
        if self._on(SlackNotificationSetting.all):
            self._post_message(f"saved checkpoint to '{path}'")

    def post_epoch(self) -> None:
        if self._on(SlackNotificationSetting.all):
            self._post_message(f"epoch {self.trainer.epoch} complete")

    def post_train(self) -> None:
        if self._on(SlackNotificationSetting.all, SlackNotificationSetting.end_only):
            if self.trainer.is_canceled:
                self._post_message("run canceled")
            else:
                self._post_message("completed successfully")

    def on_error(self, exc: BaseException) -> None:
        if self._on(SlackNotificationSetting.all, SlackNotificationSetting.end_only, SlackNotificationSetting.failure_only):
            self._post_message(f"failed with error:\n```\n{type(exc).__name__}: {exc}\n```")

    def _post_message(self, msg: str) -> None:
        import requests

        url = self.webhook_url or os.environ.get(SLACK_WEBHOOK_URL_ENV_VAR)
        progress = f"*Step:* {self.trainer.global_step:,d} ({self.trainer.training_progress})"
        title = f"Run `{self.name}`" if self.name else "Run"
        try:
            requests.post(url, json={"text": f"{title} {msg}\n{progress}"}, timeout=10)
        except Exception as e:
            log.warning(f"Failed to post Slack message: {e}")
