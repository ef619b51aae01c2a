"""
Beaker integration (options of src/olmo_core/train/callbacks/beaker.py:25-175): when the job runs inside a Beaker
batch job, rank 0 keeps the workload description up to date with the training progress, cross-links the W&B / Comet
run and stores the run config and the Python environment in the result directory.
"""

from __future__ import annotations

import dataclasses
import json
import logging
import os
import platform
import subprocess
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any, ClassVar, Dict, Optional

from ...distributed.utils import get_rank
from .callback import Callback
from .comet import CometCallback
from .wandb import WandBCallback

log = logging.getLogger(__name__)

__all__ = ["BeakerCallback", "BEAKER_RESULT_DIR"]

BEAKER_RESULT_DIR = "/results"


def _in_beaker_batch_job() -> bool:
    return "BEAKER_JOB_ID" in os.environ and os.environ.get("BEAKER_JOB_KIND", "batch") == "batch"


@dataclass
class BeakerCallback(Callback):
    priority: ClassVar[int] = min(CometCallback.priority - 1, WandBCallback.priority - 1)  # after the trackers

    experiment_id: Optional[str] = None
    update_interval: Optional[int] = None
    description: Optional[str] = None
    enabled: Optional[bool] = None
    """None: enabled exactly when running inside a Beaker batch job."""
    config: Optional[Dict[str, Any]] = None
    result_dir: str = BEAKER_RESULT_DIR

    _url: Optional[str] = dataclasses.field(repr=False, default=None)
    _last_update: Optional[float] = dataclasses.field(repr=False, default=None)

    def post_attach(self) -> None:
        if self.enabled is None:
            self.enabled = _in_beaker_batch_job()

    def _active(self) -> bool:
        return bool(self.enabled) and get_rank() == 0

    def pre_train(self) -> None:
        if not self._active():
            return
        from ...launch.beaker import get_beaker_client, get_beaker_experiment_id

        if self.experiment_id is None:
            self.experiment_id = get_beaker_experiment_id()
        with get_beaker_client() as beaker:
            beaker_url = beaker.workload.url(beaker.workload.get(self.experiment_id))
        log.info(f"Running in Beaker workload {beaker_url}")
        for cb in self.trainer.callbacks.values():
            if isinstance(cb, WandBCallback) and cb.enabled and cb.run is not None:
                cb.run.config.update({"beaker_experiment_url": beaker_url, "beaker_experiment_id": self.experiment_id})
                self._url = self._url or cb.run.get_url()
            elif isinstance(cb, CometCallback) and cb.enabled and cb.exp is not None:
                cb.exp.log_parameter("beaker_experiment_url", beaker_url)
                cb.exp.log_parameter("beaker_experiment_id", self.experiment_id)
                self._url = self._url or cb.exp.url
        out = Path(self.result_dir) / "olmo-core"
        out.mkdir(parents=True, exist_ok=True)
        if self.config is not None:
            (out / "config.json").write_text(json.dumps(self.config))
        try:
            with (out / "requirements.txt").open("w") as f:
                f.write(f"# python={platform.python_version()}\n")
                f.flush()
                subprocess.call(["pip", "freeze"], stdout=f, stderr=subprocess.DEVNULL, timeout=10)
        except Exception as e:
            log.warning(f"Error saving Python packages: {e}")
        self._update()

    def post_step(self) -> None:
        interval = self.update_interval or self.trainer.metrics_collect_interval
        if self._active() and self.step % interval == 0:
            if self._last_update is None or time.monotonic() - self._last_update > 10:  # rate limit
                self._update()

    def post_train(self) -> None:
        if self._active():
            self._update()

    def _update(self) -> None:
        self.trainer.run_bookkeeping_op(self._set_description, op_name="beaker_set_description", allow_multiple=False,
                                        distributed=False)
        self._last_update = time.monotonic()

    def _set_description(self) -> None:
        from ...launch.beaker import get_beaker_client

        text = f"[{self.trainer.training_progress}] "
        if self.description is not None:
            text += f"{self.description}\n"
        if self._url is not None:
            text += f"{self._url} "
        try:
            with get_beaker_client() as beaker:
                beaker.workload.update(beaker.workload.get(self.experiment_id), description=text.strip())
        except Exception as e:  # the description is cosmetic: never fail the run over it
            log.warning(f"Failed to update Beaker description: {e}")
