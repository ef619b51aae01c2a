"""
Launch configuration for Ai2's Beaker scheduler (API of src/olmo_core/launch/beaker.py:66-700).

The environment probes (``is_running_in_beaker`` ...) need nothing but ``os.environ``. Building and submitting an
experiment needs the optional ``beaker`` / ``gantry`` client packages; they are imported when :meth:`launch` runs and a
clear error is raised when they are absent. :meth:`BeakerLaunchConfig.dry_run` and :meth:`build_experiment_spec` work
without them and show exactly what would be submitted.
"""

from __future__ import annotations

import dataclasses
import logging
import os
import re
import threading
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any, Dict, Generator, List, Optional, Tuple

from ..config import Config, StrEnum
from ..exceptions import OLMoConfigurationError, OLMoEnvironmentError
from ..version import VERSION
from .utils import GitConfig

log = logging.getLogger(__name__)

__all__ = [
    "is_running_in_beaker", "is_running_in_beaker_batch_job", "get_beaker_experiment_id", "get_beaker_client",
    "OLMoCoreBeakerImage", "BeakerEnvVar", "BeakerEnvSecret", "BeakerWekaBucket", "BeakerLaunchConfig",
    "BEAKER_RESULT_DIR", "GantryMonitorCallback", "main",
]

BEAKER_RESULT_DIR = "/results"
_CLIENTS = threading.local()


def is_running_in_beaker() -> bool:
    """Inside a Beaker job or session (two executor variables are checked to avoid false positives)."""
    return "BEAKER_JOB_ID" in os.environ and "BEAKER_NODE_ID" in os.environ


def is_running_in_beaker_batch_job() -> bool:
    return is_running_in_beaker() and os.environ.get("BEAKER_JOB_KIND") == "batch"


def get_beaker_experiment_id() -> Optional[str]:
    return os.environ.get("BEAKER_EXPERIMENT_ID") if is_running_in_beaker_batch_job() else None


@contextmanager
def get_beaker_client(workspace: Optional[str] = None, check_for_upgrades: Optional[bool] = None) -> Generator[Any, None, None]:
    """A Beaker client, cached per thread and workspace for the duration of the outermost ``with`` block."""
    try:
        from beaker import Beaker  # type: ignore
    except ImportError as e:
        raise OLMoEnvironmentError("the 'beaker-py' package is required to talk to Beaker") from e
    cache: Dict[Optional[str], Any] = _CLIENTS.__dict__.setdefault("clients", {})
    if workspace in cache:
        yield cache[workspace]
        return
    if workspace is None and cache:
        yield next(reversed(cache.values()))  # most recently opened
        return
    if check_for_upgrades is None:
        check_for_upgrades = not is_running_in_beaker()
    client = Beaker.from_env(check_for_upgrades=check_for_upgrades, default_workspace=workspace)
    cache[workspace] = client
    try:
        yield client
    finally:
        cache.pop(workspace, None)
        client.close()


class OLMoCoreBeakerImage(StrEnum):
    """Published images: ``stable`` for releases, ``nightly`` for the main branch, one per torch / CUDA combination."""

    stable = "olmo-core-tch291cu128-2025-11-25"
    nightly = "olmo-core-tch2100cu128-2025-11-25"
    stable_cu126 = "olmo-core-tch291cu126-2025-11-25"
    stable_cu128 = "olmo-core-tch291cu128-2025-11-25"
    stable_cu130 = "olmo-core-tch291cu130-2025-11-25"


@dataclass
class BeakerEnvVar(Config):
    name: str
    value: str


@dataclass
class BeakerEnvSecret(Config):
    name: str
    secret: str
    required: bool = True


@dataclass
class BeakerWekaBucket(Config):
    bucket: str
    mount: str


@dataclass
class BeakerLaunchConfig(Config):
    name: str
    cmd: List[str]
    torchrun: Optional[bool] = None
    budget: Optional[str] = None
    task_name: str = "train"
    workspace: Optional[str] = None
    description: Optional[str] = None
    beaker_image: str = OLMoCoreBeakerImage.stable
    num_nodes: int = 1
    num_gpus: int = 8
    shared_memory: str = "10GiB"
    clusters: List[str] = dataclasses.field(default_factory=lambda: ["ai2/jupiter"])
    hostnames: Optional[List[str]] = None
    gpu_types: Optional[List[str]] = None
    tags: Optional[List[str]] = None
    shared_filesystem: bool = False
    priority: str = "normal"
    preemptible: bool = True
    retries: Optional[int] = None
    env_vars: List[BeakerEnvVar] = dataclasses.field(default_factory=list)
    env_secrets: List[BeakerEnvSecret] = dataclasses.field(default_factory=list)
    google_credentials_secret: Optional[str] = None
    aws_config_secret: Optional[str] = None
    aws_credentials_secret: Optional[str] = None
    weka_buckets: List[BeakerWekaBucket] = dataclasses.field(default_factory=list)
    allow_dirty: bool = False
    host_networking: Optional[bool] = None
    git: Optional[GitConfig] = dataclasses.field(default_factory=GitConfig.from_env)
    result_dir: str = BEAKER_RESULT_DIR
    system_python: bool = True
    num_execution_units: Optional[int] = None
    follow: bool = True
    slack_notifications: Optional[bool] = None
    launch_timeout: Optional[int] = None
    step_timeout: Optional[int] = None
    step_soft_timeout: Optional[int] = None
    pre_setup: Optional[str] = None
    post_setup: Optional[str] = None

    # -- environment -----------------------------------------------------------------------------------------
    @property
    def default_env_vars(self) -> List[Tuple[str, str]]:
        from ..distributed.utils import OLMO_SHARED_FS_ENV_VAR
        from ..utils import LOG_FILTER_TYPE_ENV_VAR, LogFilterType

        env = [
            ("NCCL_DEBUG", "INFO"),
            (LOG_FILTER_TYPE_ENV_VAR, str(LogFilterType.local_rank0_only)),
            ("OMP_NUM_THREADS", "8"),
            ("R2_PROFILE", "R2"),
            ("S3_PROFILE", "S3"),
            ("WEKA_PROFILE", "WEKA"),
            ("NUM_NODES", str(self.num_nodes)),
            ("OLMO_CORE_VERSION", VERSION),
            ("FORCE_COLOR", "1"),
        ]
        if self.shared_filesystem:
            env.append((OLMO_SHARED_FS_ENV_VAR, "1"))
        return env

    def _get_env_vars(self) -> List[Tuple[str, str]]:
        explicit = [(v.name, v.value) for v in self.env_vars]
        taken = {name for name, _ in explicit}
        return explicit + [(n, v) for n, v in self.default_env_vars if n not in taken]

    def _uses_torchrun(self) -> bool:
        if self.torchrun is not None:
            return self.torchrun
        return self.num_gpus > 1 or (self.num_gpus >= 1 and self.num_nodes > 1)

    # -- what would run --------------------------------------------------------------------------------------
    def build_command(self) -> List[str]:
        """The command each node runs: the user command, under ``torchrun`` when more than one process is needed."""
        command = list(self.cmd)
        if command[0].endswith(".py"):
            launcher = ["python"]
            if self._uses_torchrun():
                launcher = ["torchrun", f"--nproc-per-node={self.num_gpus}"]
                if self.num_nodes > 1:
                    launcher += [f"--nnodes={self.num_nodes}:{self.num_nodes}", "--rdzv_backend=static",
                                 "--rdzv_endpoint=$BEAKER_LEADER_REPLICA_HOSTNAME:29400",
                                 "--node_rank=$BEAKER_REPLICA_RANK", "--rdzv_conf=read_timeout=420"]
                else:
                    launcher += ["--standalone", "--local-addr", "127.0.0.1"]
            command = launcher + command
        return command

    def build_experiment_spec(self) -> Dict[str, Any]:
        """A plain-dict description of the experiment (what :meth:`launch` hands to the scheduler client)."""
        if self.git is not None and self.git.is_dirty and not self.allow_dirty:
            raise RuntimeError("You have uncommitted changes! Set 'allow_dirty=True' in your launch config to force.")
        if not self.follow and (self.slack_notifications or self.step_timeout is not None
                                or self.step_soft_timeout is not None):
            raise OLMoConfigurationError("Slack notifications and step timeouts require 'follow=True'")
        multi = self.num_nodes > 1
        return {
            "name": self.name, "task_name": self.task_name, "description": self.description,
            "workspace": self.workspace, "budget": self.budget, "priority": self.priority,
            "preemptible": self.preemptible, "image": str(self.beaker_image), "command": self.build_command(),
            "env_vars": self._get_env_vars(),
            "env_secrets": [(s.name, s.secret) for s in self.env_secrets],
            "weka": [(b.bucket, b.mount) for b in self.weka_buckets], "result_dir": self.result_dir,
            "gpus": self.num_gpus, "shared_memory": self.shared_memory, "clusters": self.clusters,
            "hostnames": self.hostnames, "gpu_types": self.gpu_types, "tags": self.tags,
            "replicas": self.num_nodes if multi else None, "leader_selection": multi,
            "host_networking": self.host_networking if self.host_networking is not None else multi,
            "propagate_failure": True if multi else None, "propagate_preemption": True if multi else None,
            "synchronized_start_timeout": "90m" if multi else None, "retries": self.retries,
            "git": None if self.git is None else self.git.as_dict(),
            "pre_setup": self.pre_setup, "post_setup": self.post_setup,
        }

    def dry_run(self, **overrides) -> Dict[str, Any]:
        spec = dataclasses.replace(self, **overrides).build_experiment_spec() if overrides else self.build_experiment_spec()
        try:
            import rich

            rich.print(spec)
        except ImportError:
            print(spec)
        return spec

    def launch(self, follow: Optional[bool] = None, **overrides):
        """Submit the experiment (needs the ``beaker-gantry`` client)."""
        try:
            from gantry.api import Recipe  # type: ignore
        except ImportError as e:
            raise OLMoEnvironmentError(
                "launching on Beaker needs the 'beaker-gantry' package; use launch.local.LocalLaunchConfig for one node"
            ) from e
        spec = dataclasses.replace(self, **overrides).build_experiment_spec() if overrides else self.build_experiment_spec()
        follow = self.follow if follow is None else follow
        recipe = Recipe(
            self.cmd if not self.cmd[0].endswith(".py") else ["python", *self.cmd], name=spec["name"],
            task_name=spec["task_name"], description=spec["description"], workspace=spec["workspace"],
            budget=spec["budget"], priority=spec["priority"], preemptible=spec["preemptible"],
            beaker_image=spec["image"], env_vars=spec["env_vars"], env_secrets=spec["env_secrets"], weka=spec["weka"],
            results=spec["result_dir"], system_python=self.system_python, torchrun=self._uses_torchrun(),
            pre_setup=self.pre_setup, post_setup=self.post_setup, allow_dirty=self.allow_dirty, gpus=self.num_gpus,
            shared_memory=self.shared_memory, clusters=self.clusters, hostnames=self.hostnames, gpu_types=self.gpu_types,
            tags=self.tags, replicas=spec["replicas"], leader_selection=spec["leader_selection"],
            host_networking=spec["host_networking"], propagate_failure=spec["propagate_failure"],
            propagate_preemption=spec["propagate_preemption"],
            synchronized_start_timeout=spec["synchronized_start_timeout"], retries=self.retries,
        )
        return recipe.launch(show_logs=follow, start_timeout=self.launch_timeout, inactive_timeout=self.step_timeout,
                             inactive_soft_timeout=self.step_soft_timeout)


# ---------------------------------------------------------------------------------------------------------------
# Watching a launched workload (role of ``GantryMonitorCallback``, src/olmo_core/launch/beaker.py:698-800)
# ---------------------------------------------------------------------------------------------------------------

_STEP_LINE = re.compile(r"\[.*step=\d+.*\]")


class GantryMonitorCallback:
    """
    Follows the log stream of a launched workload: announces start / failure on Slack, warns when the trainer has not
    logged a step for ``step_soft_timeout`` seconds (at most once per ``warning_frequency``) and interrupts the workload
    after ``step_timeout`` seconds without a step. Before the first step is seen the clocks only start once the run has
    been up for half an hour (soft) / an hour (hard), so that slow start-ups are not killed.

    The hooks are the ones the ``beaker-gantry`` client calls on its callbacks (``on_start``, ``on_log``,
    ``on_no_new_logs``, ``on_timeout``, ...). ``send`` posts a message (default: the Slack webhook), ``interrupt`` stops
    the workload, ``clock`` is the time source; all three can be replaced, which is how the timeouts are tested.
    """

    def __init__(self, slack_webhook_url: Optional[str] = None, step_timeout: Optional[int] = None,
                 step_soft_timeout: Optional[int] = None, warning_frequency: int = 3600, *,
                 workload_name: str = "workload", workload_url: str = "", send=None, interrupt=None, clock=None):
        import time

        self.slack_webhook_url = slack_webhook_url
        self.step_timeout = step_timeout
        self.step_soft_timeout = step_soft_timeout
        self.warning_frequency = warning_frequency
        self.workload_name, self.workload_url = workload_name, workload_url
        self._send = send if send is not None else self._post_to_slack
        self._interrupt = interrupt
        self._clock = clock if clock is not None else time.monotonic
        self._start_time = self._clock()
        self._first_step_detected = False
        self._last_step_time = 0.0
        self._last_inactivity_warning = 0.0

    def _post_to_slack(self, text: str) -> None:
        if not self.slack_webhook_url:
            return
        try:
            import requests

            requests.post(self.slack_webhook_url, json={"text": text}, timeout=10)
        except Exception as e:  # a notification must never take the monitor down
            log.warning(f"Failed to send Slack message: {e}")

    def _say(self, emoji: str, what: str) -> None:
        link = f"<{self.workload_url}|*{self.workload_name}*>" if self.workload_url else f"*{self.workload_name}*"
        self._send(f"{emoji} Workload {link} {what}")

    def interrupt_workload(self) -> None:
        if self._interrupt is not None:
            self._interrupt()

    def on_start(self, job=None) -> None:
        self._start_time = self._clock()
        self._say(":check:", "has started! :runner:")

    def on_start_timeout(self, job=None) -> None:
        self._say(":warning:", "failed to start in time!")

    def on_log(self, job=None, log_line: str = "", log_time: float = 0.0) -> None:
        if self.step_timeout is None and self.step_soft_timeout is None:
            return
        if _STEP_LINE.search(log_line) is not None:
            self._first_step_detected = True
            self._last_step_time = self._clock()
        self._check_timeouts()

    def on_no_new_logs(self, job=None) -> None:
        self._check_timeouts()

    def _overdue(self, limit: Optional[int], grace: int, now: float) -> bool:
        if limit is None:
            return False
        armed = self._first_step_detected or (now - self._start_time) > max(limit, grace)
        return armed and (now - self._last_step_time) > limit

    def _check_timeouts(self) -> None:
        now = self._clock()
        if self._overdue(self.step_soft_timeout, 1800, now) and (now - self._last_inactivity_warning) > self.warning_frequency:
            self._say(":zzz:", "hasn't stepped recently!")
            log.warning("Workload hasn't stepped recently!")
            self._last_inactivity_warning = self._clock()
        if self._overdue(self.step_timeout, 3600, now):
            self._say(":warning:", "failed to step in time!")
            log.error("Workload has failed to step in time, stopping...")
            self.interrupt_workload()

    def on_timeout(self, job=None) -> None:
        self._say(":warning:", "failed to complete in time!")

    def _inactive(self) -> None:
        if (self._clock() - self._last_inactivity_warning) > self.warning_frequency:
            self._say(":zzz:", "appears to be inactive!")
            self._last_inactivity_warning = self._clock()

    def on_inactive_timeout(self, job=None) -> None:
        self._inactive()

    def on_inactive_soft_timeout(self, job=None) -> None:
        self._inactive()

    def on_preemption(self, job=None) -> None:
        self._say(":warning:", "was preempted!")

    def on_cancellation(self, job=None) -> None:
        self._say(":warning:", "was canceled!")

    def on_success(self, job=None, *, metrics=None, results_ds=None) -> None:
        self._say(":check:", "succeeded!")

    def on_failure(self, job=None, *, metrics=None, results_ds=None) -> None:
        self._say(":check-failed:", "failed!")


def main(argv: Optional[List[str]] = None) -> None:
    """``python -m olmo_core_b200.launch.beaker [options] -- command ...``: launch a command as a Beaker experiment."""
    import argparse

    ap = argparse.ArgumentParser(prog="olmo_core_b200.launch.beaker", description=main.__doc__)
    ap.add_argument("--name", default="olmo-core-job")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--nodes", type=int, default=1)
    ap.add_argument("--cluster", action="append", default=None, help="may be given several times")
    ap.add_argument("--budget", default=None)
    ap.add_argument("--workspace", default=None)
    ap.add_argument("--priority", default=None)
    ap.add_argument("--preemptible", action="store_true")
    ap.add_argument("--allow-dirty", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("command", nargs=argparse.REMAINDER)
    opts = ap.parse_args(argv)
    command = [c for c in opts.command if c != "--"]
    if not command:
        ap.error("a command to run is required after '--'")
    kwargs: Dict[str, Any] = dict(name=opts.name, cmd=command, num_gpus=opts.gpus, num_nodes=opts.nodes,
                                  clusters=opts.cluster or [], preemptible=opts.preemptible, allow_dirty=opts.allow_dirty)
    for key in ("budget", "workspace", "priority"):
        if getattr(opts, key) is not None:
            kwargs[key] = getattr(opts, key)
    config = BeakerLaunchConfig(**kwargs)
    if opts.dry_run:
        config.dry_run()
    else:
        config.launch(follow=True)


if __name__ == "__main__":
    main()
