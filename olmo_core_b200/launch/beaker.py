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
    "BEAKER_RESULT_DIR",
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
