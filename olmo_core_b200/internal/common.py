"""
Cluster-dependent defaults for experiment scripts (role of src/olmo_core/internal/common.py:26-187): where data and
checkpoints live for a given cluster name, the launch configuration for a Beaker cluster and the GPU type behind a
cluster name. Everything that needs the Beaker service degrades to a local answer when no client is configured; the
``OLMO_CORE_ROOT_DIR`` environment variable overrides the data / checkpoint root.
"""

from __future__ import annotations

import logging
import os
from pathlib import Path
from typing import List, Optional, Union

import torch

from ..exceptions import OLMoEnvironmentError
from ..io import is_url
from ..launch.beaker import (
    BEAKER_RESULT_DIR,
    BeakerEnvSecret,
    BeakerEnvVar,
    BeakerLaunchConfig,
    BeakerWekaBucket,
    OLMoCoreBeakerImage,
    get_beaker_client,
)
from ..utils import generate_uuid

log = logging.getLogger(__name__)

__all__ = ["get_beaker_username", "get_root_dir", "get_work_dir", "build_launch_config", "get_gpu_type",
           "CLUSTER_TO_GPU_TYPE", "ROOT_DIR_ENV_VAR"]

ROOT_DIR_ENV_VAR = "OLMO_CORE_ROOT_DIR"
_WEKA_ROOT = "/weka/oe-training-default/ai2-llm"
_CLOUD_ROOT = "gs://ai2-llm"

CLUSTER_TO_GPU_TYPE = {
    "ai2/jupiter": "NVIDIA H100 80GB HBM3",
    "ai2/ceres": "NVIDIA H100 80GB HBM3",
    "ai2/titan": "NVIDIA B200",
}


def get_beaker_username() -> Optional[str]:
    try:
        with get_beaker_client() as beaker:
            return beaker.user_name
    except Exception:  # no client package, no token, no network
        return None


def get_root_dir(cluster: str) -> str:
    if (override := os.environ.get(ROOT_DIR_ENV_VAR)) is not None:
        return override
    if cluster.startswith("ai2/"):
        try:
            with get_beaker_client() as beaker:
                if "storage:weka" in set(beaker.cluster.get(cluster).tags):
                    return _WEKA_ROOT
        except OLMoEnvironmentError:
            pass
    return _CLOUD_ROOT


def get_work_dir(root_dir: str) -> str:
    if is_url(root_dir):
        return "./dataset-cache"
    user = get_beaker_username()
    middle = f"{user.lower()}/" if user is not None else ""
    return f"{root_dir}/checkpoints/{middle}dataset-cache"


def build_launch_config(*, name: str, cmd: List[str], cluster: str, root_dir: Optional[str] = None,
                        task_name: str = "train", workspace: str = "ai2/OLMo-core", budget: str = "ai2/oe-other",
                        nccl_debug: Union[bool, str] = False, flight_recorder: bool = False,
                        beaker_image: str = OLMoCoreBeakerImage.stable, num_nodes: int = 1,
                        num_execution_units: Optional[int] = None, step_timeout: Optional[int] = None,
                        step_soft_timeout: Optional[int] = 10 * 60) -> BeakerLaunchConfig:
    default_root = get_root_dir(cluster)
    if root_dir is None:
        root_dir = default_root
    elif root_dir != default_root:
        log.warning("Overriding the default root dir of %s (%s) with %s", cluster, default_root, root_dir)
    user = get_beaker_username()
    if user is None:
        raise RuntimeError("Environment not configured correctly for Beaker, you may be missing the BEAKER_TOKEN env var.")
    user = user.upper()

    def secret(name_: str, per_user: bool, required: bool) -> BeakerEnvSecret:
        return BeakerEnvSecret(name=name_, secret=f"{user}_{name_}" if per_user else name_, required=required)

    level = nccl_debug if isinstance(nccl_debug, str) else ("INFO" if nccl_debug else "WARN")
    env_vars = [BeakerEnvVar(name="NCCL_DEBUG", value=level)]
    if flight_recorder:  # NCCL flight recorder: dump the collective trace of every rank when a collective times out
        prefix = Path(BEAKER_RESULT_DIR) / "flightrecorder" / "nccl_trace_rank_"
        env_vars += [BeakerEnvVar(name="TORCH_NCCL_TRACE_BUFFER_SIZE", value="2000"),
                     BeakerEnvVar(name="TORCH_NCCL_DUMP_ON_TIMEOUT", value="1"),
                     BeakerEnvVar(name="TORCH_FR_DUMP_TEMP_FILE", value=str(prefix))]
    return BeakerLaunchConfig(
        name=f"{name}-{generate_uuid()[:8]}", budget=budget, cmd=cmd, task_name=task_name, workspace=workspace,
        clusters=[cluster], beaker_image=beaker_image, num_nodes=num_nodes, num_gpus=8,
        weka_buckets=([BeakerWekaBucket("oe-training-default", "/weka/oe-training-default")]
                      if root_dir.startswith("/weka/") else []),
        num_execution_units=num_execution_units, shared_filesystem=not is_url(root_dir), allow_dirty=False,
        env_vars=env_vars,
        env_secrets=[secret("BEAKER_TOKEN", True, True), secret("WANDB_API_KEY", True, True),
                     secret("COMET_API_KEY", True, False), secret("R2_ENDPOINT_URL", False, False),
                     secret("WEKA_ENDPOINT_URL", False, False), secret("SLACK_WEBHOOK_URL", False, False)],
        google_credentials_secret="GOOGLE_CREDENTIALS", aws_config_secret=f"{user}_AWS_CONFIG",
        aws_credentials_secret=f"{user}_AWS_CREDENTIALS", step_timeout=step_timeout,
        step_soft_timeout=step_soft_timeout,
    )


def get_gpu_type(cluster: str) -> str:
    if cluster in CLUSTER_TO_GPU_TYPE:
        return CLUSTER_TO_GPU_TYPE[cluster]
    if cluster == "local":
        return torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    if cluster.startswith("ai2/"):
        with get_beaker_client() as beaker:
            for node in beaker.node.list(cluster=beaker.cluster.get(cluster), limit=1):
                gpu_type = getattr(node.node_resources, "gpu_type", None)
                if gpu_type:
                    return str(getattr(gpu_type, "name", gpu_type)).replace("_", " ")
        raise RuntimeError(f"Could not determine GPU type for cluster '{cluster}'")
    raise ValueError(f"Unknown cluster '{cluster}'")
