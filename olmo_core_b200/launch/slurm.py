"""
SLURM launching (role of the reference's src/scripts/lambda/{launch.sh,launch_with_retries.sh,*.sbatch}): render a batch
script that runs the node health checks and then one ``torchrun`` per node (one process per GPU), submit it with
``sbatch``, and optionally resubmit a failed job a bounded number of times.

The rendered script is plain text: :meth:`SlurmLaunchConfig.render` can be inspected or written to a file without a
cluster; :meth:`launch` needs ``sbatch`` on the PATH.
"""

from __future__ import annotations

import shlex
import shutil
import subprocess
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..config import Config
from ..exceptions import OLMoConfigurationError, OLMoEnvironmentError

__all__ = ["SlurmLaunchConfig"]


@dataclass
class SlurmLaunchConfig(Config):
    name: str
    cmd: List[str]
    """The training command, e.g. ``["python", "-m", "olmo_core_b200.scripts.train", "OLMo2-7B", ...]`` (run under torchrun)."""
    nodes: int = 1
    gpus_per_node: int = 8
    cpus_per_task: int = 96
    time_limit: str = "48:00:00"
    partition: Optional[str] = None
    account: Optional[str] = None
    log_dir: str = "logs"
    env: Dict[str, str] = field(default_factory=dict)
    setup_steps: List[str] = field(default_factory=list)
    healthchecks: bool = True
    rdzv_port: int = 29400
    max_retries: int = 0
    exclude_nodes: List[str] = field(default_factory=list)

    def __post_init__(self):
        if self.nodes < 1 or self.gpus_per_node < 1:
            raise OLMoConfigurationError("nodes and gpus_per_node must be positive")
        if not self.cmd:
            raise OLMoConfigurationError("an empty command cannot be launched")

    def render(self) -> str:
        """The text of the batch script."""
        header = [
            "#!/bin/bash",
            f"#SBATCH --job-name={self.name}",
            f"#SBATCH --nodes={self.nodes}",
            "#SBATCH --ntasks-per-node=1",
            f"#SBATCH --gpus-per-node={self.gpus_per_node}",
            f"#SBATCH --cpus-per-task={self.cpus_per_task}",
            f"#SBATCH --time={self.time_limit}",
            f"#SBATCH --output={self.log_dir}/{self.name}/%j.log",
            "#SBATCH --exclusive",
        ]
        if self.partition:
            header.append(f"#SBATCH --partition={self.partition}")
        if self.account:
            header.append(f"#SBATCH --account={self.account}")
        if self.exclude_nodes:
            header.append(f"#SBATCH --exclude={','.join(self.exclude_nodes)}")
        body = ["", "set -euo pipefail", ""]
        for k, v in sorted(self.env.items()):
            body.append(f"export {k}={shlex.quote(str(v))}")
        body += [
            'export MASTER_ADDR="$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)"',
            f"export MASTER_PORT={self.rdzv_port}",
            "export OMP_NUM_THREADS=8",
            "",
        ]
        body += list(self.setup_steps)
        if self.healthchecks:
            body += [
                "# every node checks itself first: a hot, busy or short-handed node fails the job before it wastes the others' time",
                f"srun --ntasks-per-node=1 python -m olmo_core_b200.scripts.healthcheck --expect-gpus {self.gpus_per_node}",
                "",
            ]
        torchrun = (
            f"python -m torch.distributed.run --nnodes={self.nodes} --nproc-per-node={self.gpus_per_node} "
            f'--rdzv-backend=c10d --rdzv-endpoint="$MASTER_ADDR:$MASTER_PORT" --rdzv-id="$SLURM_JOB_ID" '
        )
        inner = self.cmd[1:] if self.cmd[0] in ("python", "python3") else self.cmd
        body.append("srun --ntasks-per-node=1 --kill-on-bad-exit=1 " + torchrun + " ".join(shlex.quote(c) for c in inner))
        return "\n".join(header + body) + "\n"

    def launch(self, script_path: Optional[str] = None, dry_run: bool = False) -> Optional[str]:
        """Write the script, submit it, return the job id (``None`` for a dry run)."""
        import os
        import tempfile

        text = self.render()
        if script_path is None:
            fd, script_path = tempfile.mkstemp(prefix=f"{self.name}-", suffix=".sbatch")
            os.close(fd)
        with open(script_path, "w") as f:
            f.write(text)
        if dry_run:
            return None
        if shutil.which("sbatch") is None:
            raise OLMoEnvironmentError("sbatch not found: SLURM jobs can only be submitted from a cluster login node")
        os.makedirs(os.path.join(self.log_dir, self.name), exist_ok=True)
        last_err = ""
        for _ in range(self.max_retries + 1):
            proc = subprocess.run(["sbatch", "--parsable", script_path], capture_output=True, text=True)
            if proc.returncode == 0:
                return proc.stdout.strip().split(";")[0]
            last_err = proc.stderr
        raise OLMoEnvironmentError(f"sbatch failed: {last_err}")
