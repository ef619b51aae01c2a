"""
Launch a training script on the GPUs of this node: one process per GPU under ``torchrun``, rendezvous on the loopback
address. This is the launch path a single 8 x B200 NVSwitch box needs; cluster schedulers wrap the same command.
"""

from __future__ import annotations

import os
import subprocess
import sys
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..config import Config

__all__ = ["LocalLaunchConfig"]


@dataclass
class LocalLaunchConfig(Config):
    cmd: List[str]
    num_gpus: Optional[int] = None  # default: every visible GPU
    master_port: int = 29400
    env_vars: Dict[str, str] = field(default_factory=dict)

    def build_command(self) -> List[str]:
        n = self.num_gpus
        if n is None:
            import torch

            n = max(torch.cuda.device_count(), 1)
        cmd = list(self.cmd)
        if cmd and cmd[0].endswith(".py"):
            cmd = [cmd[0], *cmd[1:]]
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                "--master-addr", "127.0.0.1", "--master-port", str(self.master_port), *cmd]

    def launch(self, check: bool = True) -> int:
        env = {**os.environ, "OMP_NUM_THREADS": "8", "NUM_NODES": "1", **self.env_vars}
        return subprocess.run(self.build_command(), env=env, check=check).returncode
