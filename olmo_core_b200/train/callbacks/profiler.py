"""
``torch.profiler`` driver (options of src/olmo_core/train/callbacks/profiler.py:21-195): profiles ``active``
steps after ``skip_first + wait + warmup`` steps, ``repeat`` times, on the selected ranks, and stores a Chrome
trace per cycle under ``<save_folder>/profiler/``.
"""

from __future__ import annotations

import logging
from contextlib import ExitStack
from dataclasses import dataclass
from typing import Optional

from ...distributed.parallel import get_cp_mesh, get_dp_mesh, get_ep_mesh, get_pp_mesh, get_tp_mesh, get_world_mesh
from ...distributed.utils import get_rank
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["ProfilerCallback"]

_MESH_GETTERS = {"dp": get_dp_mesh, "tp": get_tp_mesh, "cp": get_cp_mesh, "pp": get_pp_mesh, "ep": get_ep_mesh}


@dataclass
class ProfilerCallback(Callback):
    skip_first: int = 0
    wait: int = 1
    warmup: int = 5
    active: int = 3
    repeat: int = 1
    with_stack: bool = True
    profile_memory: bool = False
    enable_cuda_sync_events: bool = False
    enabled: bool = True
    nvtx: bool = True
    """Bracket every kernel launcher call and every transformer block with an NVTX range while profiling."""
    ranks: Optional[str] = None
    """``None``: rank 0 only; ``"all"``; or ``"dp"|"tp"|"cp"|"pp"|"ep"``: the first rank of each such group."""

    _exit_stack = None
    _profiler = None
    _first_batch: bool = True

    def _should_profile_rank(self) -> bool:
        if self.ranks is None:
            return get_rank() == 0
        if self.ranks == "all":
            return True
        if self.ranks not in _MESH_GETTERS:
            raise ValueError(f"Unknown rank shortcut '{self.ranks}'")
        mesh = get_world_mesh()
        if mesh is None:
            log.warning("No world mesh available, profiling rank 0 only")
            return get_rank() == 0
        try:
            return _MESH_GETTERS[self.ranks](mesh).get_local_rank() == 0
        except (RuntimeError, KeyError, ValueError) as e:
            log.warning(f"No '{self.ranks}' mesh dimension ({e}), profiling rank 0 only")
            return get_rank() == 0

    def pre_train(self) -> None:
        if not self.enabled or not self._should_profile_rank():
            return
        from torch.profiler import ProfilerActivity, profile, schedule

        activities = [ProfilerActivity.CPU]
        if self.trainer.device.type == "cuda":
            activities.append(ProfilerActivity.CUDA)
        experimental = None
        if self.enable_cuda_sync_events:
            from torch.profiler import _ExperimentalConfig

            experimental = _ExperimentalConfig(enable_cuda_sync_events=True)
        self._exit_stack = ExitStack()
        if self.nvtx and self.trainer.device.type == "cuda":
            from ...ops import _lib

            _lib.set_nvtx(True)
            self._exit_stack.callback(_lib.set_nvtx, False)
        self._profiler = self._exit_stack.enter_context(profile(
            activities=activities, record_shapes=False, profile_memory=self.profile_memory, with_stack=self.with_stack,
            schedule=schedule(wait=self.wait, warmup=self.warmup, active=self.active, repeat=self.repeat,
                              skip_first=self.skip_first),
            on_trace_ready=self._on_trace_ready, experimental_config=experimental,
        ))
        self._first_batch = True

    def pre_load_batch(self) -> None:
        if self._profiler is None:
            return
        if self._first_batch:
            self._first_batch = False
        else:
            self._profiler.step()

    def _on_trace_ready(self, prof) -> None:
        for key in ("self_cuda_time_total", "self_cpu_time_total"):
            log.info(f"Profile by {key} at step {prof.step_num}:\n{prof.key_averages().table(sort_by=key, row_limit=32)}")
        out_dir = self.trainer.work_dir / "profiler"
        out_dir.mkdir(parents=True, exist_ok=True)
        trace = out_dir / f"rank-{get_rank()}-step-{prof.step_num}.chrome_trace.json.gz"
        prof.export_chrome_trace(str(trace))
        log.info(f"Chrome trace saved to '{self.trainer.persist_working_file(trace)}'")

    def close(self) -> None:
        if self._exit_stack is not None:
            self._exit_stack.close()
            self._exit_stack = self._profiler = None
