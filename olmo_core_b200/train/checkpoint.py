"""
Trainer checkpoints (layout and API of src/olmo_core/train/checkpoint.py:51-520)::

    <save_folder>/step{N}/
        .metadata.json              {"ephemeral": bool, "version": "..."}   written last, by rank 0
        train/rank{r}.pt            trainer / data-loader / callback / RNG state of rank r (torch.save)
        model_and_optim/            sharded checkpoint of the train module (see distributed.checkpoint)

Local checkpoints are assembled in ``step{N}-tmp`` and renamed into place once every rank has finished, so a
directory named ``step{N}`` is always complete; ``.metadata.json`` marks a remote checkpoint as complete.
"""

from __future__ import annotations

import json
import logging
import os
import re
import shutil
import tempfile
from concurrent.futures import Future
from contextlib import contextmanager
from dataclasses import dataclass
from pathlib import Path
from typing import Any, ClassVar, Dict, Generator, Optional, Tuple, Union

import torch
import torch.distributed as dist

from ..aliases import PathOrStr
from ..config import Config
from ..distributed.checkpoint import (
    async_save_state_dict,
    get_checkpoint_metadata,
    load_state_dict,
    save_state_dict,
)
from ..distributed.utils import barrier, broadcast_object, get_fs_local_rank, get_rank, is_distributed
from ..exceptions import OLMoConfigurationError
from ..io import (
    clear_directory,
    dir_is_empty,
    file_exists,
    is_url,
    join_path,
    list_directory,
    normalize_path,
    read_bytes,
    read_text,
    upload,
)
from ..utils import wait_for
from ..version import VERSION
from .train_module import TrainModule

log = logging.getLogger(__name__)

__all__ = ["CheckpointerConfig", "Checkpointer", "CheckpointMetadata"]


@dataclass
class CheckpointerConfig(Config):
    """Serialisable settings of a :class:`Checkpointer`."""

    work_dir: Optional[str] = None
    save_overwrite: Optional[bool] = None
    pre_download: bool = False
    save_thread_count: Optional[int] = None
    load_thread_count: Optional[int] = None
    throttle_uploads: bool = False

    def build(self, process_group: Optional[dist.ProcessGroup] = None, **kwargs) -> "Checkpointer":
        opts = {k: v for k, v in self.as_dict(recurse=False).items() if v is not None}
        opts.update(kwargs)
        if opts.get("work_dir") is None:
            raise OLMoConfigurationError("'work_dir' must be provided to build a Checkpointer")
        return Checkpointer(process_group=process_group, **opts)


@dataclass
class CheckpointMetadata(Config):
    ephemeral: Optional[bool] = None
    version: str = VERSION


@dataclass
class Checkpointer:
    METADATA_FNAME: ClassVar[str] = ".metadata.json"
    CHECKPOINT_DIR: ClassVar[str] = "step{step}"
    FS_TIMEOUT: ClassVar[float] = 120.0

    work_dir: Path
    save_overwrite: bool = False
    pre_download: bool = False
    process_group: Optional[dist.ProcessGroup] = None
    save_thread_count: Optional[int] = None
    load_thread_count: Optional[int] = None
    throttle_uploads: bool = False

    def __post_init__(self):
        self.work_dir = Path(self.work_dir)
        if get_fs_local_rank() == 0:
            self.work_dir.mkdir(parents=True, exist_ok=True)

    # -- saving ------------------------------------------------------------------------------------------
    def save(self, dir: PathOrStr, train_module: TrainModule, train_state: Dict[str, Any], ephemeral: bool = False) -> None:
        """Write a complete checkpoint to ``dir`` (blocking)."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dir = normalize_path(dir)
        with self._staging(dir) as stage:
            self._write_train_state(dir, stage, train_state)
            target = f"{dir}/model_and_optim" if is_url(dir) else str(stage / "model_and_optim")
            save_state_dict(target, train_module.state_dict_to_save(), process_group=self.process_group,
                            thread_count=self.save_thread_count, throttle_uploads=self.throttle_uploads,
                            save_overwrite=True)
        self._write_metadata(dir, CheckpointMetadata(ephemeral=ephemeral))

    def save_async(self, dir: PathOrStr, train_module: TrainModule, train_state: Dict[str, Any],
                   ephemeral: bool = False) -> Future:
        """
        Stage the state in host memory and return; the future completes when the checkpoint is on storage.
        ``process_group`` must be a CPU (gloo) group reserved for checkpointing when running distributed.
        """
        if is_distributed() and self.process_group is None:
            raise OLMoConfigurationError("a checkpointer needs a dedicated CPU process group for async saves")
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dir = self._prepare_dir(normalize_path(dir))
        # Asynchronous saves go straight to the final location: the rename of a staging directory would have to
        # happen after the background writes of every rank. ``.metadata.json`` (written last) marks completion.
        with self._train_state_dir(dir) as train_dir:
            torch.save(train_state, train_dir / f"rank{get_rank()}.pt")
        fut = async_save_state_dict(f"{dir}/model_and_optim", train_module.state_dict_to_save(),
                                    process_group=self.process_group, thread_count=self.save_thread_count,
                                    throttle_uploads=self.throttle_uploads, save_overwrite=True)
        done: Future = Future()

        def finish(f) -> None:
            try:
                f.result()
                self._write_metadata(dir, CheckpointMetadata(ephemeral=ephemeral))
                done.set_result(None)
            except BaseException as e:  # surfaced to whoever waits on the future
                done.set_exception(e)

        fut.add_done_callback(finish)
        return done

    # -- loading ----------------------------------------------------------------------------------------
    def load(self, dir: PathOrStr, train_module: TrainModule, *, load_trainer_state: Optional[bool] = None,
             load_optim_state: Optional[bool] = None) -> Optional[Dict[str, Any]]:
        """
        Restore ``train_module`` from ``dir`` and return the trainer state of this rank (falling back to rank 0's
        when the world size changed), or None if there is none and it was not required.
        """
        dir = normalize_path(dir)
        trainer_state: Optional[Dict[str, Any]] = None
        if load_trainer_state is not False:
            for candidate in (f"{dir}/train/rank{get_rank()}.pt", f"{dir}/train/rank0.pt"):
                try:
                    import io

                    trainer_state = torch.load(io.BytesIO(read_bytes(candidate)), weights_only=False, map_location="cpu")
                    break
                except FileNotFoundError:
                    continue
            if load_trainer_state is True and trainer_state is None:
                raise FileNotFoundError(f"Missing trainer state in checkpoint dir '{dir}'")

        module_dir = f"{dir}/model_and_optim"
        metadata = None
        if get_rank(self.process_group) == 0:
            try:
                metadata = get_checkpoint_metadata(module_dir)
            except FileNotFoundError:
                if trainer_state is not None:
                    raise
                # a bare model(+optim) checkpoint rather than a trainer checkpoint
                metadata = get_checkpoint_metadata(dir)
                module_dir = dir
        module_dir = broadcast_object(module_dir, group=self.process_group) if is_distributed() else module_dir
        if metadata is None:
            metadata = get_checkpoint_metadata(module_dir)
        state = train_module.state_dict_to_load(metadata, optim=load_optim_state)
        load_state_dict(module_dir, state, process_group=self.process_group,
                        pre_download=is_url(dir) and self.pre_download, work_dir=self.work_dir,
                        thread_count=self.load_thread_count)
        train_module.load_state_dict(state)
        return trainer_state

    def write_file(self, dir: PathOrStr, fname: str, contents: Union[str, bytes]) -> PathOrStr:
        """Write a small auxiliary file into a checkpoint (or save) folder. Call from one rank only."""
        dir = normalize_path(dir)
        mode = "wb" if isinstance(contents, bytes) else "w"
        if not is_url(dir):
            Path(dir).mkdir(parents=True, exist_ok=True)
            path = Path(dir) / fname
            if path.exists() and not self.save_overwrite:
                raise FileExistsError(path)
            tmp = path.with_name(path.name + ".tmp")
            with open(tmp, mode) as f:
                f.write(contents)
            tmp.replace(path)
            return path
        tmp_dir = Path(tempfile.mkdtemp(dir=self.work_dir))
        try:
            with open(tmp_dir / fname, mode) as f:
                f.write(contents)
            target = f"{dir}/{fname}"
            upload(tmp_dir / fname, target, save_overwrite=self.save_overwrite)
            return target
        finally:
            shutil.rmtree(tmp_dir, ignore_errors=True)

    # -- discovery ------------------------------------------------------------------------------------------
    @classmethod
    def checkpoint_dirname(cls, step: int) -> str:
        return cls.CHECKPOINT_DIR.format(step=step)

    @classmethod
    def dir_is_checkpoint(cls, dir: PathOrStr) -> bool:
        dir = normalize_path(dir)
        if file_exists(f"{dir}/.metadata"):  # bare model(+optim) checkpoint
            return True
        return all(file_exists(f"{dir}/{rel}") for rel in ("train/rank0.pt", "model_and_optim/.metadata", cls.METADATA_FNAME))

    @classmethod
    def find_checkpoints(cls, dir: PathOrStr, ephemeral: Optional[bool] = None) -> Generator[Tuple[int, str], None, None]:
        """Yield ``(step, path)`` of every complete checkpoint directly under ``dir``."""
        dir = normalize_path(dir)
        pattern = re.compile("^" + cls.CHECKPOINT_DIR.format(step=r"(\d+)") + "$")
        for path in list_directory(dir):
            m = pattern.match(os.path.basename(str(path).rstrip("/")))
            if m is None or not cls.dir_is_checkpoint(path):
                continue
            if ephemeral is not None:
                try:
                    meta = json.loads(read_text(join_path(path, cls.METADATA_FNAME)))
                except FileNotFoundError:
                    meta = {}
                if bool(meta.get("ephemeral") or False) != ephemeral:
                    continue
            yield int(m.group(1)), str(path)

    @classmethod
    def contains_checkpoint(cls, dir: PathOrStr) -> bool:
        if cls.dir_is_checkpoint(dir):
            return True
        try:
            next(cls.find_checkpoints(dir))
            return True
        except (StopIteration, FileNotFoundError):
            return False

    @classmethod
    def latest_checkpoint(cls, dir: PathOrStr) -> str:
        found = sorted(cls.find_checkpoints(normalize_path(dir)))
        if not found:
            raise FileNotFoundError(f"No checkpoints found in '{dir}'")
        return found[-1][1]

    # -- internals -------------------------------------------------------------------------------------------
    def _prepare_dir(self, dir: str) -> str:
        """Make sure the final directory may be written: empty, or cleared when overwriting is allowed."""
        if get_rank() == 0:
            if not dir_is_empty(dir):
                if self.save_overwrite:
                    clear_directory(dir)
                else:
                    raise FileExistsError(f"'{dir}' already exists, use 'save_overwrite' to overwrite it")
            if not is_url(dir):
                Path(dir).mkdir(parents=True, exist_ok=True)
        barrier()
        if not is_url(dir):
            wait_for(Path(dir).exists, f"'{dir}' to be created", timeout=self.FS_TIMEOUT)
        return dir

    @contextmanager
    def _train_state_dir(self, dir: str) -> Generator[Path, None, None]:
        if is_url(dir):
            tmp = Path(tempfile.mkdtemp(dir=self.work_dir))
            try:
                yield tmp
                for f in tmp.iterdir():
                    upload(f, f"{dir}/train/{f.name}", save_overwrite=self.save_overwrite)
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
        else:
            train_dir = Path(dir) / "train"
            if get_fs_local_rank() == 0:
                train_dir.mkdir(parents=True, exist_ok=True)
            wait_for(train_dir.exists, f"'{train_dir}' to be created", timeout=self.FS_TIMEOUT)
            yield train_dir

    def _write_train_state(self, dir: str, stage: Path, train_state: Dict[str, Any]) -> None:
        train_dir = stage / "train"
        if is_url(dir) or get_fs_local_rank() == 0:
            train_dir.mkdir(parents=True, exist_ok=True)
        wait_for(train_dir.exists, f"'{train_dir}' to be created", timeout=self.FS_TIMEOUT)
        torch.save(train_state, train_dir / f"rank{get_rank()}.pt")

    def _write_metadata(self, dir: str, metadata: CheckpointMetadata) -> None:
        if get_rank() == 0:
            self.write_file(dir, self.METADATA_FNAME, json.dumps(metadata.as_dict(json_safe=True)))

    @contextmanager
    def _staging(self, dir: str) -> Generator[Path, None, None]:
        """
        A directory to assemble the checkpoint in. Local target: ``<dir>-tmp`` beside it, renamed to ``dir`` by
        rank 0 when all ranks are done. Remote target: a per-rank temporary directory under ``work_dir`` whose
        files are uploaded to ``dir`` on exit.
        """
        self._prepare_dir(dir) if is_url(dir) else self._check_final(dir)
        if is_url(dir):
            stage = Path(tempfile.mkdtemp(dir=self.work_dir))
        else:
            stage = Path(dir.rstrip("/") + "-tmp")
            if get_fs_local_rank() == 0:
                shutil.rmtree(stage, ignore_errors=True)
                stage.mkdir(parents=True, exist_ok=True)
            barrier()
            wait_for(stage.exists, f"'{stage}' to be created", timeout=self.FS_TIMEOUT)
        try:
            yield stage
            barrier()
            if is_url(dir):
                for f in stage.rglob("*"):
                    if f.is_file():
                        upload(f, f"{dir}/{f.relative_to(stage).as_posix()}", save_overwrite=self.save_overwrite)
            elif get_fs_local_rank() == 0:
                if Path(dir).exists():
                    shutil.rmtree(dir)
                stage.replace(dir)
            barrier()
            if not is_url(dir):
                wait_for(Path(dir).exists, f"'{dir}' to appear", timeout=self.FS_TIMEOUT)
        finally:
            if is_url(dir):
                shutil.rmtree(stage, ignore_errors=True)

    def _check_final(self, dir: str) -> None:
        if get_rank() == 0 and not dir_is_empty(dir) and not self.save_overwrite:
            raise FileExistsError(f"'{dir}' already exists, use 'save_overwrite' to overwrite it")
        barrier()
