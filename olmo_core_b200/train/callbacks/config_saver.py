"""Writes the experiment config (and data paths) into the save folder and every checkpoint (config_saver.py:18-76)."""

from __future__ import annotations

import json
import logging
from dataclasses import dataclass
from typing import Any, ClassVar, Dict, List, Optional

from ...aliases import PathOrStr
from ...distributed.utils import get_rank
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["ConfigSaverCallback"]


@dataclass
class ConfigSaverCallback(Callback):
    fname: str = "config.json"
    save_data_paths: Optional[bool] = None
    data_paths_fname: str = "data_paths.txt"
    priority: ClassVar[int] = 1

    def __post_init__(self):
        self._config: Optional[Dict[str, Any]] = None

    @property
    def config(self) -> Optional[Dict[str, Any]]:
        return self._config

    @config.setter
    def config(self, config: Dict[str, Any]) -> None:
        self._config = config

    def _data_paths(self) -> Optional[List[str]]:
        ds = getattr(self.trainer.data_loader, "dataset", None)
        paths = getattr(ds, "paths", None)
        return None if paths is None else [str(p) for p in paths]

    def _write(self, directory: Optional[PathOrStr] = None) -> None:
        if get_rank() != 0:
            return
        if self._config is None:
            log.warning(f"Config not set on {self.__class__.__name__}, doing nothing")
            return
        self.trainer.write_file(self.fname, json.dumps(self._config), dir=directory)
        if self.save_data_paths is not False and (paths := self._data_paths()):
            self.trainer.write_file(self.data_paths_fname, "\n".join(paths), dir=directory)

    def pre_train(self) -> None:
        self._write()

    def post_checkpoint_saved(self, path: PathOrStr) -> None:
        self._write(path)
