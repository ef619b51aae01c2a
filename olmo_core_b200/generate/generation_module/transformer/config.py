"""Builder of :class:`TransformerGenerationModule` (src/olmo_core/generate/generation_module/transformer/config.py)."""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Union

import torch
import torch.distributed as dist

from ....aliases import PathOrStr
from ....config import Config, DType
from ....float8 import Float8Config
from ....nn.transformer import TransformerConfig
from ....train.train_module.transformer.config import TransformerDataParallelConfig
from ..config import GenerationConfig

log = logging.getLogger(__name__)

__all__ = ["TransformerGenerationModuleConfig"]


@dataclass
class TransformerGenerationModuleConfig(Config):
    generation_config: GenerationConfig
    compile_model: bool = False
    float8_config: Optional[Float8Config] = None
    dp_config: Optional[TransformerDataParallelConfig] = None
    state_dict_load_opts: Optional[Dict[str, Any]] = None
    load_key_mapping: Optional[Dict[str, str]] = None
    dtype: Optional[DType] = None
    """The dtype to build the model in."""

    def build(self, checkpoint_dir: Union[PathOrStr, List[PathOrStr]], transformer_config: Optional[TransformerConfig] = None,
              device: Optional[torch.device] = None, process_group: Optional[dist.ProcessGroup] = None,
              work_dir: Optional[PathOrStr] = None, pre_download: bool = True, load_thread_count: Optional[int] = None):
        from .generation_module import TransformerGenerationModule

        kwargs = self.as_dict(exclude_none=True, recurse=False)
        dtype = kwargs.pop("dtype", None)
        dirs = list(checkpoint_dir) if isinstance(checkpoint_dir, (list, tuple)) else [checkpoint_dir]
        return TransformerGenerationModule.from_checkpoints(
            dirs, transformer_config=transformer_config, device=device, process_group=process_group, work_dir=work_dir,
            pre_download=pre_download, load_thread_count=load_thread_count, dtype=DType(dtype) if dtype is not None else None,
            **kwargs)
