"""
Export of the final checkpoint in Hugging Face format at the end of training
(options of src/olmo_core/train/callbacks/hf_converter.py:20-222).

All ranks take part in gathering the full model state (each contributes its rows of the sharded parameters);
rank 0 converts and writes ``<checkpoint>-hf`` (or ``output_folder``).
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch

from ...config import DType
from ...distributed.utils import barrier, get_full_tensor, get_rank
from .callback import Callback
from .checkpointer import CheckpointerCallback

log = logging.getLogger(__name__)

__all__ = ["HFConverterCallback"]


@dataclass
class HFConverterCallback(Callback):
    enabled: bool = True
    output_folder: Optional[str] = None
    dtype: Optional[DType] = DType.bfloat16
    validate: bool = False
    """Compare the converted model's logits with the original's on random tokens."""
    debug: bool = False
    tokenizer_id: Optional[str] = None
    max_sequence_length: Optional[int] = None
    device: Optional[str] = None
    moe_capacity_factor: Optional[float] = None

    def _latest_checkpoint_path(self) -> Optional[str]:
        ckpt = next((cb for cb in self.trainer.callbacks.values() if isinstance(cb, CheckpointerCallback)), None)
        if ckpt is None:
            log.warning("CheckpointerCallback not found, cannot determine latest checkpoint path")
            return None
        return ckpt._latest_checkpoint_path or (ckpt._checkpoints[-1] if ckpt._checkpoints else None)

    def _full_model_state_dict(self) -> Dict[str, Any]:
        """Collective: every rank must call it. Full tensors land in host memory."""
        from ...distributed.checkpoint import model_state

        return {name: get_full_tensor(t).detach().to("cpu") for name, t in model_state(self.trainer.train_module.model).items()}

    def post_train(self) -> None:
        try:
            self._convert()
        finally:
            barrier()

    def _convert(self) -> None:
        if not self.enabled:
            return
        path = self._latest_checkpoint_path()
        if path is None:
            log.warning("No checkpoint found, skipping HF conversion")
            return
        try:
            from ...nn.hf import convert_checkpoint_to_hf, load_config
        except ImportError:
            log.error("HF conversion needs the 'transformers' library, which could not be imported")
            return
        experiment_config: Optional[dict] = None
        if get_rank() == 0:
            try:
                experiment_config = load_config(path)
            except Exception as e:
                log.error(f"Failed to load config from checkpoint: {e}")
        state = self._full_model_state_dict()
        if get_rank() != 0:
            return
        if experiment_config is None or experiment_config.get("model") is None:
            log.error("No model config found beside the checkpoint, cannot convert to HF format")
            return
        tokenizer_cfg = experiment_config.get("dataset", {}).get("tokenizer") or {}
        output = self.output_folder if self.output_folder is not None else f"{path}-hf"
        convert_checkpoint_to_hf(
            original_checkpoint_path=path, output_path=output, transformer_config_dict=experiment_config["model"],
            tokenizer_config_dict=tokenizer_cfg, model_state_dict=state, dtype=self.dtype, tokenizer_id=self.tokenizer_id,
            max_sequence_length=self.max_sequence_length, validate=self.validate, debug=self.debug,
            device=torch.device(self.device) if self.device else None, moe_capacity_factor=self.moe_capacity_factor,
        )
        log.info(f"Converted checkpoint to Hugging Face format at '{output}'")
