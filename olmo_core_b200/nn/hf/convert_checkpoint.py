"""
Converting a trainer checkpoint to a Hugging Face folder, with optional validation of the result
(role of src/olmo_core/nn/hf/convert_checkpoint.py).
"""

from __future__ import annotations

import json
import logging
import tempfile
from pathlib import Path
from typing import Any, Dict, Optional

import torch

from ...aliases import PathOrStr
from ...config import DType
from ...io import file_exists, join_path, normalize_path, read_text

log = logging.getLogger(__name__)

__all__ = ["convert_checkpoint_to_hf", "load_config", "validate_conversion"]


def load_config(checkpoint_input_dir: PathOrStr) -> Optional[dict]:
    """The experiment config saved beside a checkpoint (``config.json`` in the step folder or in its parent)."""
    base = normalize_path(checkpoint_input_dir)
    for candidate in (join_path(base, "config.json"), join_path(str(base).rstrip("/").rsplit("/", 1)[0], "config.json")):
        if file_exists(candidate):
            return json.loads(read_text(candidate))
    log.warning(f"No config.json found for checkpoint '{base}'")
    return None


def convert_checkpoint_to_hf(original_checkpoint_path: PathOrStr, output_path: PathOrStr, transformer_config_dict: Dict[str, Any],
                             tokenizer_config_dict: Dict[str, Any], *, model_state_dict: Optional[Dict[str, Any]] = None,
                             dtype: Optional[DType] = None, tokenizer_id: Optional[str] = None,
                             max_sequence_length: Optional[int] = None, validate: bool = True, debug: bool = False,
                             device: Optional[torch.device] = None, moe_capacity_factor: Optional[float] = None,
                             validation_device: Optional[torch.device] = None,
                             validation_sliding_window: Optional[int] = None) -> None:
    """
    Build the model from its config, load weights (from ``model_state_dict`` or from the sharded checkpoint), write the
    Hugging Face folder (model + tokenizer + generation config), optionally compare logits of both models.
    """
    del moe_capacity_factor, validation_sliding_window, debug
    from ...distributed.checkpoint import load_model_and_optim_state
    from ..transformer import TransformerConfig
    from .checkpoint import save_hf_model

    config = TransformerConfig.from_dict(dict(transformer_config_dict))
    model = config.build(init_device="cpu")
    if model_state_dict is not None:
        model.load_state_dict({k: torch.as_tensor(v) for k, v in model_state_dict.items()}, strict=True)
    else:
        path = normalize_path(original_checkpoint_path)
        module_dir = join_path(path, "model_and_optim")
        load_model_and_optim_state(module_dir if file_exists(join_path(module_dir, ".metadata")) else path, model)
    vocab_size = tokenizer_config_dict.get("vocab_size")
    state = {k: v for k, v in model.state_dict().items()}
    torch_dtype = DType(dtype).as_pt() if dtype is not None else None
    save_hf_model(output_path, state, model, dtype=torch_dtype, vocab_size=vocab_size, save_overwrite=True)

    identifier = tokenizer_id or tokenizer_config_dict.get("identifier")
    if identifier is not None:
        try:
            from transformers import AutoTokenizer, GenerationConfig

            tok = AutoTokenizer.from_pretrained(identifier)
            if max_sequence_length is not None:
                tok.model_max_length = max_sequence_length
            tok.save_pretrained(output_path)
            GenerationConfig(pad_token_id=tokenizer_config_dict.get("pad_token_id"),
                             eos_token_id=tokenizer_config_dict.get("eos_token_id"),
                             bos_token_id=tokenizer_config_dict.get("bos_token_id")).save_pretrained(output_path)
        except Exception as e:  # no network / unknown tokenizer: the weights are still exported
            log.warning(f"Could not export tokenizer '{identifier}': {e}")
    if validate:
        validate_conversion(output_path, model, vocab_size or model.vocab_size, device=validation_device or device, dtype=torch_dtype)


@torch.no_grad()
def validate_conversion(hf_path: PathOrStr, model, vocab_size: int, debug: bool = False,
                        dtype: Optional[torch.dtype] = None, device: Optional[torch.device] = None,
                        sliding_window: Optional[int] = None, *, rtol: float = 1e-3, atol: float = 1e-3, **kwargs) -> None:
    """Feed the same random token ids through both models and compare the logits over the real vocabulary
    (``debug`` and ``sliding_window`` are accepted for call compatibility)."""
    del kwargs, debug, sliding_window
    from transformers import AutoModelForCausalLM

    device = device or torch.device("cpu")
    hf_model = AutoModelForCausalLM.from_pretrained(str(hf_path)).to(device).eval()
    model = model.to(device).eval()
    if dtype is not None:
        model = model.to(dtype)
        hf_model = hf_model.to(dtype)
    ids = torch.randint(0, vocab_size, (2, 32), device=device)
    ours = model(ids)[..., :vocab_size].float()
    theirs = hf_model(input_ids=ids).logits[..., :vocab_size].float()
    torch.testing.assert_close(theirs, ours, rtol=rtol, atol=atol)
    log.info("Hugging Face export reproduces the logits of the original model")
