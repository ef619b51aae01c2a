"""Saving to / loading from Hugging Face model folders (role of src/olmo_core/nn/hf/checkpoint.py)."""

from __future__ import annotations

import logging
import tempfile
from pathlib import Path
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ...aliases import PathOrStr
from ...distributed.utils import barrier, get_full_tensor, get_rank
from ...io import copy_dir, is_url
from .config import get_hf_config
from .convert import convert_state_from_hf, convert_state_to_hf

log = logging.getLogger(__name__)

__all__ = ["save_hf_model", "load_hf_model"]


def save_hf_model(save_dir: PathOrStr, model_state_dict: Dict[str, Any], model, huggingface_tokenizer=None, *,
                  dtype: Optional[torch.dtype] = None, vocab_size: Optional[int] = None,
                  process_group: Optional[dist.ProcessGroup] = None, work_dir: Optional[PathOrStr] = None,
                  save_overwrite: bool = False) -> None:
    """
    Write ``model`` (weights from ``model_state_dict``, possibly sharded) as a Hugging Face ``save_pretrained`` folder.
    All ranks must call it (sharded tensors are gathered); rank 0 writes. With a ``huggingface_tokenizer`` the generation
    config gets its end-of-text ids (``<|im_end|>``, ``<|endoftext|>``) and pad id from it, as the reference does
    (src/olmo_core/nn/hf/checkpoint.py:184-188).
    """
    from transformers import AutoModelForCausalLM

    hf_config = get_hf_config(model)
    full = {k: get_full_tensor(v).detach().cpu() for k, v in model_state_dict.items()}
    if get_rank(process_group) == 0:
        hf_state = convert_state_to_hf(hf_config, full)
        if dtype is not None:
            hf_state = {k: v.to(dtype) for k, v in hf_state.items()}
        if vocab_size is not None and vocab_size < hf_config.vocab_size:  # drop the padding rows of the vocabulary
            for key in ("model.embed_tokens.weight", "lm_head.weight"):
                if key in hf_state:
                    hf_state[key] = hf_state[key][:vocab_size]
            hf_config.vocab_size = vocab_size
        with torch.device("meta"):
            hf_model = AutoModelForCausalLM.from_config(hf_config)
        if any(k.endswith("experts.gate_up_proj") for k in hf_model.state_dict()):
            from .convert import fuse_expert_weights  # this transformers version holds the experts of a layer stacked

            hf_state = fuse_expert_weights(hf_state, hf_config.num_hidden_layers, int(getattr(hf_config, "num_experts", 0) or 0))
        hf_model.load_state_dict(hf_state, assign=True)
        if getattr(hf_model, "generation_config", None) is not None:
            hf_model.generation_config.do_sample = True
            if huggingface_tokenizer is not None:
                hf_model.generation_config.eos_token_id = huggingface_tokenizer.convert_tokens_to_ids(
                    ["<|im_end|>", "<|endoftext|>"])
                hf_model.generation_config.pad_token = huggingface_tokenizer.pad_token_id
        target = Path(tempfile.mkdtemp(dir=work_dir)) if is_url(save_dir) else Path(save_dir)
        if target.exists() and any(target.iterdir()) and not save_overwrite:
            raise FileExistsError(f"'{target}' is not empty, use save_overwrite=True to overwrite it")
        target.mkdir(parents=True, exist_ok=True)
        hf_model.save_pretrained(target)
        if is_url(save_dir):
            copy_dir(target, save_dir, save_overwrite=save_overwrite)
        log.info(f"Saved Hugging Face model to '{save_dir}'")
    barrier(process_group)


def load_hf_model(model_name_or_path: PathOrStr, model_state_dict: Dict[str, Any], *, revision: str = "main",
                  model_id: Optional[str] = None, num_embeddings: Optional[int] = None,
                  process_group: Optional[dist.ProcessGroup] = None, work_dir: Optional[PathOrStr] = None) -> None:
    """
    Fill ``model_state_dict`` (this framework's parameter names -> tensors, possibly local shards) in place with the
    weights of a Hugging Face causal LM. ``num_embeddings``: size of the (padded) vocabulary of the target model.
    """
    del model_id, process_group, work_dir
    from transformers import AutoModelForCausalLM

    from ...distributed.utils import distribute_like

    hf_model = AutoModelForCausalLM.from_pretrained(str(model_name_or_path), revision=revision, torch_dtype="auto")
    converted = convert_state_from_hf(hf_model.config, hf_model.state_dict())
    for name, target in model_state_dict.items():
        if name not in converted:
            raise KeyError(f"'{name}' has no counterpart in the Hugging Face model at {model_name_or_path}")
        src = converted[name]
        if num_embeddings is not None and name in ("embeddings.weight", "lm_head.w_out.weight") and src.shape[0] < num_embeddings:
            pad = torch.zeros(num_embeddings - src.shape[0], src.shape[1], dtype=src.dtype)
            src = torch.cat([src, pad], dim=0)
        src = distribute_like(target, src.to(dtype=target.dtype))
        with torch.no_grad():
            from ...distributed.utils import get_local_tensor

            get_local_tensor(target).copy_(get_local_tensor(src))


def __getattr__(name: str):
    # defined in ``hybrid.py``; reachable under this module's name as well
    if name in ('save_hf_hybrid_model',):
        from . import hybrid

        return getattr(hybrid, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
