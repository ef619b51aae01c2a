"""
Autoregressive generation with a transformer: batched prefill, KV-cached decode, sampling, stop tokens
(behaviour of src/olmo_core/generate/generation_module/transformer/generation_module.py:46-604).

Prompts of different lengths are LEFT-padded; the per-sequence pad counts are recorded in the KV cache so that padded
positions are never attended to. With ``use_cache`` each decode step feeds one token per sequence and attends over the
cache; without it the whole sequence is re-run every step (useful as an oracle).
"""

from __future__ import annotations

import json
import logging
import tempfile
import time
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ....aliases import PathOrStr
from ....config import DType
from ....data.utils import attention_mask_to_cache_leftpad
from ....distributed.checkpoint import get_checkpoint_metadata, load_model_state, load_state_dict, model_state
from ....distributed.utils import broadcast_object, get_fs_local_rank, get_rank, get_world_size
from ....exceptions import OLMoConfigurationError
from ....io import is_url, join_path, normalize_path, read_text
from ....nn.transformer import Transformer, TransformerConfig
from ....utils import get_default_device, log_or_print, move_to_device
from ...sampling import select_next_token
from ...utils import selective_log_softmax
from ..config import GenerationConfig
from ..generation_module import GenerationModule

log = logging.getLogger(__name__)

__all__ = ["TransformerGenerationModule"]


class TransformerGenerationModule(GenerationModule):
    def __init__(self, model: Transformer, generation_config: GenerationConfig, compile_model: bool = False,
                 float8_config=None, dp_config=None, device: Optional[torch.device] = None,
                 state_dict_load_opts: Optional[Dict[str, Any]] = None, state_dict_save_opts: Optional[Dict[str, Any]] = None,
                 load_key_mapping: Optional[Dict[str, str]] = None):
        del compile_model, float8_config, dp_config  # generation runs every rank on its own replica
        self.device = device or get_default_device()
        self.model = model
        if any(p.device.type == "meta" for p in model.parameters()):
            self.model.to_empty(device=self.device)
        else:
            self.model.to(self.device)
        self.model.eval()
        self._generation_config = generation_config
        self.state_dict_load_opts = state_dict_load_opts or {}
        self.state_dict_save_opts = state_dict_save_opts or {}
        self.load_key_mapping = load_key_mapping
        self._cache_shape: Optional[Tuple[int, int]] = None

    @property
    def dp_process_group(self) -> Optional[dist.ProcessGroup]:
        return None

    @property
    def world_size(self) -> int:
        return get_world_size()

    def state_dict(self) -> Dict[str, Any]:
        return {"model": model_state(self.model)}

    def state_dict_to_load(self, metadata) -> Dict[str, Any]:
        sd = self.state_dict()
        if self.load_key_mapping is not None:
            from ....distributed.checkpoint import swap_param_keys

            swap_param_keys(sd, self.load_key_mapping, metadata=metadata)
        return sd

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        if self.load_key_mapping is not None:
            from ....distributed.checkpoint import swap_param_keys

            swap_param_keys(state_dict, self.load_key_mapping, reverse=True, quiet=True)
        load_model_state(self.model, state_dict["model"], strict=self.state_dict_load_opts.get("strict", True))

    # -- cache -------------------------------------------------------------------------------------------
    def prepare_inference_cache(self, batch_size: int, max_seq_len: int) -> None:
        dtype = next(self.model.parameters()).dtype
        dtype = dtype if dtype in (torch.bfloat16, torch.float16) else torch.float32
        self.model.init_kv_cache(batch_size, max_seq_len, dtype)
        self._cache_shape = (batch_size, max_seq_len)

    def free_inference_cache(self) -> None:
        self.model.reset_kv_cache()
        self._cache_shape = None

    def model_forward(self, input_ids: torch.Tensor, **kwargs) -> torch.Tensor:
        return self.model(input_ids, **kwargs)

    # -- generation ----------------------------------------------------------------------------------------
    @torch.inference_mode()
    def generate_batch(self, input_ids: torch.Tensor, *, attention_mask: Optional[torch.Tensor] = None,
                       return_logits: bool = False, return_logprobs: bool = False, completions_only: bool = False,
                       log_timing: bool = True, **generation_kwargs
                       ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
        """
        ``attention_mask`` marks real tokens of LEFT-padded prompts. Keyword arguments override fields of the
        generation config for this call. Returns ``(ids [B, L], logits [B, new, V] | None, logprobs [B, new] | None)``.
        """
        start = time.perf_counter()
        cfg = self._generation_config.replace(**generation_kwargs)
        eos, pad = cfg.eos_token_id, cfg.pad_token_id
        input_ids = move_to_device(input_ids, self.device)
        B, prompt_len = input_ids.shape
        if cfg.max_new_tokens is not None:
            max_length: Optional[int] = prompt_len + cfg.max_new_tokens
        else:
            max_length = cfg.max_length
        stop = (torch.tensor(cfg.stop_token_ids, device=self.device, dtype=torch.long)
                if cfg.stop_token_ids is not None else None)
        leftpad = None
        if cfg.use_cache:
            if max_length is None:
                raise OLMoConfigurationError("max_length or max_new_tokens must be provided if use_cache is True")
            if attention_mask is None:
                attention_mask = torch.ones_like(input_ids, dtype=torch.bool)
            leftpad = attention_mask_to_cache_leftpad(move_to_device(attention_mask, self.device)).to(self.device)
            self.prepare_inference_cache(B, max_length)
        else:
            self.free_inference_cache()

        finished = torch.zeros(B, dtype=torch.bool, device=self.device)
        generated = input_ids
        logits_out: List[torch.Tensor] = []
        logprobs_out: List[torch.Tensor] = []
        first_token_time = None
        n_new = 0
        try:
            while not ((max_length is not None and generated.shape[1] >= max_length) or bool(finished.all())):
                first = generated.shape[1] == prompt_len
                step_input = generated if (first or not cfg.use_cache) else generated[:, -1:]
                kwargs: Dict[str, Any] = {"logits_to_keep": 1}
                if cfg.use_cache and first:
                    kwargs["cache_leftpad"] = leftpad
                logits = self.model_forward(step_input, **kwargs)[:, -1]  # [B, V]
                next_tokens = select_next_token(logits, do_sample=cfg.do_sample, temperature=cfg.temperature,
                                                top_k=cfg.top_k, top_p=cfg.top_p)
                if return_logits:
                    logits_out.append(logits.unsqueeze(1))
                if return_logprobs:
                    logprobs_out.append(selective_log_softmax(logits, next_tokens).unsqueeze(1))
                next_tokens = torch.where(finished, torch.full_like(next_tokens, pad), next_tokens)
                hit = next_tokens.eq(eos)
                if stop is not None:
                    hit |= next_tokens.unsqueeze(-1).eq(stop).any(dim=-1)
                finished |= hit
                generated = torch.cat([generated, next_tokens.unsqueeze(-1)], dim=1)
                if n_new == 0:
                    first_token_time = time.perf_counter() - start
                n_new += 1
        finally:
            if cfg.use_cache:
                self.free_inference_cache()
        if log_timing and n_new:
            total = time.perf_counter() - start
            log_or_print(log, f"generated {n_new} tokens x {B} sequences in {total:.3f}s "
                              f"(time to first token {first_token_time:.3f}s, {n_new * B / total:.1f} tokens/s)")
        logits_t = torch.cat(logits_out, dim=1) if logits_out else None
        logprobs_t = torch.cat(logprobs_out, dim=1) if logprobs_out else None
        return (generated[:, prompt_len:] if completions_only else generated), logits_t, logprobs_t

    # -- checkpoints ----------------------------------------------------------------------------------------
    def load_checkpoint(self, checkpoint_dir: PathOrStr, work_dir: PathOrStr, process_group=None, pre_download: bool = True,
                        load_thread_count: Optional[int] = None) -> None:
        """Load model weights from a trainer checkpoint (``<dir>/model_and_optim``) or a bare model checkpoint."""
        work_dir = Path(work_dir)
        if get_fs_local_rank() == 0:
            work_dir.mkdir(parents=True, exist_ok=True)
        checkpoint_dir = normalize_path(checkpoint_dir)
        module_dir = join_path(checkpoint_dir, "model_and_optim")
        metadata = None
        if get_rank(process_group) == 0:
            try:
                metadata = get_checkpoint_metadata(module_dir)
            except FileNotFoundError:
                metadata = get_checkpoint_metadata(checkpoint_dir)
                module_dir = checkpoint_dir
        module_dir = broadcast_object(module_dir)
        if metadata is None:
            metadata = get_checkpoint_metadata(module_dir)
        sd = self.state_dict_to_load(metadata)
        load_state_dict(module_dir, sd, process_group=process_group, pre_download=is_url(checkpoint_dir) and pre_download,
                        work_dir=work_dir, thread_count=load_thread_count)
        self.load_state_dict(sd)

    @classmethod
    def from_checkpoint(cls, checkpoint_dir: PathOrStr, *, transformer_config: Optional[TransformerConfig] = None,
                        generation_config: Optional[GenerationConfig] = None, process_group=None,
                        work_dir: Optional[PathOrStr] = None, pre_download: bool = True,
                        load_thread_count: Optional[int] = None, dtype: Optional[DType] = None,
                        attention_backend=None, **kwargs) -> "TransformerGenerationModule":
        """Build the model from the ``config.json`` beside the checkpoint (unless a config is given) and load it."""
        checkpoint_dir = normalize_path(checkpoint_dir)
        tokenizer_config = None
        if transformer_config is None and get_rank(process_group) == 0:
            from ....data import TokenizerConfig

            config_path = join_path(checkpoint_dir, "config.json")
            cfg = json.loads(read_text(config_path))
            try:
                transformer_config = TransformerConfig.from_dict(cfg["model"])
                tokenizer_config = TokenizerConfig.from_dict(cfg["dataset"]["tokenizer"])
            except KeyError as e:
                raise OLMoConfigurationError(f"Failed to load config from checkpoint at {config_path}: missing field {e}") from e
        work_dir = Path(work_dir or (tempfile.mkdtemp() if get_rank(process_group) == 0 else tempfile.gettempdir()))
        transformer_config, work_dir, tokenizer_config = broadcast_object((transformer_config, work_dir, tokenizer_config))
        if transformer_config is None:
            raise OLMoConfigurationError("A transformer config is required: pass one or use a checkpoint with config.json")
        if generation_config is None:
            if tokenizer_config is None:
                raise OLMoConfigurationError("A tokenizer config is required to derive a generation config")
            generation_config = GenerationConfig(pad_token_id=tokenizer_config.pad_token_id,
                                                 eos_token_id=tokenizer_config.eos_token_id)
        if attention_backend is not None:
            def set_backend(c):
                if hasattr(c, "backend"):
                    c.backend = attention_backend

            transformer_config.apply(set_backend)
        model = transformer_config.build(init_device="meta")
        if dtype is not None:
            model = model.to(dtype=DType(dtype).as_pt())
        module = cls(model, generation_config, **kwargs)
        module.load_checkpoint(checkpoint_dir, work_dir=work_dir, process_group=process_group, pre_download=pre_download,
                               load_thread_count=load_thread_count)
        return module

    @classmethod
    def from_checkpoints(cls, checkpoint_dirs: List[PathOrStr], **kwargs) -> "TransformerGenerationModule":
        """From several checkpoints of the same architecture: weights are averaged (a "model soup")."""
        module = cls.from_checkpoint(checkpoint_dirs[0], **kwargs)
        if len(checkpoint_dirs) == 1:
            return module
        total = {n: p.detach().float().clone() for n, p in module.model.named_parameters()}
        work_dir = Path(kwargs.get("work_dir") or tempfile.mkdtemp())
        for path in checkpoint_dirs[1:]:
            module.load_checkpoint(path, work_dir=work_dir, process_group=kwargs.get("process_group"))
            for n, p in module.model.named_parameters():
                total[n] += p.detach().float()
        with torch.no_grad():
            for n, p in module.model.named_parameters():
                p.copy_((total[n] / len(checkpoint_dirs)).to(p.dtype))
        return module
