"""
Transformer models (API of src/olmo_core/nn/transformer/model.py:82-1217):
``embeddings -> [embed_scale] -> [embedding_norm] -> blocks["0".."L-1"] -> lm_head``.

Parallelism hooks differ from the reference in mechanism, not in names: ``apply_fsdp`` / ``apply_ddp`` hand
the module to the sharded-parameter runtime in ``olmo_core_b200.parallel.fsdp`` (flat fp32 master shards,
resident bf16 compute copies, fused reduce-scatter + AdamW), ``apply_tp`` shards projections by rows /
columns with sequence-parallel activations, ``apply_cp`` installs a load balancer that shards inputs,
labels and RoPE tables consistently.
"""

from __future__ import annotations

import logging
from collections import defaultdict
from functools import cached_property
from typing import Any, Dict, List, Literal, Optional, Tuple, Union

import torch
import torch.nn as nn

from ...data.utils import get_cumulative_document_lengths
from ...doc_utils import beta_feature
from ...ops.elementwise import embedding as embedding_op
from ...utils import get_default_device, move_to_device
from ..attention import (
    Attention,
    FusedAttention,
    RingContextParallelStyle,
    UlyssesContextParallelStyle,
)
from ..attention.ring import RingAttentionLoadBalancer
from ..buffer_cache import BufferCache
from ..layer_norm import LayerNormConfig
from ..lm_head import LMHeadConfig, LMOutputWithLoss
from .block import MoETransformerBlock, NormalizedTransformerBlock, TransformerBlockBase
from .config import (
    TransformerActivationCheckpointingMode,
    TransformerBlockConfig,
    TransformerDataParallelWrappingStrategy,
    resolve_block_configs,
)
from .init import InitMethod

__all__ = ["Transformer", "NormalizedTransformer", "MoETransformer", "Embedding",
           "TransformerDataParallelWrappingStrategy", "TransformerActivationCheckpointingMode"]

log = logging.getLogger(__name__)


class Embedding(nn.Module):
    """Token embedding table (parameter name ``weight``) looked up with the gather kernel."""

    def __init__(self, num_embeddings: int, embedding_dim: int, dtype: torch.dtype = torch.float32, device: str = "cpu"):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim, dtype=dtype, device=device))
        if device != "meta":
            nn.init.normal_(self.weight)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return embedding_op(input_ids, self.weight)

    def extra_repr(self) -> str:
        return f"{self.num_embeddings}, {self.embedding_dim}"


def _checkpoint_module(module: nn.Module, determinism_check: str = "default") -> None:
    """Recompute ``module``'s forward in the backward pass (while training with gradients on) instead of saving its
    intermediate activations. Idempotent. ``determinism_check``: "default" compares the metadata of recomputed tensors
    with the forward pass', "none" skips that check."""
    if getattr(module, "_checkpointed_forward", None) is not None:
        return
    inner = module.forward

    def forward(*args, **kwargs):
        if module.training and torch.is_grad_enabled():
            from torch.utils.checkpoint import checkpoint

            return checkpoint(inner, *args, use_reentrant=False, determinism_check=determinism_check, **kwargs)
        return inner(*args, **kwargs)

    module._checkpointed_forward = inner  # type: ignore[assignment]
    module.forward = forward  # type: ignore[method-assign]


class Transformer(nn.Module):
    def __init__(
        self,
        *,
        d_model: int,
        vocab_size: int,
        n_layers: int,
        block: Union[TransformerBlockConfig, Dict[str, TransformerBlockConfig]],
        lm_head: LMHeadConfig,
        embedding_norm: Optional[LayerNormConfig] = None,
        dtype: torch.dtype = torch.float32,
        init_method: InitMethod = InitMethod.normal,
        init_device: str = "cpu",
        init_seed: int = 0,
        init_std: float = 0.02,
        embedding_init_std: Optional[float] = None,
        block_overrides: Optional[Dict[int, TransformerBlockConfig]] = None,
        block_pattern: Optional[List[str]] = None,
        embed_scale: Optional[float] = None,
        tie_word_embeddings: bool = False,
    ):
        super().__init__()
        cache = BufferCache()
        self.d_model = d_model
        self.vocab_size = vocab_size
        self.n_layers = n_layers
        self.dtype = dtype
        self.embed_scale = embed_scale
        self.embeddings: Optional[Embedding] = Embedding(vocab_size, d_model, dtype=dtype, device=init_device)
        self.embedding_norm = None if embedding_norm is None else embedding_norm.build(d_model, init_device=init_device)
        self.blocks = nn.ModuleDict()
        for idx, cfg in enumerate(resolve_block_configs(n_layers, block, block_pattern, block_overrides)):
            self.blocks[str(idx)] = self._build_block(cfg, idx, init_device, cache)
        self.lm_head = lm_head.build(d_model=d_model, vocab_size=vocab_size, init_device=init_device)
        self.init_method = InitMethod(init_method)
        self.init_seed = init_seed
        self.init_std = init_std
        self.embedding_init_std = embedding_init_std
        self.tie_word_embeddings = tie_word_embeddings
        if tie_word_embeddings:
            self._tie_weights()
        self._cache = cache
        self._pp_enabled = False
        self._pp_group_size = 1
        self._fp8_enabled = False
        self._compile_enabled = False
        self._device: Optional[torch.device] = None
        self._cp_load_balancer: Optional[RingAttentionLoadBalancer] = None
        self._tp_enabled = False
        self._tp_mesh = None
        self._cp_mesh = None
        self._sharding_runtime = None  # set by olmo_core_b200.parallel.fsdp

    def _build_block(self, cfg: TransformerBlockConfig, idx: int, init_device: str, cache: BufferCache) -> TransformerBlockBase:
        return cfg.build(d_model=self.d_model, block_idx=idx, n_layers=self.n_layers, init_device=init_device, cache=cache)

    def _tie_weights(self) -> None:
        if self.lm_head is not None and self.embeddings is not None:
            self.lm_head.w_out.weight = self.embeddings.weight

    # -- flags -------------------------------------------------------------------------------------------
    @property
    def pp_enabled(self) -> bool:
        return self._pp_enabled

    @property
    def fp8_enabled(self) -> bool:
        return self._fp8_enabled

    @property
    def compile_enabled(self) -> bool:
        return self._compile_enabled

    @property
    def tp_enabled(self) -> bool:
        return self._tp_enabled

    @property
    def fsdp_enabled(self) -> bool:
        return bool(getattr(self, "_fsdp_enabled", False))

    def compute_auxiliary_metrics(self, reset: bool = True):
        """Model-internal metrics to log (none for a dense model; the MoE model reports router statistics)."""
        del reset
        return {}

    def reset_auxiliary_metrics(self) -> None:
        pass

    def get_rope_buffers(self, seq_len: int, device: Optional[torch.device] = None):
        """Per layer, the rotary tables of its attention for ``seq_len`` positions (``None`` for layers without RoPE)."""
        device = device if device is not None else self.device
        out = {}
        for key, block in self.blocks.items():
            rope = getattr(getattr(block, "attention", None), "rope", None)
            out[int(key)] = None if rope is None else rope.get_buffers(seq_len, device)
        return out

    @property
    def cp_enabled(self) -> bool:
        return self._cp_load_balancer is not None

    @property
    def ep_enabled(self) -> bool:
        return False

    @property
    def is_moe(self) -> bool:
        return False

    @property
    def device(self) -> torch.device:
        if self._device is None:
            for p in self.parameters():
                if p.device.type != "meta":
                    self._device = p.device
                    break
            else:
                self._device = get_default_device()
        return self._device

    def _apply(self, fn, *args, **kwargs):
        # ``.to()`` / ``.cuda()`` / ``.cpu()`` move the parameters: forget the cached device so that inputs follow them
        out = super()._apply(fn, *args, **kwargs)
        self._device = None
        return out

    # -- initialisation ------------------------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(
        self,
        *,
        max_seq_len: Optional[int] = None,
        max_local_microbatch_size: Optional[int] = None,
        device: Optional[torch.device] = None,
        world_mesh=None,
        model_part_idx: int = 0,
    ) -> torch.Generator:
        """
        Materialise parameters on ``device`` and draw them from one seeded generator, in module order:
        embeddings, then per block attention -> MLP / MoE, then the LM head.
        """
        device = device or self.device
        if any(p.device.type == "meta" for p in self.parameters()):
            self.to_empty(device=device)
            if self.tie_word_embeddings:
                self._tie_weights()
        elif device != self.device:
            self.to(device)
        self._device = device
        for m in self.modules():
            if m is not self and hasattr(m, "reset_parameters"):
                m.reset_parameters()
        seed = self.init_seed
        if world_mesh is not None and self.pp_enabled:
            from ...distributed.parallel import get_pp_mesh

            pp_mesh = get_pp_mesh(world_mesh)
            seed += pp_mesh.get_local_rank() + model_part_idx * pp_mesh.size()
        gen = torch.Generator(device).manual_seed(seed)
        if self.embeddings is not None:
            self.init_method.init_embeddings(
                self.embeddings, d_model=self.d_model, embed_scale=self.embed_scale,
                std=self.embedding_init_std if self.embedding_init_std is not None else self.init_std, generator=gen,
            )
        for block in self.blocks.values():
            self.init_method.init_attention(block.attention, d_model=self.d_model, block_idx=block.block_idx,
                                            num_blocks=self.n_layers, std=self.init_std, generator=gen)
            if hasattr(block, "feed_forward"):
                self.init_method.init_feed_forward(block.feed_forward, d_model=self.d_model, block_idx=block.block_idx,
                                                   num_blocks=self.n_layers, std=self.init_std, generator=gen)
            if hasattr(block, "feed_forward_moe"):
                if max_local_microbatch_size is not None:
                    block.feed_forward_moe.warmup_cache(max_local_microbatch_size)
                self.init_method.init_feed_forward_moe(block.feed_forward_moe, d_model=self.d_model,
                                                       block_idx=block.block_idx, num_blocks=self.n_layers,
                                                       std=self.init_std, generator=gen)
            att = block.attention
            if max_seq_len is not None and isinstance(att, (Attention, FusedAttention)) and att.rope is not None:
                att.rope.warmup_cache(max_seq_len, device)
        if self.lm_head is not None and not self.tie_word_embeddings:
            self.init_method.init_final_w_out(self.lm_head.w_out, d_model=self.d_model, std=self.init_std, generator=gen)
        return gen

    # -- forward ---------------------------------------------------------------------------------------------
    def _prepare_inputs(
        self,
        input_ids: torch.Tensor,
        labels: Optional[torch.Tensor] = None,
        *,
        ignore_index: int = -100,
        loss_reduction: Literal["mean", "sum", "none"] = "mean",
        z_loss_multiplier: Optional[float] = None,
        loss_div_factor: Optional[Union[torch.Tensor, float]] = None,
        return_logits: Optional[bool] = None,
        logits_to_keep: Union[int, torch.Tensor] = 0,
        **kwargs,
    ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Dict[str, Any], Dict[int, Dict[str, Any]], Dict[str, Any]]:
        B, S = input_ids.shape[:2]
        block_kwargs: Dict[str, Any] = {}
        per_block: Dict[int, Dict[str, Any]] = defaultdict(dict)
        head_kwargs: Dict[str, Any] = dict(ignore_index=ignore_index, loss_reduction=loss_reduction,
                                           z_loss_multiplier=z_loss_multiplier, return_logits=return_logits,
                                           logits_to_keep=logits_to_keep)
        if loss_div_factor is not None:
            loss_div_factor = move_to_device(loss_div_factor, self.device)
            head_kwargs["loss_div_factor"] = loss_div_factor
            block_kwargs["loss_div_factor"] = loss_div_factor

        max_doc_len: Optional[int] = None
        cu_doc_lens: Optional[torch.Tensor] = None
        cache_leftpad = kwargs.pop("cache_leftpad", None)
        doc_lens = kwargs.pop("doc_lens", None)
        max_doc_lens = kwargs.pop("max_doc_lens", None)
        if doc_lens is not None and max_doc_lens is not None:
            max_doc_len = max(max_doc_lens)
            cu_doc_lens = get_cumulative_document_lengths(doc_lens)

        if (lb := self._cp_load_balancer) is not None:
            # Shard ids, labels and every block's RoPE tables the same way, on the host.
            inputs = [input_ids] + ([labels] if labels is not None else [])
            seq_dims = [1] * len(inputs)
            pad_values: List[Union[int, float]] = [0] + ([ignore_index] if labels is not None else [])
            rope_keys: List[Tuple[int, str]] = []
            for key, block in self.blocks.items():
                att = block.attention
                rope = getattr(att, "rope", None)
                if rope is None or cu_doc_lens is not None:  # packed documents: explicit positions instead (below)
                    continue
                bufs = rope.get_buffers(S, torch.device("cpu"))
                for name in ("pos_sin", "pos_cos", "freqs_cis"):
                    t = getattr(bufs, name)
                    if t is not None:
                        inputs.append(t[:S])
                        seq_dims.append(0)
                        pad_values.append(0.0)
                        rope_keys.append((int(key), name))
            # The sequence is sharded by POSITION whatever it contains; with packed documents every rank additionally gets
            # the document boundaries of the whole sequence and the attention kernels mask by them (the reference shards
            # document by document instead, src/olmo_core/nn/transformer/model.py:426-499; the attended pairs are the same).
            if cu_doc_lens is not None:
                # rotary positions restart at every document; each rank gets the positions of ITS tokens
                cu_cpu = cu_doc_lens.cpu().long()
                flat = torch.arange(B * S, dtype=torch.long)
                doc = torch.bucketize(flat, cu_cpu[1:], right=True).clamp(max=cu_cpu.numel() - 2)
                inputs.append((flat - cu_cpu[doc]).view(B, S))
                seq_dims.append(1)
                pad_values.append(0)
            shards = lb.batch_shard(inputs=inputs, seq_dims=seq_dims, pad_values=pad_values)
            if cu_doc_lens is not None:
                block_kwargs["cu_doc_lens"] = move_to_device(cu_doc_lens, self.device)
                block_kwargs["max_doc_len"] = max_doc_len
                block_kwargs["rope_pos_ids"] = move_to_device(shards.pop(), self.device)
                block_kwargs["rope_table_len"] = S
            input_ids = shards[0]
            n = 1
            if labels is not None:
                labels = shards[1]
                n = 2
            for (bidx, name), t in zip(rope_keys, shards[n:]):
                per_block[bidx][name] = move_to_device(t, self.device)
        elif cu_doc_lens is not None:
            block_kwargs["max_doc_len"] = max_doc_len
            block_kwargs["cu_doc_lens"] = move_to_device(cu_doc_lens, self.device)

        if cache_leftpad is not None:
            block_kwargs["cache_leftpad"] = move_to_device(cache_leftpad, self.device)
        input_ids = move_to_device(input_ids, self.device)
        if labels is not None:
            labels = move_to_device(labels, self.device)
        return input_ids, labels, block_kwargs, per_block, head_kwargs

    def forward(
        self,
        input_ids: torch.Tensor,
        *,
        input_embeddings: Optional[torch.Tensor] = None,
        labels: Optional[torch.Tensor] = None,
        ignore_index: int = -100,
        loss_reduction: Literal["mean", "sum", "none"] = "mean",
        z_loss_multiplier: Optional[float] = None,
        loss_div_factor: Optional[Union[torch.Tensor, float]] = None,
        return_logits: Optional[bool] = None,
        logits_to_keep: Union[int, torch.Tensor] = 0,
        **kwargs,
    ) -> Union[torch.Tensor, LMOutputWithLoss]:
        """
        Logits ``[B, S, V]`` when ``labels`` is None, else :class:`LMOutputWithLoss`. Extra keyword arguments:
        ``doc_lens`` + ``max_doc_lens`` (intra-document masking) and ``cache_leftpad`` (KV-cache decoding).
        """
        if input_embeddings is not None and self._cp_load_balancer is not None:
            raise RuntimeError("`input_embeddings` is not supported with context parallelism")
        input_ids, labels, block_kwargs, per_block, head_kwargs = self._prepare_inputs(
            input_ids, labels, ignore_index=ignore_index, loss_reduction=loss_reduction,
            z_loss_multiplier=z_loss_multiplier, loss_div_factor=loss_div_factor, return_logits=return_logits,
            logits_to_keep=logits_to_keep, **kwargs,
        )
        if input_embeddings is not None:
            h = move_to_device(input_embeddings, self.device)
        else:
            h = self.embeddings(input_ids) if self.embeddings is not None else input_ids
            if self.embeddings is not None and self.embed_scale is not None:
                h = h * self.embed_scale
            if self.embedding_norm is not None:
                h = self.embedding_norm(h)
        if self._tp_enabled and self.embeddings is not None:
            from ...parallel.tensor import scatter_to_sequence_parallel

            h = scatter_to_sequence_parallel(h, self._tp_mesh.get_group(),
                                             partial_producer_grads=getattr(self, "_tp_embedding_partial", False))
        for key, block in self.blocks.items():
            h = self._run_block(block, h, {**block_kwargs, **per_block.get(int(key), {})})
        if self.lm_head is None:
            return h
        if self._tp_enabled:
            # the head works on this rank's sequence shard and gathers / sums only what it returns
            head_kwargs["tp_sequence_sharded"] = True
        if labels is not None:
            head_kwargs["labels"] = labels
        return self.lm_head(h, **head_kwargs)

    def _run_block(self, block: nn.Module, h: torch.Tensor, kwargs: Dict[str, Any]) -> torch.Tensor:
        if h.is_cuda:
            from ...ops import _lib

            if _lib.nvtx_enabled():
                with torch.cuda.nvtx.range(f"block.{getattr(block, 'block_idx', '?')}"):
                    return self._run_block_inner(block, h, kwargs)
        return self._run_block_inner(block, h, kwargs)

    def _run_block_inner(self, block: nn.Module, h: torch.Tensor, kwargs: Dict[str, Any]) -> torch.Tensor:
        if getattr(block, "_activation_checkpointing", False) and self.training and torch.is_grad_enabled():
            from torch.utils.checkpoint import checkpoint

            return checkpoint(
                block, h, use_reentrant=False,
                determinism_check=getattr(block, "_checkpoint_determinism_check", "default"), **kwargs
            )
        return block(h, **kwargs)

    # -- parallelism and memory --------------------------------------------------------------------------------
    def apply_pp(self, pp_mesh) -> None:
        self._pp_enabled = True
        self._pp_group_size = pp_mesh.size()

    def apply_fp8(self, float8_config) -> None:
        if float8_config is None or not float8_config.enabled:
            return
        float8_config.apply_float8_linear(self)
        self._fp8_enabled = True

    def apply_tp(self, tp_mesh, float8_enabled: Optional[bool] = None) -> None:
        from ...parallel.tensor import shard_lm_head_, shard_model_

        shard_model_(self, tp_mesh)
        self._tp_enabled = True
        self._tp_mesh = tp_mesh

    def apply_cp(self, cp_mesh, ring: Optional[RingContextParallelStyle] = None,
                 uly: Optional[UlyssesContextParallelStyle] = None) -> None:
        if (ring is None) == (uly is None):
            raise ValueError("exactly one of 'ring' or 'uly' must be given")
        lb_type = ring.load_balancer if ring is not None else uly.load_balancer
        self._cp_load_balancer = lb_type.build(cp_mesh)
        self._cp_mesh = cp_mesh
        for block in self.blocks.values():
            block.apply_cp(cp_mesh, ring=ring, uly=uly)
        if self.lm_head is not None:
            self.lm_head.apply_cp(cp_mesh)

    def apply_activation_checkpointing(
        self,
        mode: TransformerActivationCheckpointingMode,
        block_interval: Optional[int] = None,
        modules: Optional[List[str]] = None,
        activation_memory_budget: Optional[float] = None,
        determinism_check: str = "default",
    ) -> None:
        """
        Choose what is recomputed in the backward pass instead of being kept from the forward pass
        (reference: src/olmo_core/nn/transformer/model.py:726-838).

        * ``full``: every block; ``selected_blocks``: every ``block_interval``-th block; ``budget``: the fraction
          ``1 - activation_memory_budget`` of the blocks, evenly spaced.
        * ``selected_modules``: every module whose dotted name matches one of the ``modules`` globs, at any depth
          (``"blocks.*.feed_forward"``, ``"blocks.3"``, ``"*.attention"``). A match inside an already selected module
          is dropped: its parent recomputes it anyway.
        * ``selected_ops``: keep the outputs of GEMMs and attention, recompute the element-wise results between them.
          With the fused kernels the only such tensor of any size is the gated activation ``silu(a) * b`` of every MLP;
          the backward kernel of the down-projection re-derives it from ``a | b`` in its epilogue, so the forward pass
          stops saving it (one ``[tokens, hidden]`` tensor per layer).
        """
        from fnmatch import fnmatch

        mode = TransformerActivationCheckpointingMode(mode)
        blocks = list(self.blocks.items())
        chosen: List[str] = []
        if mode == TransformerActivationCheckpointingMode.full:
            chosen = [k for k, _ in blocks]
        elif mode == TransformerActivationCheckpointingMode.selected_blocks:
            if not block_interval:
                raise ValueError("'block_interval' is required for 'selected_blocks' activation checkpointing")
            chosen = [k for k, _ in blocks if int(k) % block_interval == 0]
        elif mode == TransformerActivationCheckpointingMode.selected_modules:
            if not modules:
                raise ValueError("'modules' is required for 'selected_modules' activation checkpointing")
            matched = [(name, m) for name, m in self.named_modules()
                       if name and any(fnmatch(name, pat) for pat in modules)]
            if not matched:
                raise ValueError(f"no module matches any of {modules}")
            taken: List[str] = []
            for name, module in sorted(matched, key=lambda nm: nm[0].count(".")):
                if any(name.startswith(parent + ".") for parent in taken):
                    continue
                taken.append(name)
                if name.startswith("blocks.") and name.count(".") == 1:
                    chosen.append(name.split(".")[1])
                else:
                    _checkpoint_module(module, determinism_check)
        elif mode == TransformerActivationCheckpointingMode.budget:
            if activation_memory_budget is None:
                raise ValueError("'activation_memory_budget' is required for 'budget' activation checkpointing")
            n_ckpt = round((1.0 - activation_memory_budget) * len(blocks))
            if n_ckpt > 0:
                stride = len(blocks) / n_ckpt
                chosen = [blocks[min(int(i * stride), len(blocks) - 1)][0] for i in range(n_ckpt)]
        elif mode == TransformerActivationCheckpointingMode.selected_ops:
            from ..feed_forward import FeedForward

            for module in self.modules():
                if isinstance(module, FeedForward):
                    module.recompute_activation = True
        for key in chosen:
            self.blocks[key]._activation_checkpointing = True
            self.blocks[key]._checkpoint_determinism_check = determinism_check

    def apply_compile(self) -> None:
        """Accepted for API compatibility; the GPU path uses explicit fused kernels rather than a compiler."""
        self._compile_enabled = True

    def apply_fsdp(
        self,
        dp_mesh=None,
        param_dtype: Optional[torch.dtype] = None,
        reduce_dtype: torch.dtype = torch.float32,
        pp_enabled: bool = False,
        prefetch_factor: int = 0,
        wrapping_strategy: TransformerDataParallelWrappingStrategy = TransformerDataParallelWrappingStrategy.full,
    ) -> None:
        from ...parallel.fsdp import ShardedParamRuntime

        self._sharding_runtime = ShardedParamRuntime(
            self, group=None if dp_mesh is None else _mesh_group(dp_mesh), param_dtype=param_dtype,
            reduce_dtype=reduce_dtype, shard=True,
        )

    def apply_ddp(self, dp_mesh=None, param_dtype: Optional[torch.dtype] = None, compile_enabled: bool = False,
                  autograd_compile_enabled: bool = False) -> None:
        from ...parallel.fsdp import ShardedParamRuntime

        self._sharding_runtime = ShardedParamRuntime(
            self, group=None if dp_mesh is None else _mesh_group(dp_mesh), param_dtype=param_dtype,
            reduce_dtype=torch.float32, shard=False,
        )

    # -- bookkeeping ----------------------------------------------------------------------------------------------
    @cached_property
    def num_params(self) -> int:
        return sum(_full_numel(p) for p in self.parameters())

    @property
    def num_trainable_params(self) -> int:
        return sum(_full_numel(p) for p in self.parameters() if p.requires_grad)

    @cached_property
    def num_non_embedding_params(self) -> int:
        return self.num_params - (_full_numel(self.embeddings.weight) if self.embeddings is not None else 0)

    def num_flops_per_token(self, seq_len: int) -> int:
        n = sum(b.num_flops_per_token(seq_len) for b in self.blocks.values())
        if self.lm_head is not None:
            n += self.lm_head.num_flops_per_token(seq_len)
        return n

    def post_batch(self, dry_run: bool = False) -> None:
        """Called after the last backward of a batch, before the optimizer step."""

    def post_optim_step(self) -> None:
        """Called after each optimizer step."""
        if self._fp8_enabled:
            from ...float8 import refresh_float8_scales

            refresh_float8_scales(self)

    def init_kv_cache(self, batch_size: int, max_seq_len: int, dtype: torch.dtype = torch.bfloat16) -> None:
        for block in self.blocks.values():
            att = block.attention
            if hasattr(att, "init_kv_cache_manager"):
                att.init_kv_cache_manager(batch_size, max_seq_len, dtype)

    def reset_kv_cache(self) -> None:
        for block in self.blocks.values():
            att = block.attention
            if hasattr(att, "reset_kv_cache_manager"):
                att.reset_kv_cache_manager()


def _mesh_group(mesh):
    if hasattr(mesh, "ndim") and mesh.ndim == 2:
        return mesh  # hybrid sharding: the runtime takes the 2-D mesh
    return mesh.get_group()


def _full_numel(p: torch.Tensor) -> int:
    info = getattr(p, "_shard_info", None)
    if info is not None:
        n = 1
        for s in info.full_shape:
            n *= s
        return n
    return p.numel()


@beta_feature
class NormalizedTransformer(Transformer):
    """nGPT: all matrices are re-normalised to unit norm after every optimizer step."""

    def __init__(self, **kwargs):
        kwargs.setdefault("init_method", InitMethod.normalized)
        super().__init__(**kwargs)

    @torch.no_grad()
    def init_weights(self, **kwargs) -> torch.Generator:
        gen = super().init_weights(**kwargs)
        self.normalize_matrices()
        return gen

    @torch.no_grad()
    def normalize_matrices(self) -> None:
        from ..layer_norm import l2_normalize

        if self.embeddings is not None:
            self.embeddings.weight.copy_(l2_normalize(self.embeddings.weight, dim=-1))
        for block in self.blocks.values():
            if hasattr(block, "normalize_matrices"):
                block.normalize_matrices()
        if self.lm_head is not None and hasattr(self.lm_head, "normalize_matrices"):
            self.lm_head.normalize_matrices()

    def post_optim_step(self) -> None:
        super().post_optim_step()
        self.normalize_matrices()

    def apply_tp(self, *args, **kwargs) -> None:
        raise NotImplementedError("TP is not implemented yet for the normalized transformer variant")


@beta_feature
class MoETransformer(Transformer):
    """Transformer whose blocks contain mixture-of-experts layers."""

    @property
    def is_moe(self) -> bool:
        return True

    @property
    def ep_enabled(self) -> bool:
        return any(getattr(b, "ep_enabled", False) for b in self.blocks.values())

    def compute_auxiliary_metrics(self, reset: bool = True) -> Dict[str, Tuple[torch.Tensor, Optional[object]]]:
        """
        Router statistics per block (``block NN/<name>``) and over all blocks under the bare name: sums for metrics that
        are summed or averaged over ranks, the maximum for max-reduced ones
        (src/olmo_core/nn/transformer/model.py:1114-1152). With pipeline parallelism a mean-reduced value is scaled by
        the pipeline group size, because only one rank in that many holds the block.
        """
        from ...train.common import ReduceType

        offset = float(getattr(self, "_pp_group_size", 1)) if self.pp_enabled else 1.0
        out: Dict[str, Tuple[torch.Tensor, Optional[object]]] = {}
        for key, block in self.blocks.items():
            if not isinstance(block, MoETransformerBlock):
                continue
            for name, (val, reduce_type) in block.compute_metrics(reset=reset).items():
                out[f"block {int(key):02d}/{name}"] = (val, reduce_type)
                if self.pp_enabled and reduce_type == ReduceType.mean:
                    val = val.float() * offset
                if name not in out:
                    out[name] = (val, reduce_type)
                elif reduce_type in (ReduceType.mean, ReduceType.sum):
                    out[name] = (out[name][0] + val, reduce_type)
                elif reduce_type == ReduceType.max:
                    out[name] = (torch.max(out[name][0], val), reduce_type)
                else:
                    raise NotImplementedError(reduce_type)
        return out

    def reset_auxiliary_metrics(self) -> None:
        for block in self.blocks.values():
            if isinstance(block, MoETransformerBlock):
                block.reset_metrics()

    def apply_ep(self, ep_mesh, **kwargs) -> None:
        for block in self.blocks.values():
            if isinstance(block, MoETransformerBlock):
                block.apply_ep(ep_mesh, **kwargs)

    def prepare_experts_for_fsdp(self, **kwargs) -> None:
        for block in self.blocks.values():
            if isinstance(block, MoETransformerBlock):
                block.feed_forward_moe.prepare_experts_for_fsdp(**kwargs)

    def prepare_experts_for_ddp(self, **kwargs) -> None:
        for block in self.blocks.values():
            if isinstance(block, MoETransformerBlock):
                block.feed_forward_moe.prepare_experts_for_ddp(**kwargs)

    def post_batch(self, dry_run: bool = False) -> None:
        for block in self.blocks.values():
            if isinstance(block, MoETransformerBlock):
                block.post_batch(dry_run=dry_run)
