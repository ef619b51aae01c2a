"""
Named training recipes (the per-model scripts of src/scripts/train/ and src/scripts/official/, as one table).

A recipe fixes the model factory, sequence length, global batch, per-GPU micro-batch, optimizer settings, duration and
the parallelism layout; everything else follows :func:`olmo_core_b200.internal.experiment.build_config`. Micro-batches
are quoted for 80 GB GPUs and doubled on a B200 (180 GB), except where a recipe pins them.
"""

from __future__ import annotations

from dataclasses import dataclass
from functools import partial
from typing import Any, Callable, Dict, Optional

import torch

from ...config import DType
from ...distributed.parallel import DataParallelType
from ...float8 import AOFloat8LinearConfig, Float8Config
from ...internal.experiment import CliContext, CommonComponents, ExperimentConfig, build_config
from ...nn.transformer import TransformerConfig
from ...optim import CosWithWarmup, LinearWithWarmup, OptimGroupOverride, SkipStepAdamWConfig
from ...optim.scheduler import WSD, SchedulerUnits
from ...train import Duration, TrainerConfig
from ...train.callbacks import CheckpointerCallback, CometCallback, WandBCallback
from ...train.train_module import (
    TransformerActivationCheckpointingConfig,
    TransformerActivationCheckpointingMode,
    TransformerContextParallelConfig,
    TransformerDataParallelConfig,
    TransformerDataParallelWrappingStrategy,
    TransformerExpertParallelConfig,
    TransformerTrainModuleConfig,
)

__all__ = ["Recipe", "RECIPES", "config_builder_for"]


@dataclass(frozen=True)
class Recipe:
    model: str  # name of a TransformerConfig factory
    sequence_length: int = 4096
    global_batch_sequences: int = 1024
    microbatch_sequences: int = 2  # per GPU, on an 80 GB device
    lr: float = 3e-4
    warmup_steps: int = 2000
    max_tokens: int = int(4e12)
    dp: DataParallelType = DataParallelType.hsdp
    shard_degree: Optional[int] = None
    cp_degree: Optional[int] = None
    ep_degree: Optional[int] = None
    float8: bool = False
    full_activation_checkpointing: bool = False
    project: str = "OLMo-core"
    model_kwargs: Optional[Dict[str, Any]] = None
    hybrid: bool = False  # three Gated-DeltaNet layers for every attention layer (the OLMo-hybrid layout)
    schedule: str = "cosine"  # "cosine" | "decay" (no warm-up, linear to zero over the run) | "linear" (warm-up, then to zero)
    warmup_fraction: Optional[float] = None  # "linear" only: instead of `warmup_steps`
    cp_style: str = "llama3"  # "llama3" | "zig_zag" | "ulysses"
    ac_budget: Optional[float] = None  # activation-memory budget instead of checkpointing every block
    ac_modules: Optional[tuple] = None  # checkpoint only the modules that match these patterns
    chinchilla_multiple: Optional[float] = None  # duration as a multiple of 20 tokens per parameter, instead of `max_tokens`
    epochs: Optional[int] = None  # duration in epochs (fine-tuning), instead of `max_tokens`
    weight_decay: float = 0.1
    z_loss: Optional[float] = 1e-5
    packed_documents: bool = False  # fine-tuning data: whole documents packed per instance, loss on the labelled tokens only
    no_rope_in_attention: bool = False  # hybrid long-context: the attention layers rely on the recurrent layers for order


RECIPES: Dict[str, Recipe] = {
    "OLMo2-1B": Recipe("olmo2_1B_v2", global_batch_sequences=512, microbatch_sequences=8, lr=4e-4, project="OLMo-core-1B"),
    "OLMo2-7B": Recipe("olmo2_7B", project="OLMo-core-7B"),
    "OLMo2-13B": Recipe("olmo2_13B", global_batch_sequences=2048, microbatch_sequences=1, project="OLMo-core-13B"),
    "OLMo2-32B": Recipe("olmo2_32B", global_batch_sequences=2048, microbatch_sequences=2, lr=6e-4, max_tokens=int(6.5e12),
                        shard_degree=64, full_activation_checkpointing=True, project="OLMo-core-32B"),
    "OLMo3-7B": Recipe("olmo3_7B", sequence_length=8192, global_batch_sequences=512, microbatch_sequences=1,
                       project="OLMo3-7B"),
    "OLMo3-7B-long-context": Recipe("olmo3_7B", sequence_length=65536, global_batch_sequences=64, microbatch_sequences=1,
                                    lr=2e-4, warmup_steps=200, max_tokens=int(50e9), shard_degree=1, cp_degree=8,
                                    float8=True, project="OLMo3-7B-long-context"),
    # -- the published OLMo-3 / OLMo-hybrid runs (src/scripts/official/): batch sizes in sequences of the recipe's length
    "OLMo3-7B-midtrain": Recipe("olmo3_7B", sequence_length=8192, global_batch_sequences=256, microbatch_sequences=1,
                                lr=0.00020712352850360292, warmup_steps=0, max_tokens=int(100e9), project="OLMo3-7B-midtrain"),
    "OLMo3-32B": Recipe("olmo3_32B", sequence_length=8192, global_batch_sequences=1024, microbatch_sequences=1, lr=6e-4,
                        max_tokens=int(5.5e12), shard_degree=64, full_activation_checkpointing=True, project="OLMo3-32B"),
    "OLMo3-32B-midtrain": Recipe("olmo3_32B", sequence_length=8192, global_batch_sequences=512, microbatch_sequences=1,
                                 lr=0.0002071235285, warmup_steps=0, max_tokens=int(100e9), shard_degree=64,
                                 full_activation_checkpointing=True, project="OLMo3-32B-midtrain"),
    "OLMo3-32B-long-context": Recipe("olmo3_32B", sequence_length=65536, global_batch_sequences=128, microbatch_sequences=1,
                                     lr=0.0002071235285, warmup_steps=200, max_tokens=int(100e9), shard_degree=8, cp_degree=8,
                                     full_activation_checkpointing=True, float8=True, project="OLMo3-32B-long-context"),
    "OLMo-hybrid-7B": Recipe("olmo3_7B", sequence_length=8192, global_batch_sequences=512, microbatch_sequences=1,
                             hybrid=True, project="OLMo-hybrid-7B"),
    "OLMo-hybrid-7B-midtrain": Recipe("olmo3_7B", sequence_length=8192, global_batch_sequences=512, microbatch_sequences=1,
                                      lr=0.00020712352850360292, warmup_steps=0, max_tokens=int(100e9), hybrid=True,
                                      project="OLMo-hybrid-7B-midtrain"),
    # -- further stages of the same models (src/scripts/train/{OLMo2,OLMo3,OLMo_hybrid,sft}/) ---------------------------
    "OLMo2-7B-long-context": Recipe("olmo2_7B", sequence_length=65536, global_batch_sequences=64, microbatch_sequences=1,
                                    lr=1e-5, warmup_steps=2000, cp_degree=8, project="OLMo2-7B-long-context"),
    "OLMo2-7B-anneal": Recipe("olmo2_7B", global_batch_sequences=1024, microbatch_sequences=2, lr=6.135113558011711e-05,
                              warmup_steps=0, max_tokens=int(100e9), shard_degree=32, schedule="decay",
                              project="OLMo2-7B-anneal"),
    "OLMo3-190M": Recipe("olmo3_190M", sequence_length=8192, global_batch_sequences=64, microbatch_sequences=2, lr=3e-4,
                         chinchilla_multiple=1.0, dp=DataParallelType.fsdp, project="OLMo3-190M"),
    "OLMo3-7B-anneal": Recipe("olmo3_7B", sequence_length=8192, global_batch_sequences=512, microbatch_sequences=2,
                              lr=0.00020712352850360292, warmup_steps=0, max_tokens=int(100e9), shard_degree=32,
                              schedule="decay", ac_budget=0.85, project="OLMo3-7B-anneal"),
    "OLMo-hybrid-7B-long-context": Recipe("olmo3_7B", sequence_length=65536, global_batch_sequences=64,
                                          microbatch_sequences=1, lr=0.00020712352850360292, warmup_steps=200,
                                          max_tokens=int(100e9), hybrid=True, schedule="linear", cp_degree=2,
                                          cp_style="ulysses", ac_budget=0.5, no_rope_in_attention=True,
                                          project="OLMo-hybrid-7B-long-context"),
    "OLMo2-7B-SFT": Recipe("olmo2_7B", sequence_length=16384, global_batch_sequences=64, microbatch_sequences=1, lr=8e-5,
                           schedule="linear", warmup_fraction=0.03, epochs=3, weight_decay=0.0, z_loss=None,
                           shard_degree=8, ac_modules=("blocks.*.feed_forward",), packed_documents=True,
                           project="OLMo2-7B-sft"),
    "OLMo3-7B-SFT": Recipe("olmo3_7B", sequence_length=16384, global_batch_sequences=64, microbatch_sequences=1, lr=8e-5,
                           schedule="linear", warmup_fraction=0.03, epochs=3, weight_decay=0.0, z_loss=None,
                           shard_degree=8, ac_modules=("blocks.*.feed_forward",), packed_documents=True,
                           project="OLMo3-7B-sft"),
    "OLMo3-32B-SFT": Recipe("olmo3_32B", sequence_length=16384, global_batch_sequences=64, microbatch_sequences=1, lr=8e-5,
                            schedule="linear", warmup_fraction=0.03, epochs=3, weight_decay=0.0, z_loss=None,
                            shard_degree=4, cp_degree=2, ac_modules=("blocks.*.feed_forward",), packed_documents=True,
                            project="OLMo3-32B-sft"),
    "OLMo-hybrid-7B-SFT": Recipe("olmo3_7B", sequence_length=16384, global_batch_sequences=64, microbatch_sequences=1,
                                 lr=8e-5, schedule="linear", warmup_fraction=0.03, epochs=3, weight_decay=0.0, z_loss=None,
                                 shard_degree=8, ac_modules=("blocks.*.feed_forward",), packed_documents=True, hybrid=True,
                                 project="OLMo-hybrid-7B-sft"),
    "Llama3-8B": Recipe("llama3_8B", sequence_length=8192, global_batch_sequences=512, microbatch_sequences=1,
                        project="Llama3-8B"),
    "OLMoE-1B-7B": Recipe("olmoe_1B_7B", global_batch_sequences=1024, microbatch_sequences=2, lr=4e-4, max_tokens=int(5e12),
                          dp=DataParallelType.fsdp, project="OLMoE-1B-7B"),
    "OLMoE2-medium": Recipe("llama_like_moe", global_batch_sequences=1024, microbatch_sequences=2, lr=3e-4,
                            shard_degree=32, project="OLMoE2-medium",
                            model_kwargs=dict(d_model=3328, n_layers=16, n_heads=16, num_experts=64, top_k=8,
                                              expert_hidden_size=1664, shared_expert_hidden_size=6656, capacity_factor=1.2,
                                              lb_loss_weight=0.01, z_loss_weight=0.001, reordered_norm=True, qk_norm=True,
                                              rope_theta=500_000, layer_norm_eps=1e-6)),
    "OLMoE2-large": Recipe("llama_like_moe", global_batch_sequences=2048, microbatch_sequences=2, lr=3e-4, ep_degree=-1,
                           float8=True, project="OLMoE2-large",
                           model_kwargs=dict(d_model=4096, n_layers=32, n_heads=32, num_experts=64, top_k=2,
                                             expert_hidden_size=2048, shared_expert_hidden_size=8192, capacity_factor=1.05,
                                             lb_loss_weight=0.01, z_loss_weight=0.001, reordered_norm=True, qk_norm=True,
                                             rope_theta=500_000, layer_norm_eps=1e-6)),
    "small-moe": Recipe("smallmoe", global_batch_sequences=256, microbatch_sequences=4, lr=4e-4, max_tokens=int(1e11),
                        dp=DataParallelType.fsdp, ep_degree=None, project="small-moe"),
    "nGPT-1B": Recipe("ngpt_1B", global_batch_sequences=512, microbatch_sequences=4, lr=1e-3, warmup_steps=0,
                      project="nGPT-1B"),
}


def _on_b200() -> bool:
    return torch.cuda.is_available() and "B200" in torch.cuda.get_device_name(0)


def _model(recipe: Recipe, common: CommonComponents) -> TransformerConfig:
    factory: Callable[..., TransformerConfig] = getattr(TransformerConfig, recipe.model)
    config = factory(vocab_size=common.tokenizer.padded_vocab_size(), **(recipe.model_kwargs or {}))
    if recipe.hybrid:
        config = _hybridize(config)
        if recipe.no_rope_in_attention:
            attn = config.block["attn"]
            mixer = attn.sequence_mixer if getattr(attn, "sequence_mixer", None) is not None else attn.attention
            mixer.rope = None
    return config


def _hybridize(config: TransformerConfig, remove_heads: int = 2) -> TransformerConfig:
    """
    The OLMo-hybrid layout (src/scripts/official/OLMo-hybrid/OLMo-hybrid-7B-pretrain.py:60-85): two attention heads fewer
    (and ``d_model`` narrower by as many heads of 128), then every group of four layers is three Gated-DeltaNet layers
    (head size 0.75 x 128, two value channels per key channel) followed by one attention layer.
    """
    import copy

    from ...nn.attention import GatedDeltaNetConfig

    attn_block = config.block
    mixer = attn_block.sequence_mixer if getattr(attn_block, "sequence_mixer", None) is not None else attn_block.attention
    config.d_model -= remove_heads * 128
    mixer.n_heads -= remove_heads
    if getattr(mixer, "n_kv_heads", None) is not None and mixer.n_kv_heads > mixer.n_heads:
        mixer.n_kv_heads = mixer.n_heads
    gdn_block = copy.deepcopy(attn_block)
    gdn = GatedDeltaNetConfig(n_heads=mixer.n_heads, head_dim=int(0.75 * 128), expand_v=2.0, allow_neg_eigval=True)
    if getattr(gdn_block, "sequence_mixer", None) is not None:
        gdn_block.sequence_mixer = gdn
    else:
        gdn_block.attention = gdn
    config.block = {"gdn": gdn_block, "attn": attn_block}
    config.block_pattern = ["gdn", "gdn", "gdn", "attn"]
    if config.n_layers % 4 != 0:
        raise ValueError(f"the hybrid pattern needs a multiple of 4 layers, got {config.n_layers}")
    return config


def _scheduler(recipe: Recipe):
    if recipe.schedule == "cosine":
        return CosWithWarmup(warmup_steps=recipe.warmup_steps)
    if recipe.schedule == "decay":  # an anneal: straight down to zero over the tokens of the run
        return WSD(units=SchedulerUnits.tokens, warmup=0, decay=recipe.max_tokens, decay_fraction=None)
    if recipe.schedule == "linear":
        if recipe.warmup_fraction is not None:
            return LinearWithWarmup(warmup_fraction=recipe.warmup_fraction, alpha_f=0.0)
        return LinearWithWarmup(units=SchedulerUnits.steps, warmup=recipe.warmup_steps, alpha_f=0.0)
    raise ValueError(f"unknown schedule '{recipe.schedule}'")


def _context_parallel(recipe: Recipe) -> Optional[TransformerContextParallelConfig]:
    if not recipe.cp_degree:
        return None
    if recipe.cp_style == "ulysses":
        return TransformerContextParallelConfig.ulysses(degree=recipe.cp_degree)
    if recipe.cp_style == "zig_zag":
        return TransformerContextParallelConfig.zig_zag(degree=recipe.cp_degree)
    return TransformerContextParallelConfig.llama3(degree=recipe.cp_degree, head_stride=4)


def _activation_checkpointing(recipe: Recipe) -> Optional[TransformerActivationCheckpointingConfig]:
    if recipe.full_activation_checkpointing:
        return TransformerActivationCheckpointingConfig(mode=TransformerActivationCheckpointingMode.full)
    if recipe.ac_budget is not None:
        return TransformerActivationCheckpointingConfig(mode=TransformerActivationCheckpointingMode.budget,
                                                        activation_memory_budget=recipe.ac_budget)
    if recipe.ac_modules:
        return TransformerActivationCheckpointingConfig(mode=TransformerActivationCheckpointingMode.selected_modules,
                                                        modules=list(recipe.ac_modules))
    return None


def _train_module(recipe: Recipe, common: CommonComponents) -> TransformerTrainModuleConfig:
    micro = recipe.microbatch_sequences * (2 if _on_b200() and recipe.sequence_length <= 8192 else 1)
    return TransformerTrainModuleConfig(
        rank_microbatch_size=micro * common.max_sequence_length, max_sequence_length=common.max_sequence_length,
        optim=SkipStepAdamWConfig(lr=recipe.lr, weight_decay=recipe.weight_decay, betas=(0.9, 0.95),
                                  group_overrides=[OptimGroupOverride(params=["embeddings.weight"],
                                                                      opts=dict(weight_decay=0.0))]),
        compile_model=True,
        dp_config=TransformerDataParallelConfig(name=recipe.dp, param_dtype=DType.bfloat16, reduce_dtype=DType.float32,
                                                shard_degree=recipe.shard_degree,
                                                wrapping_strategy=TransformerDataParallelWrappingStrategy.blocks),
        cp_config=_context_parallel(recipe),
        ep_config=TransformerExpertParallelConfig(degree=recipe.ep_degree) if recipe.ep_degree else None,
        ac_config=_activation_checkpointing(recipe),
        float8_config=Float8Config(enabled=recipe.float8, ao=AOFloat8LinearConfig.recommended()),
        z_loss_multiplier=recipe.z_loss, max_grad_norm=1.0, scheduler=_scheduler(recipe))


def _duration(recipe: Recipe, common: CommonComponents) -> Duration:
    if recipe.epochs is not None:
        return Duration.epochs(recipe.epochs)
    if recipe.chinchilla_multiple is not None:
        params = _model(recipe, common).num_active_non_embedding_params
        return Duration.chinchilla_tokens(recipe.chinchilla_multiple, model_params=params)
    return Duration.tokens(recipe.max_tokens)


def _trainer(recipe: Recipe, common: CommonComponents) -> TrainerConfig:
    config = (
        TrainerConfig(save_folder=common.save_folder, save_overwrite=True, metrics_collect_interval=10,
                      cancel_check_interval=10, max_duration=_duration(recipe, common))
        .with_callback("checkpointer", CheckpointerCallback(save_interval=10_000, ephemeral_save_interval=250,
                                                            save_async=True))
        .with_callback("comet", CometCallback(name=common.run_name, workspace="ai2", project=recipe.project, enabled=False,
                                              cancel_check_interval=10))
        .with_callback("wandb", WandBCallback(name=common.run_name, entity="ai2-llm", project=recipe.project,
                                              enabled=False, cancel_check_interval=10))
    )
    cluster = common.launch.clusters[0] if common.launch is not None else "local"
    try:
        config = config.with_recommended_evals(common.tokenizer, common.max_sequence_length, cluster)
    except Exception:  # evaluation data not reachable from here: train without in-loop evals
        pass
    return config


SFT_DATASET_ENV_VAR = "OLMO_SFT_DATASET"


def _sft_data(common: CommonComponents, **kwargs):
    """
    Fine-tuning data (src/scripts/train/sft/Olmo-3-7B-SFT.py:198-223): a directory of ``token_ids_part_*.npy`` with
    ``labels_mask_*.npy`` beside them, whole conversations packed per instance (longer ones truncated), attention kept
    inside each conversation, the loss on the labelled tokens only. The directory comes from ``$OLMO_SFT_DATASET`` or the
    override ``--dataset.paths=[...]``.
    """
    import os

    from ...data import NumpyDataLoaderConfig, NumpyPackedFSLDatasetConfig
    from ...data.types import LongDocStrategy
    from ...internal.experiment import DataComponents

    del kwargs
    root = os.environ.get(SFT_DATASET_ENV_VAR, f"{common.root_dir}/sft-dataset").rstrip("/")
    dataset = NumpyPackedFSLDatasetConfig(
        tokenizer=common.tokenizer, work_dir=common.work_dir, paths=[f"{root}/token_ids_part_*.npy"], expand_glob=True,
        label_mask_paths=[f"{root}/labels_mask_*.npy"], generate_doc_lengths=True,
        long_doc_strategy=LongDocStrategy.truncate, sequence_length=common.max_sequence_length)
    loader = NumpyDataLoaderConfig(global_batch_size=common.global_batch_size, seed=34521, num_workers=4)
    return DataComponents(dataset=dataset, data_loader=loader)


def config_builder_for(name: str) -> Callable[[CliContext], ExperimentConfig]:
    if name not in RECIPES:
        raise KeyError(f"unknown recipe '{name}'; available: {sorted(RECIPES)}")
    recipe = RECIPES[name]
    extra: Dict[str, Any] = dict(data_config_builder=_sft_data) if recipe.packed_documents else {}
    return partial(
        build_config, global_batch_size=recipe.global_batch_sequences * recipe.sequence_length,
        max_sequence_length=recipe.sequence_length, model_config_builder=partial(_model, recipe),
        train_module_config_builder=partial(_train_module, recipe), trainer_config_builder=partial(_trainer, recipe),
        include_default_evals=False, include_instance_filter=False, **extra)
