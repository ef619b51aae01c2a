"""
What the example training scripts share: the command line, a tokenized dataset (real ``.npy`` files or random tokens
written on the spot) and an ``ExperimentConfig`` built around a model config that each example supplies.
"""

import argparse
import os
import sys
from typing import Callable, List, Optional

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source checkout

from olmo_core.config import DType  # noqa: E402
from olmo_core.data import NumpyDataLoaderConfig, NumpyFSLDatasetConfig, TokenizerConfig  # noqa: E402
from olmo_core.distributed.parallel import DataParallelType  # noqa: E402
from olmo_core.nn.transformer import TransformerConfig  # noqa: E402
from olmo_core.optim import CosWithWarmup, OptimConfig  # noqa: E402
from olmo_core.script_utils import ExperimentConfig, get_cli_parser, main  # noqa: E402
from olmo_core.train import Duration, TrainerConfig  # noqa: E402
from olmo_core.train.callbacks import CheckpointerCallback, ConfigSaverCallback, GPUMemoryMonitorCallback  # noqa: E402
from olmo_core.train.train_module import TransformerDataParallelConfig, TransformerTrainModuleConfig  # noqa: E402


def token_files(opts: argparse.Namespace, tokenizer: TokenizerConfig) -> List[str]:
    """The example corpus under ``--data-root``, or (``--synthetic``) 32 Mi random token ids in the work dir."""
    if not opts.synthetic:
        return [f"{opts.data_root}/examples/c4-en/gpt2/c4-train.00000-00099.npy"]
    os.makedirs(opts.work_dir, exist_ok=True)
    path = os.path.join(opts.work_dir, "synthetic-tokens.npy")
    if not os.path.exists(path):
        np.random.default_rng(0).integers(0, tokenizer.vocab_size, 32 * 1024 * 1024, dtype=np.uint16).tofile(path)
    return [path]


def experiment(opts: argparse.Namespace, overrides: List[str], *, model: TransformerConfig, optim: OptimConfig,
               tokenizer: Optional[TokenizerConfig] = None, sequence_length: int = 2048, global_batch_sequences: int = 256,
               micro_batch_sequences: int = 8, steps: int = 1000, warmup_steps: int = 100,
               max_grad_norm: Optional[float] = 1.0, **train_module_kwargs) -> ExperimentConfig:
    tokenizer = tokenizer or TokenizerConfig.gpt2()
    sequence_length = opts.sequence_length or sequence_length
    dataset = NumpyFSLDatasetConfig(paths=token_files(opts, tokenizer), sequence_length=sequence_length, tokenizer=tokenizer,
                                    work_dir=opts.work_dir, max_target_sequence_length=max(8192, sequence_length))
    data_loader = NumpyDataLoaderConfig(global_batch_size=global_batch_sequences * sequence_length, seed=0, num_workers=4)
    train_module_kwargs.setdefault("dp_config", TransformerDataParallelConfig(
        name=DataParallelType.fsdp, param_dtype=DType.bfloat16, reduce_dtype=DType.float32))
    train_module_kwargs.setdefault("scheduler", CosWithWarmup(warmup_steps=warmup_steps))
    train_module = TransformerTrainModuleConfig(rank_microbatch_size=micro_batch_sequences * sequence_length,
                                                max_sequence_length=sequence_length, optim=optim,
                                                max_grad_norm=max_grad_norm, **train_module_kwargs)
    trainer = (
        TrainerConfig(save_folder=opts.save_folder, save_overwrite=True, metrics_collect_interval=5, cancel_check_interval=5,
                      max_duration=Duration.steps(steps))
        .with_callback("gpu_monitor", GPUMemoryMonitorCallback())
        .with_callback("checkpointer", CheckpointerCallback(save_interval=steps, ephemeral_save_interval=100, save_async=True))
        .with_callback("config_saver", ConfigSaverCallback())
    )
    return ExperimentConfig(model=model, dataset=dataset, data_loader=data_loader, train_module=train_module,
                            trainer=trainer).merge(overrides)


def run(build: Callable[[argparse.Namespace, List[str]], ExperimentConfig], *, default_model: str) -> None:
    parser = get_cli_parser()
    parser.add_argument("--model-factory", default=default_model, help="name of a TransformerConfig factory")
    parser.add_argument("--synthetic", action="store_true", help="train on random tokens written to the work dir")
    main(build, parser)
