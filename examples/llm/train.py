"""
Minimal end-to-end language-model training script (the role of src/examples/llm/train.py)::

    torchrun --nproc-per-node=8 examples/llm/train.py --save-folder /tmp/run1 [--sequence-length 2048] \
        [--model-factory olmo2_190M] [trainer.max_duration.value=1000 ...]
    python examples/llm/train.py --save-folder /tmp/run1 --dry-run

Data: tokenized ``.npy`` files under ``--data-root`` (the default mix is public but slow to stream); for a quick check
without any data pass ``--synthetic`` and random token ids are written to the work dir first.
"""

import argparse
from typing import List

import numpy as np

from olmo_core.config import DType
from olmo_core.data import NumpyDataLoaderConfig, NumpyFSLDatasetConfig, TokenizerConfig
from olmo_core.distributed.parallel import DataParallelType
from olmo_core.nn.transformer import TransformerConfig
from olmo_core.optim import AdamWConfig, CosWithWarmup, OptimGroupOverride
from olmo_core.script_utils import ExperimentConfig, get_cli_parser, main
from olmo_core.train import Duration, TrainerConfig
from olmo_core.train.callbacks import CheckpointerCallback, ConfigSaverCallback, GPUMemoryMonitorCallback
from olmo_core.train.train_module import TransformerDataParallelConfig, TransformerTrainModuleConfig

DEFAULT_SEQUENCE_LENGTH = 2048


def build_config(opts: argparse.Namespace, overrides: List[str]) -> ExperimentConfig:
    sequence_length = opts.sequence_length or DEFAULT_SEQUENCE_LENGTH
    tokenizer = TokenizerConfig.gpt2()
    model = getattr(TransformerConfig, opts.model_factory)(vocab_size=tokenizer.padded_vocab_size())
    if opts.synthetic:
        import os

        os.makedirs(opts.work_dir, exist_ok=True)
        path = os.path.join(opts.work_dir, "synthetic-tokens.npy")
        if not os.path.exists(path):
            np.random.default_rng(0).integers(0, tokenizer.vocab_size, 64 * 1024 * 1024 // 2, dtype=np.uint16).tofile(path)
        paths = [path]
    else:
        paths = [f"{opts.data_root}/examples/c4-en/gpt2/c4-train.00000-00099.npy"]
    dataset = NumpyFSLDatasetConfig(paths=paths, sequence_length=sequence_length, tokenizer=tokenizer,
                                    work_dir=opts.work_dir, max_target_sequence_length=max(8192, sequence_length))
    data_loader = NumpyDataLoaderConfig(global_batch_size=256 * sequence_length, seed=0, num_workers=4)
    train_module = TransformerTrainModuleConfig(
        rank_microbatch_size=16 * sequence_length, max_sequence_length=sequence_length,
        optim=AdamWConfig(lr=1e-3, group_overrides=[OptimGroupOverride(params=["embeddings.weight"],
                                                                     opts=dict(weight_decay=0.0))]),
        compile_model=True,
        dp_config=TransformerDataParallelConfig(name=DataParallelType.fsdp, param_dtype=DType.bfloat16,
                                                reduce_dtype=DType.float32),
        max_grad_norm=1.0, scheduler=CosWithWarmup(warmup_steps=100))
    trainer = (
        TrainerConfig(save_folder=opts.save_folder, save_overwrite=True, metrics_collect_interval=5,
                      cancel_check_interval=5, max_duration=Duration.steps(1000))
        .with_callback("gpu_monitor", GPUMemoryMonitorCallback())
        .with_callback("checkpointer", CheckpointerCallback(save_interval=1000, ephemeral_save_interval=100,
                                                            save_async=True))
        .with_callback("config_saver", ConfigSaverCallback())
    )
    config = ExperimentConfig(model=model, dataset=dataset, data_loader=data_loader, train_module=train_module,
                              trainer=trainer)
    return config.merge(overrides)


if __name__ == "__main__":
    parser = get_cli_parser()
    parser.add_argument("--model-factory", default="olmo2_190M", help="name of a TransformerConfig factory")
    parser.add_argument("--synthetic", action="store_true", help="train on random tokens written to the work dir")
    main(build_config, parser)
