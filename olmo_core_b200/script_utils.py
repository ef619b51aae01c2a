"""
Helpers shared by stand-alone training scripts (role of src/olmo_core/script_utils.py:28-201).

A script supplies ``config_builder(opts, overrides) -> ExperimentConfig`` and calls :func:`main`, which parses the
common command line (``--save-folder``, ``--data-root``, ``--sequence-length``, ``--dry-run``, ``--train-single`` plus
dotted ``key=value`` overrides passed through to the builder), brings up the process group, builds
model → train module → dataset → data loader → trainer, resumes from the save folder (or ``load_path``) and fits.
"""

from __future__ import annotations

import argparse
import logging
import sys
from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch

from .aliases import PathOrStr
from .config import Config
from .data import NumpyDataLoaderConfig, NumpyDatasetConfig
from .distributed.checkpoint import get_checkpoint_metadata, load_state_dict
from .io import is_url, join_path, normalize_path
from .nn.transformer import TransformerConfig
from .train import TrainerConfig, prepare_training_environment, teardown_training_environment
from .train.callbacks import ConfigSaverCallback
from .train.train_module import TransformerTrainModuleConfig
from .utils import prepare_cli_environment, seed_all

log = logging.getLogger(__name__)

__all__ = ["ExperimentConfig", "get_cli_parser", "main", "get_lr_from_checkpoint"]

_REMOTE_WORK_DIR = "/tmp/olmo-core/dataset-cache"


@dataclass
class ExperimentConfig(Config):
    model: TransformerConfig
    dataset: NumpyDatasetConfig
    data_loader: NumpyDataLoaderConfig
    train_module: TransformerTrainModuleConfig
    trainer: TrainerConfig
    init_seed: int = 12536
    load_path: Optional[str] = None


def get_cli_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog=sys.argv[0], usage=f"python {sys.argv[0]} [OPTIONS...] [CONFIG_OVERRIDES...]",
                                formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    p.add_argument("--name", type=str, help="Name of the run, used for logging.")
    p.add_argument("--sequence-length", type=int, default=None,
                   help="Sequence length to train and evaluate on; each script has its own default.")
    p.add_argument("--data-root", type=str, default="https://olmo-data.org",
                   help="Root directory or URL of the tokenized source files (the public default can be slow; "
                        "a mounted copy or 'gs://ai2-llm' / 's3://ai2-llm' is faster where available).")
    p.add_argument("--save-folder", type=str, required=True,
                   help="Local or remote directory for checkpoints; every rank must be able to reach it.")
    p.add_argument("--work-dir", type=str,
                   help="Local scratch directory for dataset preprocessing; derived from the save folder if unset.")
    p.add_argument("--dry-run", action="store_true", help="Print the config and exit.")
    p.add_argument("--train-single", action="store_true", help="Train on one rank without any parallelism (debugging).")
    return p


def _parse_args(parser: Optional[argparse.ArgumentParser] = None) -> Tuple[argparse.Namespace, List[str]]:
    opts, overrides = (parser or get_cli_parser()).parse_known_args()
    if opts.work_dir is None:
        opts.work_dir = _REMOTE_WORK_DIR if is_url(opts.save_folder) else opts.save_folder
    return opts, overrides


def main(config_builder: Callable[[argparse.Namespace, List[str]], ExperimentConfig],
         parser: Optional[argparse.ArgumentParser] = None) -> None:
    opts, overrides = _parse_args(parser)
    if opts.dry_run:
        prepare_cli_environment()
    config = config_builder(opts, overrides)
    if opts.dry_run:
        try:
            import rich

            rich.print(config)
        except ImportError:
            print(config)
        return

    if opts.train_single:
        for field in ("dp_config", "tp_config"):
            if getattr(config.train_module, field, None) is not None:
                log.warning("'%s' is set but a single-rank run cannot use it; disabling", field)
                setattr(config.train_module, field, None)

    backend = "cpu:gloo,cuda:nccl" if torch.cuda.is_available() else None
    prepare_training_environment(shared_filesystem=not is_url(opts.save_folder), backend=backend)
    seed_all(config.init_seed)

    model = config.model.build(init_device="meta")
    train_module = config.train_module.build(model)
    dataset = config.dataset.build()
    data_loader = config.data_loader.build(dataset, dp_process_group=train_module.dp_process_group)
    trainer = config.trainer.build(train_module, data_loader)

    # the full experiment config goes into every checkpoint directory (and to the experiment trackers)
    for callback in trainer.callbacks.values():
        if isinstance(callback, ConfigSaverCallback):
            callback.config = config.as_config_dict()
            break

    # resume from the save folder when it has a checkpoint, otherwise start from ``load_path`` (weights + optimizer only)
    if not trainer.no_checkpoints and not trainer.maybe_load_checkpoint() and config.load_path:
        log.info("No checkpoint in the save folder; loading from %s", config.load_path)
        trainer.load_checkpoint(config.load_path, load_trainer_state=False)

    trainer.fit()
    teardown_training_environment()


def get_lr_from_checkpoint(path: PathOrStr, param: Optional[str] = None, param_group: Optional[int] = None) -> float:
    """
    Read the learning rate stored in a checkpoint's optimizer state without loading anything else. Optimizer state is
    saved either with numbered groups (``optim.param_groups.<i>.lr``) or flattened per parameter
    (``optim.param_groups.<fqn>.lr``); ``param_group`` applies to the former and ``param`` to the latter.
    """
    path = normalize_path(path)
    if not path.endswith("/model_and_optim"):
        path = join_path(path, "model_and_optim")
    metadata = get_checkpoint_metadata(path)
    if "optim.param_groups.0.params" in metadata.state_dict_metadata:
        if param is not None:
            log.warning("'param' is ignored: the checkpoint stores optimizer state by numbered group")
        key = f"optim.param_groups.{param_group or 0}.lr"
    else:
        if param_group is not None:
            raise RuntimeError("'param_group' cannot be used: the checkpoint stores optimizer state per parameter")
        key = f"optim.param_groups.{param or 'embeddings.weight'}.lr"
    state = {key: None}
    load_state_dict(path, state)
    if state[key] is None:
        raise KeyError(f"{key} not found in {path}")
    return float(state[key])  # type: ignore[arg-type]
