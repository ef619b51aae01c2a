"""
Turn a distributed checkpoint into plain files (role of src/scripts/unshard.py)::

    python -m olmo_core_b200.scripts.unshard CHECKPOINT_DIR TARGET_DIR [--safetensors] [--optim] [--strategy one_file]
"""

import argparse

from ..distributed.checkpoint import UnshardStrategy, UnshardStrategyType, unshard_checkpoint
from ..utils import prepare_cli_environment


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("checkpoint_dir", help="a trainer checkpoint (step dir) or its model_and_optim folder; local or URL")
    p.add_argument("target_dir", help="local output directory")
    p.add_argument("--safetensors", action="store_true", help="write safetensors instead of torch pickles (model only)")
    p.add_argument("--optim", action=argparse.BooleanOptionalAction, default=None, help="also unshard the optimizer state")
    p.add_argument("--strategy", choices=[s.value for s in UnshardStrategyType], default="one_file")
    p.add_argument("--chunk-size", type=int, default=None, help="bytes per file for the 'chunks' strategy")
    p.add_argument("--overwrite", action="store_true")
    p.add_argument("--pre-download", action="store_true", help="copy a remote checkpoint to --work-dir first")
    p.add_argument("--work-dir", default=None)
    args = p.parse_args(argv)
    prepare_cli_environment()
    kind = UnshardStrategyType(args.strategy)
    if kind == UnshardStrategyType.one_file:
        strategy = UnshardStrategy.one_file()
    elif kind == UnshardStrategyType.one_file_per_tensor:
        strategy = UnshardStrategy.one_file_per_tensor()
    else:
        strategy = UnshardStrategy.chunks(args.chunk_size or 4 * 1024**3)
    source = args.checkpoint_dir.rstrip("/")
    if not source.endswith("model_and_optim"):
        source += "/model_and_optim"
    model_path, optim_path = unshard_checkpoint(source, args.target_dir, optim=args.optim, save_overwrite=args.overwrite,
                                                use_safetensors=args.safetensors, unshard_strategy=strategy,
                                                pre_download=args.pre_download, work_dir=args.work_dir)
    print(f"model: {model_path}" + (f"\noptim: {optim_path}" if optim_path is not None else ""))


if __name__ == "__main__":
    main()
