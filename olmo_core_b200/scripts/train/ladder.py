"""
The OLMo-3 model ladder (the role of src/scripts/train/ladder/olmo3_ladder.py)::

    python -m olmo_core_b200.scripts.train.ladder dry-run --size 190M --name my-ladder ...

Sizes, batch sizes, learning rates and durations come from :class:`Olmo3ModelConfigurator` and the default
chinchilla-multiple run configurator; ``--rank-mbz`` pins the per-GPU micro-batch (in sequences).
"""

import argparse

from ...internal.ladder import main
from ...model_ladder import ModelConfigurator, Olmo3ModelConfigurator

__all__ = ["configure_model"]


def configure_model(args: argparse.Namespace) -> ModelConfigurator:
    rank_mbz = getattr(args, "rank_mbz", None)
    return Olmo3ModelConfigurator(rank_microbatch_size=None if rank_mbz is None else rank_mbz * args.sequence_length)


if __name__ == "__main__":
    main(configure_model=configure_model)
