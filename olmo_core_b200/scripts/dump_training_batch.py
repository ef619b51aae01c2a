"""
Write the token ids of chosen training batches as text and as a tensor file (role of src/scripts/dump_training_batch.py)::

    python -m olmo_core_b200.scripts.dump_training_batch CONFIG_JSON STEP [STEP ...] --out DIR [--tokenizer IDENT]

``CONFIG_JSON`` is the ``config.json`` a run saved beside its checkpoints (or any JSON with ``dataset`` and ``data_loader``
sections). Batches are addressed by step, so nothing before them is read.
"""

import argparse
import json
from pathlib import Path

import torch

from ..data import NumpyDataLoaderConfig, NumpyDatasetConfig
from ..io import read_text
from ..utils import prepare_cli_environment


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("config")
    p.add_argument("steps", type=int, nargs="+", help="1-based training steps")
    p.add_argument("--out", required=True)
    p.add_argument("--epoch", type=int, default=1)
    p.add_argument("--tokenizer", default=None, help="Hugging Face tokenizer used to decode the ids")
    args = p.parse_args(argv)
    prepare_cli_environment()
    cfg = json.loads(read_text(args.config))
    dataset = NumpyDatasetConfig.from_dict(cfg["dataset"]).build()
    loader = NumpyDataLoaderConfig.from_dict(cfg["data_loader"]).build(dataset)
    loader.reshuffle(args.epoch)
    tok = None
    if args.tokenizer:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(args.tokenizer)
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    for step in args.steps:
        batch = loader[step - 1]
        torch.save(batch, out / f"batch_step{step}.pt")
        with open(out / f"batch_step{step}.txt", "w") as f:
            for i, ids in enumerate(batch["input_ids"].tolist()):
                f.write(f"=== instance {i} (index {int(batch['index'][i]) if 'index' in batch else '?'}) ===\n")
                f.write((tok.decode(ids) if tok is not None else " ".join(map(str, ids))) + "\n")
        print(f"step {step}: {tuple(batch['input_ids'].shape)} -> {out}/batch_step{step}.*")


if __name__ == "__main__":
    main()
