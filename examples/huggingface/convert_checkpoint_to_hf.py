"""
Write a trained checkpoint in Hugging Face format (the role of src/examples/huggingface/convert_checkpoint_to_hf.py)::

    python examples/huggingface/convert_checkpoint_to_hf.py -i /runs/my-run/step1000 -o /tmp/my-run-hf \
        [--max-sequence-length 4096] [--skip-validation] [--dtype bfloat16]

The input is a step directory of a run (it holds ``model_and_optim/`` and the ``config.json`` saved by the config-saver
callback). The weights are renamed and re-laid out for the matching ``transformers`` architecture, saved with
``save_pretrained`` together with the tokenizer settings, and -- unless skipped -- loaded back with ``transformers`` to
compare logits on random token ids.
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from olmo_core.config import DType  # noqa: E402
from olmo_core.nn.hf.convert_checkpoint import convert_checkpoint_to_hf, load_config  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("-i", "--checkpoint-input-path", required=True)
    ap.add_argument("-o", "--huggingface-output-dir", required=True)
    ap.add_argument("-s", "--max-sequence-length", type=int, default=None)
    ap.add_argument("--dtype", default=None, help="dtype of the written weights (default: as trained)")
    ap.add_argument("--skip-validation", action="store_true")
    ap.add_argument("--device", default=None)
    a = ap.parse_args()
    config = load_config(a.checkpoint_input_path)
    if config is None:
        raise SystemExit(f"no config.json found in '{a.checkpoint_input_path}': was the run started with the config-saver callback?")
    tokenizer = config.get("dataset", {}).get("tokenizer", {})
    convert_checkpoint_to_hf(
        original_checkpoint_path=a.checkpoint_input_path, output_path=a.huggingface_output_dir,
        transformer_config_dict=config["model"], tokenizer_config_dict=tokenizer,
        max_sequence_length=a.max_sequence_length, dtype=DType(a.dtype) if a.dtype else None,
        validate=not a.skip_validation, device=a.device)
    print(f"wrote {a.huggingface_output_dir}")


if __name__ == "__main__":
    main()
