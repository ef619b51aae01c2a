"""
Turn a Hugging Face checkpoint into this framework's checkpoint format
(the role of src/examples/huggingface/convert_checkpoint_from_hf.py)::

    python examples/huggingface/convert_checkpoint_from_hf.py -i allenai/OLMo-2-0425-1B -o /tmp/olmo2-1b \
        --model-factory olmo2_1B_v2 [--revision main]

The model is built from the named ``TransformerConfig`` factory, the ``transformers`` weights are renamed / re-laid
out into it, and the result is saved as a sharded checkpoint (``model_and_optim/``) plus a ``config.json`` that a
trainer can resume from with ``load_path``.
"""

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402

from olmo_core.data import TokenizerConfig  # noqa: E402
from olmo_core.distributed.checkpoint import save_model_and_optim_state  # noqa: E402
from olmo_core.nn.hf.checkpoint import load_hf_model  # noqa: E402
from olmo_core.nn.transformer import TransformerConfig  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("-i", "--checkpoint-input-path", required=True, help="hub id or local directory")
    ap.add_argument("-o", "--output-dir", required=True)
    ap.add_argument("--model-factory", required=True, help="name of a TransformerConfig factory")
    ap.add_argument("--tokenizer", default="dolma2", help="name of a TokenizerConfig factory")
    ap.add_argument("--revision", default="main")
    a = ap.parse_args()
    tokenizer = getattr(TokenizerConfig, a.tokenizer)()
    config = getattr(TransformerConfig, a.model_factory)(vocab_size=tokenizer.padded_vocab_size())
    model = config.build(init_device="cpu")
    state = model.state_dict()
    load_hf_model(a.checkpoint_input_path, state, revision=a.revision, work_dir=os.path.join(a.output_dir, "hf-download"),
                  num_embeddings=config.vocab_size)
    model.load_state_dict(state)
    save_model_and_optim_state(os.path.join(a.output_dir, "model_and_optim"), model, save_overwrite=True)
    with open(os.path.join(a.output_dir, "config.json"), "w") as f:
        json.dump({"model": config.as_config_dict(), "dataset": {"tokenizer": tokenizer.as_config_dict()}}, f, indent=2)
    n = sum(p.numel() for p in model.parameters())
    print(f"wrote {a.output_dir} ({n / 1e9:.2f} B parameters, dtype {next(model.parameters()).dtype})")
    del torch


if __name__ == "__main__":
    main()
