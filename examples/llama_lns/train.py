"""
Train a Llama-style model with LayerNorm scaling (the role of src/examples/llama_lns/train.py)::

    torchrun --nproc-per-node=4 examples/llama_lns/train.py --save-folder /tmp/lns-run --synthetic

LayerNorm scaling multiplies the output of the pre-norms of layer ``l`` by ``1 / sqrt(l)``, which keeps the variance of
the residual stream from growing with depth; it is one block type of the model config, nothing else changes.
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from common import TokenizerConfig, TransformerConfig, experiment, run  # noqa: E402

from olmo_core.nn.transformer import TransformerBlockType  # noqa: E402
from olmo_core.optim import AdamWConfig, OptimGroupOverride  # noqa: E402


def build_config(opts, overrides):
    tokenizer = TokenizerConfig.gpt2()
    model = getattr(TransformerConfig, opts.model_factory)(vocab_size=tokenizer.padded_vocab_size())
    model.block.name = TransformerBlockType.default_scaled
    optim = AdamWConfig(lr=1e-3, group_overrides=[OptimGroupOverride(params=["embeddings.weight"], opts=dict(weight_decay=0.0))])
    return experiment(opts, overrides, model=model, optim=optim, tokenizer=tokenizer)


if __name__ == "__main__":
    run(build_config, default_model="llama2_271M")
