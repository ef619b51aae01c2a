"""
Train a normalized transformer, nGPT (the role of src/examples/ngpt/train.py)::

    torchrun --nproc-per-node=8 examples/ngpt/train.py --save-folder /tmp/ngpt-run --synthetic

All hidden states and weight rows live on the unit sphere: the model re-normalises its matrices after every optimizer
step, so there is no weight decay, no gradient clipping and no learning-rate warm-up.
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from common import TokenizerConfig, TransformerConfig, experiment, run  # noqa: E402

from olmo_core.optim import AdamConfig, ConstantWithWarmup  # noqa: E402


def build_config(opts, overrides):
    tokenizer = TokenizerConfig.gpt2()
    model = getattr(TransformerConfig, opts.model_factory)(vocab_size=tokenizer.padded_vocab_size())
    return experiment(opts, overrides, model=model, optim=AdamConfig(lr=1e-3), tokenizer=tokenizer, max_grad_norm=None,
                      scheduler=ConstantWithWarmup(warmup_steps=0))


if __name__ == "__main__":
    run(build_config, default_model="ngpt_271M")
