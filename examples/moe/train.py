"""
Train a dropless mixture-of-experts language model (the role of src/examples/moe/train.py)::

    torchrun --nproc-per-node=8 examples/moe/train.py --save-folder /tmp/moe-run --synthetic [--expert-parallel 8]

Every MoE layer routes each token to its top-k experts (softmax router, load-balancing and router z-losses added to
the objective), sorts the routed copies by expert on the device and runs ONE grouped GEMM per projection. With
``--expert-parallel N`` the experts are spread over N ranks and tokens travel to their expert's GPU through
peer-mapped memory.
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from common import TokenizerConfig, TransformerConfig, experiment, run  # noqa: E402

from olmo_core.optim import AdamWConfig, OptimGroupOverride  # noqa: E402
from olmo_core.train.train_module import TransformerExpertParallelConfig  # noqa: E402


def build_config(opts, overrides):
    tokenizer = TokenizerConfig.gpt2()
    model = getattr(TransformerConfig, opts.model_factory)(vocab_size=tokenizer.padded_vocab_size())
    extra = {}
    if opts.expert_parallel > 1:
        extra["ep_config"] = TransformerExpertParallelConfig(degree=opts.expert_parallel)
    optim = AdamWConfig(lr=4e-4, weight_decay=0.1, betas=(0.9, 0.95),
                        group_overrides=[OptimGroupOverride(params=["embeddings.weight"], opts=dict(weight_decay=0.0))])
    return experiment(opts, overrides, model=model, optim=optim, tokenizer=tokenizer, micro_batch_sequences=4,
                      warmup_steps=200, **extra)


if __name__ == "__main__":
    from common import get_cli_parser, main

    parser = get_cli_parser()
    parser.add_argument("--model-factory", default="smallmoe", help="a MoE factory of TransformerConfig (smallmoe, olmoe_1B_7B)")
    parser.add_argument("--synthetic", action="store_true", help="train on random tokens written to the work dir")
    parser.add_argument("--expert-parallel", type=int, default=1, help="number of ranks the experts are spread over")
    main(build_config, parser)
