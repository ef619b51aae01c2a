"""
Average the weights of several Hugging Face checkpoints (the role of src/scripts/merge_hf_checkpoints.py)::

    python -m olmo_core_b200.scripts.merge_hf_checkpoints --output ./merged ckpt_a ckpt_b ckpt_c [--weights 0.5 0.25 0.25]
    python -m olmo_core_b200.scripts.merge_hf_checkpoints --output ./merged --model allenai/OLMo-2-0425-1B \
        --revisions stage1-step1000000-tokens2098B stage1-step1010000-tokens2119B

The running (weighted) mean is kept in fp32, one source model in memory at a time, and written back in the dtype of
the first checkpoint together with its config and tokenizer files. Integer buffers are taken from the first model.
"""

from __future__ import annotations

import argparse
import gc
import logging
from typing import Dict, List, Optional

import torch

log = logging.getLogger(__name__)


def merge(sources: List[dict], output: str, weights: Optional[List[float]] = None) -> None:
    from transformers import AutoModelForCausalLM, AutoTokenizer

    if len(sources) < 2:
        raise ValueError("need at least two checkpoints to merge")
    weights = weights or [1.0 / len(sources)] * len(sources)
    if len(weights) != len(sources) or abs(sum(weights) - 1.0) > 1e-6:
        raise ValueError("one weight per checkpoint, summing to 1")
    mean: Dict[str, torch.Tensor] = {}
    first = None
    for i, (src, w) in enumerate(zip(sources, weights)):
        log.info(f"[{i + 1}/{len(sources)}] {src} (weight {w:g})")
        model = AutoModelForCausalLM.from_pretrained(**src, torch_dtype="auto")
        sd = model.state_dict()
        if first is None:
            first = model
            keys = set(sd)
        elif set(sd) != keys:
            raise ValueError(f"{src} has different parameter names than the first checkpoint: "
                             f"{sorted(set(sd) ^ keys)[:5]} ...")
        for k, v in sd.items():
            if not v.is_floating_point():
                mean.setdefault(k, v.clone())
                continue
            if k in mean and mean[k].shape != v.shape:
                raise ValueError(f"'{k}' has shape {tuple(v.shape)} in {src}, {tuple(mean[k].shape)} before")
            contrib = v.to(torch.float32) * w
            mean[k] = contrib if k not in mean else mean[k].add_(contrib)
        if model is not first:
            del model, sd
            gc.collect()
    assert first is not None
    target = first.state_dict()
    first.load_state_dict({k: v.to(target[k].dtype) for k, v in mean.items()})
    first.save_pretrained(output)
    try:
        AutoTokenizer.from_pretrained(**sources[0]).save_pretrained(output)
    except Exception as e:  # a checkpoint without tokenizer files is still a valid merge
        log.warning(f"no tokenizer copied: {e}")
    log.info(f"wrote the average of {len(sources)} checkpoints to '{output}'")


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("checkpoints", nargs="*", help="local directories or hub ids")
    ap.add_argument("--model", default=None, help="one hub id whose --revisions are merged")
    ap.add_argument("--revisions", nargs="*", default=None)
    ap.add_argument("--weights", nargs="*", type=float, default=None)
    ap.add_argument("--output", required=True)
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    if a.model is not None:
        if not a.revisions:
            raise SystemExit("--model needs --revisions")
        sources = [dict(pretrained_model_name_or_path=a.model, revision=r) for r in a.revisions]
    else:
        sources = [dict(pretrained_model_name_or_path=p) for p in a.checkpoints]
    merge(sources, a.output, a.weights)


if __name__ == "__main__":
    main()
