"""Tensor + sequence parallelism on two gloo ranks must reproduce the single-process losses (CPU)."""

import json
from pathlib import Path

import pytest
import torch

from olmo_core_b200.testing import run_distributed_test

VOCAB, SEQ = 256, 32


def _losses(tp: bool, steps: int = 3, mx: bool = False):
    from olmo_core_b200.float8 import AOMXLinearConfig, Float8Config
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.optim import AdamWConfig
    from olmo_core_b200.train.train_module import (
        TransformerDataParallelConfig,
        TransformerTensorParallelConfig,
        TransformerTrainModule,
    )

    torch.manual_seed(0)
    model = TransformerConfig.olmo2_30M(vocab_size=VOCAB, n_layers=2).build(init_device="cpu")
    torch.manual_seed(0)
    model.init_weights(max_seq_len=SEQ, device=torch.device("cpu"))
    # both layouts start from these weights: the train module must not re-initialise (sliced) parameters
    model.init_weights = lambda *a, **k: None
    tm = TransformerTrainModule(
        model=model, optim=AdamWConfig(lr=1e-3, weight_decay=0.0), rank_microbatch_size=4 * SEQ, max_sequence_length=SEQ,
        max_grad_norm=1.0, device=torch.device("cpu"),
        tp_config=TransformerTensorParallelConfig(degree=2) if tp else None,
        dp_config=TransformerDataParallelConfig(name="ddp") if tp else None,
        float8_config=Float8Config(ao_mx=AOMXLinearConfig.mxfp8_cublas_rceil()) if mx else None,
    )
    if mx:
        assert any(getattr(m, "float8", None) is not None for m in tm.model.modules())
    gen = torch.Generator().manual_seed(7)
    out = []
    for _ in range(steps):
        ids = torch.randint(0, VOCAB, (4, SEQ), generator=gen)
        tm.zero_grads()
        tm.train_batch({"input_ids": ids})
        tm.optim_step()
        out.append(float(tm.latest_ce_loss))
    return out


def _tp_worker(path: str, mx: bool = False):
    import torch.distributed as dist

    losses = _losses(tp=True, mx=mx)
    if dist.get_rank() == 0:
        Path(path).write_text(json.dumps(losses))


def test_tensor_parallel_matches_single_process(tmp_path):
    want = _losses(tp=False)
    out = tmp_path / "tp.json"
    run_distributed_test(_tp_worker, world_size=2, func_args=(str(out),))
    got = json.loads(out.read_text())
    assert got == pytest.approx(want, rel=2e-4), (got, want)


def test_tensor_parallel_with_mx_quantised_projections(tmp_path):
    """Block-scaled 8-bit projections under tensor parallelism: the sliced weights quantise in the same 32-element blocks
    as the whole ones, so the losses follow the single-process run up to the order of the partial sums."""
    want = _losses(tp=False, mx=True)
    plain = _losses(tp=False)
    assert want != plain  # the quantised layers are really in use
    out = tmp_path / "tp_mx.json"
    run_distributed_test(_tp_worker, world_size=2, func_args=(str(out), True))
    got = json.loads(out.read_text())
    assert got == pytest.approx(want, rel=5e-3), (got, want)
