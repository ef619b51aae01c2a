"""
Pipeline parallelism on two gloo ranks (CPU): a 4-layer model cut into two stages trains through the 1F1B schedule with
the same losses as the whole model in one process, every rank learns the loss, gradient clipping uses the norm over
all stages, and the train module's state dict (parameter-name keys, optimizer state included) round-trips.
"""

import json
from pathlib import Path

import pytest
import torch
import torch.distributed as dist

from olmo_core_b200.nn.transformer import TransformerConfig
from olmo_core_b200.optim import AdamWConfig
from olmo_core_b200.testing import run_distributed_test

VOCAB, SEQ, LAYERS = 256, 16, 4


def _batches(n):
    g = torch.Generator().manual_seed(11)
    return [torch.randint(0, VOCAB, (4, SEQ), generator=g) for _ in range(n)]


def _single_process_reference(steps, init_path):
    from olmo_core_b200.train.train_module import TransformerTrainModule

    torch.manual_seed(0)
    model = TransformerConfig.olmo2_30M(vocab_size=VOCAB, n_layers=LAYERS).build(init_device="cpu")
    tm = TransformerTrainModule(model=model, optim=AdamWConfig(lr=1e-2), rank_microbatch_size=2 * SEQ,
                                max_sequence_length=SEQ, max_grad_norm=1.0, device=torch.device("cpu"))
    # the pipeline stages seed their own initialisation, so both runs start from this state dict
    torch.save({n: p.detach().clone() for n, p in model.named_parameters()}, init_path)
    losses = []
    for ids in _batches(steps):
        tm.zero_grads()
        tm.train_batch({"input_ids": ids})
        tm.optim_step()
        losses.append(float(tm.latest_ce_loss))
    return losses, {n: p.detach().clone() for n, p in model.named_parameters()}


def _pp_worker(tmp: str, steps: int):
    from olmo_core_b200.train.train_module.transformer.config import (
        TransformerDataParallelConfig,
        TransformerPipelineParallelConfig,
    )
    from olmo_core_b200.train.train_module.transformer.pipeline_train_module import TransformerPipelineTrainModule

    rank = dist.get_rank()
    torch.manual_seed(0)
    model = TransformerConfig.olmo2_30M(vocab_size=VOCAB, n_layers=LAYERS).build(init_device="meta")
    pp = TransformerPipelineParallelConfig(degree=2, schedule="1F1B")

    def build():
        return TransformerPipelineTrainModule(model=model, optim=AdamWConfig(lr=1e-2), rank_microbatch_size=2 * SEQ,
                                              max_sequence_length=SEQ, pp_config=pp, max_grad_norm=1.0,
                                              dp_config=TransformerDataParallelConfig(name="fsdp"),
                                              device=torch.device("cpu"))

    tm = build()
    tm.load_state_dict({"model": torch.load(Path(tmp) / "init.pt", weights_only=False)})  # whole-model dict, own stages taken
    owned = sorted(n for part in tm.model_parts for n, _ in part.named_parameters())
    assert any(n.startswith("embeddings") for n in owned) == (rank == 0)
    assert any(n.startswith("lm_head") for n in owned) == (rank == 1)
    assert any(n.startswith("blocks.0.") for n in owned) == (rank == 0) and any(n.startswith("blocks.3.") for n in owned) == (rank == 1)
    losses = []
    for ids in _batches(steps):
        tm.zero_grads()
        tm.train_batch({"input_ids": ids})
        tm.optim_step()
        losses.append(float(tm.latest_ce_loss))  # known on EVERY pipeline rank
    sd = tm.state_dict()
    assert set(sd) == {"model", "optim"} and all(k in sd["model"] for k in owned)
    assert all(f"state.{k}.exp_avg" in sd["optim"] for k in owned)
    # round trip into a freshly built module on the same ranks
    saved = {k: (v.detach().clone() if torch.is_tensor(v) else v) for k, v in sd["model"].items()}
    saved_opt = {k: (v.detach().clone() if torch.is_tensor(v) else v) for k, v in sd["optim"].items()}
    tm2 = build()
    tm2.load_state_dict({"model": saved, "optim": saved_opt})
    sd2 = tm2.state_dict()
    for k in owned:
        assert torch.equal(sd2["model"][k], saved[k]), k
        assert torch.equal(sd2["optim"][f"state.{k}.exp_avg"], saved_opt[f"state.{k}.exp_avg"]), k
    torch.save({"losses": losses, "params": saved}, Path(tmp) / f"rank{rank}.pt")


def test_two_stage_pipeline_matches_single_process(tmp_path):
    steps = 3
    ref_losses, ref_params = _single_process_reference(steps, tmp_path / "init.pt")
    run_distributed_test(_pp_worker, world_size=2, func_args=(str(tmp_path), steps))
    r0 = torch.load(tmp_path / "rank0.pt", weights_only=False)
    r1 = torch.load(tmp_path / "rank1.pt", weights_only=False)
    assert r0["losses"] == pytest.approx(r1["losses"], rel=1e-6)  # the loss reached the first stage's rank too
    assert r0["losses"] == pytest.approx(ref_losses, rel=2e-4)
    merged = {**r0["params"], **r1["params"]}
    assert set(merged) == set(ref_params)
    for n, want in ref_params.items():
        err = (merged[n] - want).norm() / want.norm().clamp(min=1e-12)
        assert err < 2e-3, (n, float(err))
