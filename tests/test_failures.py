"""
Failure handling, exercised on the host only (gloo ranks on CPU, files on disk): a rank that cancels or raises, a
checkpoint that is truncated or lost its metadata, a loss that turns into NaN, a resume on a different world size.
No test here touches a GPU.
"""

import json
import time
from dataclasses import dataclass
from pathlib import Path

import pytest
import torch

from test_trainer import Recorder, _build, _write_data

from olmo_core_b200.distributed.utils import get_rank
from olmo_core_b200.testing import run_distributed_test
from olmo_core_b200.train.callbacks import Callback


# ---------------------------------------------------------------------------------------------------------
# ranks that cancel / raise
# ---------------------------------------------------------------------------------------------------------
def _cancel_from_rank_one(tmp: str):
    tmp_path = Path(tmp)
    rec = Recorder(cancel_at=2 if get_rank() == 1 else -1)
    trainer, _ = _build(tmp_path, max_steps=8, dp=True, recorder=rec)
    trainer.fit()
    (tmp_path / f"rank{get_rank()}.json").write_text(json.dumps(
        {"step": trainer.global_step, "canceled": trainer.is_canceled, "reason": trainer._cancel_reason,
         "by": trainer._canceling_rank}))


def test_cancellation_from_one_rank_stops_all_ranks(tmp_path):
    _write_data(tmp_path / "tokens.npy")
    run_distributed_test(_cancel_from_rank_one, world_size=2, func_args=(str(tmp_path),))
    r0, r1 = (json.loads((tmp_path / f"rank{r}.json").read_text()) for r in (0, 1))
    assert r0["canceled"] and r1["canceled"] and r0["by"] == r1["by"] == 1
    assert r0["reason"] == r1["reason"] == "test asked for it"
    assert r0["step"] == r1["step"] < 8  # both stopped at the same step, long before the end


@dataclass
class _Bomb(Callback):
    at: int = 2

    def post_step(self) -> None:
        if self.step == self.at and get_rank() == 1:
            raise RuntimeError("injected failure on rank 1")


def _one_rank_raises(tmp: str):
    tmp_path = Path(tmp)
    trainer, _ = _build(tmp_path, max_steps=50, dp=True)
    trainer.callbacks["bomb"] = _Bomb()
    trainer.callbacks["bomb"].trainer = trainer
    t0 = time.time()
    try:
        trainer.fit()
        outcome = "finished"
    except BaseException as e:  # noqa: BLE001 - the point is that *something* comes back instead of a hang
        outcome = f"{type(e).__name__}: {str(e)[:200]}"
    (tmp_path / f"rank{get_rank()}.json").write_text(json.dumps(
        {"outcome": outcome, "seconds": time.time() - t0, "step": trainer.global_step}))


def test_a_rank_that_raises_surfaces_on_its_peer(tmp_path):
    """Rank 1 dies in a callback; rank 0's next collective over gloo must fail promptly, not wait forever."""
    _write_data(tmp_path / "tokens.npy")
    t0 = time.time()
    try:
        run_distributed_test(_one_rank_raises, world_size=2, func_args=(str(tmp_path),))
    except Exception:
        pass  # the launcher may report the children's exit; what matters is what the ranks saw
    assert time.time() - t0 < 240
    r1 = json.loads((tmp_path / "rank1.json").read_text())
    assert "injected failure" in r1["outcome"]
    r0_file = tmp_path / "rank0.json"
    if r0_file.exists():  # rank 0 got as far as reporting: it must have seen an error, not a completed run
        r0 = json.loads(r0_file.read_text())
        assert r0["outcome"] != "finished" and r0["step"] < 50


# ---------------------------------------------------------------------------------------------------------
# damaged checkpoints
# ---------------------------------------------------------------------------------------------------------
def _saved_checkpoint(tmp_path: Path) -> Path:
    trainer, _ = _build(tmp_path, max_steps=2, save_interval=2)
    trainer.fit()
    ckpt = tmp_path / "run" / "step2" / "model_and_optim"
    assert (ckpt / ".metadata").is_file()
    return ckpt


def test_truncated_shard_file_is_reported(tmp_path):
    from olmo_core_b200.distributed.checkpoint import load_model_and_optim_state

    ckpt = _saved_checkpoint(tmp_path)
    shard = max(ckpt.glob("*.distcp"), key=lambda p: p.stat().st_size)
    data = shard.read_bytes()
    shard.write_bytes(data[: len(data) // 3])
    from olmo_core_b200.exceptions import OLMoCheckpointError

    (tmp_path / "fresh").mkdir()
    trainer, _ = _build(tmp_path / "fresh", max_steps=1)
    with pytest.raises(OLMoCheckpointError) as info:
        load_model_and_optim_state(str(ckpt), trainer.train_module.model, trainer.train_module.optim)
    assert shard.name in str(info.value) and ("truncated" in str(info.value) or "damaged" in str(info.value))


def test_missing_metadata_is_reported(tmp_path):
    from olmo_core_b200.distributed.checkpoint import load_model_and_optim_state

    ckpt = _saved_checkpoint(tmp_path)
    (ckpt / ".metadata").unlink()
    (tmp_path / "fresh").mkdir()
    trainer, _ = _build(tmp_path / "fresh", max_steps=1)
    with pytest.raises((FileNotFoundError, OSError, RuntimeError, Exception)) as info:
        load_model_and_optim_state(str(ckpt), trainer.train_module.model, trainer.train_module.optim)
    assert ".metadata" in str(info.value) or "metadata" in str(info.value).lower()


def test_trainer_ignores_a_checkpoint_directory_without_trainer_metadata(tmp_path):
    """A step directory whose ``.metadata.json`` never got written (a save that died half way) is not resumed from."""
    trainer, _ = _build(tmp_path, max_steps=4, save_interval=2)
    trainer.fit()
    (tmp_path / "run" / "step4" / ".metadata.json").unlink()
    again, rec = _build(tmp_path, max_steps=4, save_interval=2)
    again.fit()
    assert again.checkpoint_loaded and sorted(rec.losses) == [3, 4]  # resumed from step 2, the last complete one


# ---------------------------------------------------------------------------------------------------------
# NaN loss
# ---------------------------------------------------------------------------------------------------------
def test_nan_loss_skips_the_optimizer_step():
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.optim import SkipStepAdamWConfig

    torch.manual_seed(0)
    model = TransformerConfig.olmo2_30M(vocab_size=128, n_layers=1).build(init_device="cpu")
    model.init_weights(max_seq_len=16, device=torch.device("cpu"))
    optim = SkipStepAdamWConfig(lr=1e-2, rolling_interval_length=4, sigma_factor=3).build(model)
    ids = torch.randint(0, 128, (2, 16))
    for _ in range(6):  # fill the loss window with ordinary values
        optim.zero_grad()
        out = model(ids, labels=ids)
        out.loss.backward()
        optim.latest_loss = out.loss.detach()
        optim.step()
    before = [p.detach().clone() for p in model.parameters()]
    optim.zero_grad()
    out = model(ids, labels=ids)
    out.loss.backward()
    optim.latest_loss = torch.tensor(float("nan"))
    optim.step()
    assert float(optim.step_skipped) == 1.0
    for p, q in zip(model.parameters(), before):
        assert torch.equal(p.detach(), q)


# ---------------------------------------------------------------------------------------------------------
# resume on another world size
# ---------------------------------------------------------------------------------------------------------
def _two_ranks_two_steps(tmp: str):
    # the full four-step schedule, interrupted after two steps (the learning rate depends on the planned length)
    trainer, _ = _build(Path(tmp), max_steps=4, save_interval=2, dp=True, recorder=Recorder(cancel_at=2))
    trainer.fit()


def test_resume_on_a_different_world_size(tmp_path):
    ref_dir, run_dir = tmp_path / "ref", tmp_path / "run2to1"
    ref_dir.mkdir(), run_dir.mkdir()
    ref, ref_rec = _build(ref_dir, max_steps=4)
    ref.fit()
    _write_data(run_dir / "tokens.npy")
    run_distributed_test(_two_ranks_two_steps, world_size=2, func_args=(str(run_dir),))
    resumed, rec = _build(run_dir, max_steps=4, save_interval=2)
    resumed.fit()
    # the cancellation is agreed on one step after it was asked for, so the two-rank run ended at step 2 or 3
    assert resumed.checkpoint_loaded and resumed.global_step == 4 and 4 in rec.losses and set(rec.losses) <= {3, 4}
    for step, loss in rec.losses.items():  # the same global batches in the same order, whatever the number of ranks
        assert loss == pytest.approx(ref_rec.losses[step], rel=5e-4), step
