"""Trainer end to end on CPU: fit, metrics, checkpoints, resume, cancellation, and two gloo ranks against one."""

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List

import numpy as np
import pytest
import torch

from olmo_core_b200.data import DataCollator, NumpyFSLDataLoader, NumpyFSLDatasetConfig, TokenizerConfig
from olmo_core_b200.distributed.utils import get_rank, get_world_size
from olmo_core_b200.nn.transformer import TransformerConfig
from olmo_core_b200.optim import AdamWConfig, CosWithWarmup
from olmo_core_b200.testing import run_distributed_test
from olmo_core_b200.train import Duration, TrainerConfig
from olmo_core_b200.train.callbacks import Callback, CheckpointerCallback
from olmo_core_b200.train.train_module import TransformerDataParallelConfig, TransformerTrainModule

VOCAB, SEQ = 512, 32


def _write_data(path: Path, n_tokens: int = 64 * SEQ * 8) -> None:
    rng = np.random.default_rng(0)
    arr = rng.integers(2, VOCAB, n_tokens).astype(np.uint16)
    arr[SEQ - 1:: SEQ] = 1
    mm = np.memmap(path, mode="w+", dtype=np.uint16, shape=arr.shape)
    mm[:] = arr
    mm.flush()


@dataclass
class Recorder(Callback):
    steps: List[int] = field(default_factory=list)
    losses: Dict[int, float] = field(default_factory=dict)
    cancel_at: int = -1

    def log_metrics(self, step: int, metrics: Dict[str, float]) -> None:
        self.steps.append(step)
        if "train/CE loss" in metrics:
            self.losses[step] = metrics["train/CE loss"]

    def post_step(self) -> None:
        if self.step == self.cancel_at:
            self.trainer.cancel_run("test asked for it")


def _build(tmp_path: Path, *, max_steps: int, save_interval: int = 1000, dp: bool = False, gbs_instances: int = 8,
           recorder: Recorder = None, seed: int = 0):
    torch.manual_seed(seed)
    data = tmp_path / "tokens.npy"
    if not data.exists() and get_rank() == 0:
        _write_data(data)
    if dp:
        torch.distributed.barrier()
    tok = TokenizerConfig(vocab_size=VOCAB, eos_token_id=1, pad_token_id=0)
    ds = NumpyFSLDatasetConfig(tokenizer=tok, paths=[str(data)], sequence_length=SEQ, work_dir=str(tmp_path / "dwork")).build()
    ds.prepare()
    ws = get_world_size()
    loader = NumpyFSLDataLoader(ds, collator=DataCollator(pad_token_id=0), global_batch_size=gbs_instances * SEQ,
                                work_dir=tmp_path / "dwork", seed=1, dp_world_size=ws, dp_rank=get_rank(), fs_local_rank=get_rank())
    model = TransformerConfig.olmo2_30M(vocab_size=VOCAB, n_layers=2).build(init_device="cpu")
    tm = TransformerTrainModule(
        model=model, optim=AdamWConfig(lr=1e-3), rank_microbatch_size=2 * SEQ, max_sequence_length=SEQ,
        scheduler=CosWithWarmup(warmup_steps=2), max_grad_norm=1.0, device=torch.device("cpu"),
        dp_config=TransformerDataParallelConfig(name="fsdp") if dp else None,
    )
    rec = recorder or Recorder()
    cfg = TrainerConfig(save_folder=str(tmp_path / "run"), max_duration=Duration.steps(max_steps), metrics_collect_interval=2,
                        save_overwrite=True, device="cpu", cancel_check_interval=1,
                        callbacks={"rec": rec, "checkpointer": CheckpointerCallback(save_interval=save_interval, save_async=False)})
    return cfg.build(tm, loader), rec


def test_fit_checkpoints_and_resumes_identically(tmp_path):
    a_dir, b_dir = tmp_path / "a", tmp_path / "b"
    a_dir.mkdir(), b_dir.mkdir()
    trainer, rec = _build(a_dir, max_steps=6)
    trainer.fit()
    assert trainer.global_step == 6 and sorted(rec.losses) == [1, 2, 3, 4, 5, 6]
    assert all(np.isfinite(v) for v in rec.losses.values()) and len(rec.losses) == 6
    run = a_dir / "run"
    assert (run / "step0" / ".metadata.json").is_file() and (run / "step6" / "train" / "rank0.pt").is_file()
    assert json.loads((run / "step6" / ".metadata.json").read_text())["ephemeral"] is False

    # same run, interrupted after 3 steps and resumed: identical losses and weights
    part, rec1 = _build(b_dir, max_steps=6, save_interval=3, recorder=Recorder(cancel_at=3))
    part.fit()
    assert part.global_step == 3 and part.is_canceled
    resumed, rec2 = _build(b_dir, max_steps=6, save_interval=3)
    resumed.fit()
    assert resumed.checkpoint_loaded and resumed.global_step == 6 and sorted(rec2.losses) == [4, 5, 6]
    for step in (4, 5, 6):
        assert rec2.losses[step] == pytest.approx(rec.losses[step], rel=1e-5)
    for p, q in zip(trainer.train_module.model.parameters(), resumed.train_module.model.parameters()):
        torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)


def _two_rank_run(tmp_path_str: str):
    tmp_path = Path(tmp_path_str)
    trainer, rec = _build(tmp_path, max_steps=4, dp=True)
    trainer.fit()
    if get_rank() == 0:
        (tmp_path / "losses.json").write_text(json.dumps(rec.losses))


def test_two_sharded_ranks_match_one_rank(tmp_path):
    one, two = tmp_path / "one", tmp_path / "two"
    one.mkdir(), two.mkdir()
    trainer, rec = _build(one, max_steps=4)
    trainer.fit()
    _write_data(two / "tokens.npy")
    run_distributed_test(_two_rank_run, world_size=2, func_args=(str(two),))
    losses = {int(k): v for k, v in json.loads((two / "losses.json").read_text()).items()}
    for step in range(1, 5):
        assert losses[step] == pytest.approx(rec.losses[step], rel=2e-4), step
    # the sharded checkpoint of two ranks restores into one unsharded rank
    from olmo_core_b200.distributed.checkpoint import load_model_and_optim_state

    fresh = TransformerConfig.olmo2_30M(vocab_size=VOCAB, n_layers=2).build(init_device="cpu")
    fresh.init_weights(max_seq_len=SEQ, device=torch.device("cpu"))
    load_model_and_optim_state(two / "run" / "step4" / "model_and_optim", fresh)
    for (n, p), q in zip(trainer.train_module.model.named_parameters(), fresh.parameters()):
        torch.testing.assert_close(p, q, rtol=1e-3, atol=1e-5, msg=n)


def _inconsistent_metrics_worker():
    import torch.distributed as dist

    from olmo_core_b200.train.common import ReduceType
    from olmo_core_b200.train.utils import check_metrics_consistent, reduce_metrics

    rank = dist.get_rank()
    kinds = {"shared": ReduceType.mean, "norm": ReduceType.l2_norm}
    metrics = {1: {"shared": torch.tensor(float(rank + 1)), "norm": torch.tensor(3.0 if rank == 0 else 4.0)}}
    if rank == 1:  # only this rank knows the loss, as with the last stage of a pipeline
        kinds["loss"] = ReduceType.mean
        metrics[1]["loss"] = torch.tensor(2.5)
        kinds["peak"] = ReduceType.max
        metrics[1]["peak"] = torch.tensor(7.0)
    consistent = check_metrics_consistent(kinds)
    assert not consistent
    out = reduce_metrics(metrics, kinds, torch.device("cpu"), metrics_consistent=consistent)
    assert out[1]["shared"] == pytest.approx(1.5) and out[1]["norm"] == pytest.approx(5.0)
    assert out[1]["loss"] == pytest.approx(2.5) and out[1]["peak"] == pytest.approx(7.0)


def test_reduce_metrics_that_only_some_ranks_record():
    run_distributed_test(_inconsistent_metrics_worker, world_size=2)
