"""Trainer callbacks in a short CPU fit: monitors, savers, schedulers, notifier, weight averaging."""

import json
import sys
import types
from pathlib import Path

import pytest
import torch

from olmo_core_b200.train import Duration
from olmo_core_b200.train.callbacks import (
    BatchSizeSchedulerCallback,
    ConfigSaverCallback,
    ConsoleLoggerCallback,
    GAPMonitorCallback,
    GarbageCollectorCallback,
    MetricSaverCallback,
    ModelMergeCallback,
    SlackNotifierCallback,
    SpeedMonitorCallback,
    StabilityMonitorCallback,
)

from test_trainer import SEQ, Recorder, _build  # noqa: E402  (same folder; pytest puts it on sys.path)


def _fit(tmp_path, callbacks, max_steps=6, **kwargs):
    trainer, rec = _build(tmp_path, max_steps=max_steps, **kwargs)
    for name, cb in callbacks.items():
        trainer.add_callback(name, cb)
    trainer.fit()
    return trainer, rec


def test_monitors_and_savers(tmp_path):
    seen = {}

    class Grab(Recorder):
        def log_metrics(self, step, metrics):
            seen[step] = dict(metrics)

    trainer, _ = _fit(tmp_path, {
        "speed": SpeedMonitorCallback(),
        "stability": StabilityMonitorCallback(window_size=2),
        "metrics": MetricSaverCallback(fixed_steps=[4]),
        "config": ConfigSaverCallback(),
        "gc": GarbageCollectorCallback(gc_interval=2),
        "console": ConsoleLoggerCallback(log_interval=1),
        "grab": Grab(),
    })
    last = {}
    for step in sorted(seen):
        last.update(seen[step])
    assert any(k.startswith("throughput/") for k in last), sorted(last)
    tps = [v for k, v in last.items() if k.startswith("throughput/") and "TPS" in k]
    assert tps and all(v > 0 for v in tps)
    run = Path(trainer.save_folder)
    assert json.loads((run / "metrics.json").read_text())["step"] == max(seen)
    assert json.loads((run / "metrics_step4.json").read_text())["step"] == 4
    assert any("spike" in k.lower() for k in last), sorted(last)


def test_config_saver_writes_config_and_data_paths(tmp_path):
    cb = ConfigSaverCallback(save_data_paths=True)
    cb.config = {"model": {"d_model": 64}, "seed": 3}
    trainer, _ = _fit(tmp_path, {"config": cb}, max_steps=2, save_interval=2)
    run = Path(trainer.save_folder)
    assert json.loads((run / "config.json").read_text())["seed"] == 3
    assert (run / "data_paths.txt").read_text().strip().endswith("tokens.npy")
    assert (run / "step2" / "config.json").exists()  # copied next to every checkpoint


def test_slack_notifier_posts_start_checkpoint_and_end(tmp_path, monkeypatch):
    posts = []
    requests = types.ModuleType("requests")
    requests.post = lambda url, json, timeout: posts.append((url, json["text"]))
    monkeypatch.setitem(sys.modules, "requests", requests)
    _fit(tmp_path, {"slack": SlackNotifierCallback(name="probe", notifications="all", webhook_url="https://hooks.invalid/x")},
         max_steps=2, save_interval=2)
    texts = [t for _, t in posts]
    assert all(u == "https://hooks.invalid/x" for u, _ in posts)
    assert any("probe" in t and "completed successfully" in t for t in texts), texts
    assert len(texts) >= 2  # at least the start and the end of the run

    posts.clear()

    class Boom(Recorder):
        def post_step(self):
            raise RuntimeError("boom")

    (tmp_path / "b").mkdir()
    with pytest.raises(RuntimeError):
        _fit(tmp_path / "b", {"slack": SlackNotifierCallback(notifications="failure_only", webhook_url="https://hooks.invalid/x"),
                              "boom": Boom()}, max_steps=2)
    assert len(posts) == 1 and "RuntimeError: boom" in posts[0][1]


def test_batch_size_scheduler_doubles_batch_and_scales_lr(tmp_path):
    tokens = 8 * SEQ
    cb = BatchSizeSchedulerCallback(batch_sizes=[tokens, 2 * tokens], schedule=[Duration.steps(0), Duration.steps(3)])
    sizes = {}

    class Sizes(Recorder):
        def pre_step(self, batch):
            sizes[self.step] = batch["input_ids"].numel() * 1  # tokens of this rank's batch

    trainer, _ = _fit(tmp_path, {"bs": cb, "sizes": Sizes()}, max_steps=6)
    assert sizes[1] == tokens and sizes[max(sizes)] == 2 * tokens
    assert trainer.data_loader.global_batch_size == 2 * tokens
    with pytest.raises(Exception):
        BatchSizeSchedulerCallback(batch_sizes=[tokens, 3 * tokens // 2], schedule=[Duration.steps(0), Duration.steps(3)])
    with pytest.raises(Exception):
        BatchSizeSchedulerCallback(batch_sizes=[tokens, 2 * tokens], schedule=[Duration.steps(1), Duration.steps(3)])


def test_gap_monitor_records_activation_and_gradient_statistics(tmp_path):
    seen = {}

    class Grab(Recorder):
        def log_metrics(self, step, metrics):
            seen.update(metrics)

    _fit(tmp_path, {"gap": GAPMonitorCallback(interval=1), "grab": Grab()}, max_steps=3)
    gap = [k for k in seen if k.lower().startswith("gap")]
    assert gap, sorted(seen)[:20]
    assert all(torch.isfinite(torch.tensor(float(seen[k]))) for k in gap)


def test_model_merge_averages_the_last_steps(tmp_path):
    cb = ModelMergeCallback(merge_step=6, merge_last_n_steps=3, enabled=True)
    snapshots = {}

    class Snap(Recorder):
        def post_train_batch(self):
            pass

        def post_step(self):
            p = next(iter(self.trainer.train_module.model.parameters()))
            snapshots[self.step] = p.detach().float().clone()

    trainer, _ = _fit(tmp_path, {"merge": cb, "snap": Snap()}, max_steps=6)
    merged = Path(trainer.save_folder) / "step6-merged"
    assert merged.exists(), sorted(p.name for p in Path(trainer.save_folder).iterdir())
    from olmo_core_b200.distributed.checkpoint import load_model_and_optim_state
    from olmo_core_b200.nn.transformer import TransformerConfig

    model = TransformerConfig.olmo2_30M(vocab_size=512, n_layers=2).build(init_device="cpu")
    load_model_and_optim_state(str(merged / "model_and_optim"), model)
    want = (snapshots[4] + snapshots[5] + snapshots[6]) / 3
    got = next(iter(model.parameters())).detach().float()
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
