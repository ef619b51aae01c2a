"""
Reference arm of the benchmark: runs the UNMODIFIED reference implementation (installed under ``baseline/_ref``)
through its own public API -- ``TransformerConfig.olmo2_7B`` -> ``TransformerTrainModuleConfig.build`` ->
``TrainerConfig.build(...).fit()`` -- on the same config as ``bench.py``'s own arm, and prints the same JSON line with
``"impl": "reference"``. Nothing of this repository's package is imported here.

Settings follow the reference's own OLMo-2 7B recipe (``src/scripts/train/OLMo2/OLMo2-7B.py:29-58``): FSDP with
per-block wrapping, bf16 parameters / fp32 reduction, ``compile_model=True``, SkipStep-AdamW lr 3e-4 betas (0.9, 0.95)
weight decay 0.1 (none on embeddings), z-loss 1e-5, gradient clipping at 1.0, and the best attention backend that can be
imported on the box (``flash_2`` from the flash-attn package, else PyTorch SDPA).

Inputs come from pinned host memory through a synthetic ``DataLoaderBase`` subclass; the timed region is bracketed by
callback hooks (``pre_step`` of the first timed step, ``post_step`` of the last) with a barrier and a device
synchronisation on both sides, measured with CUDA events, max over ranks. The loss of every step is read back to the
host by the trainer's metric collection (``metrics_collect_interval=1``).
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import statistics
import subprocess
import sys
import tempfile
import time
from dataclasses import dataclass
from typing import Any, Dict, Iterable, Optional

PEAK_BF16_FLOPS = 2.25e15


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}), flush=True)
    sys.exit(0)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="reference")
    ap.add_argument("--model", default="olmo2_7B")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=2)
    ap.add_argument("--seqs-per-gpu", type=int, default=128)
    ap.add_argument("--vocab-size", type=int, default=100352)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--config", default="olmo2_7B_fsdp")
    ap.add_argument("--no-compile", action="store_true", help="debugging only: skip torch.compile")
    ap.add_argument("--ac", choices=["none", "full"], default="none",
                    help="activation checkpointing; 'full' is selected automatically when one GPU runs out of memory")
    ap.add_argument("--no-foreach", action="store_true",
                    help="SkipStepAdamWConfig(foreach=False): the reference's own single-tensor update, without the "
                         "multi-tensor temporaries; selected automatically as the last attempt on one GPU")
    return ap.parse_args()


class _OverBudget(RuntimeError):
    pass


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Clocks:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, idx: int):
        self.idx, self.proc = idx, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        clocks, maxc, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                maxc.append(float(parts[2]))
            except ValueError:
                continue
            reasons.update(n for n, v in zip(names, parts[5:9]) if v.lower().startswith("active"))
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(maxc) if maxc else None,
                "reasons": sorted(reasons), "samples": len(clocks)}


def main() -> None:
    args = parse_args()
    if args.config != "olmo2_7B_fsdp":
        _unavailable(f"the reference arm is written for the headline configuration (olmo2_7B_fsdp) only, not '{args.config}'")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N>1")
    if world == 1 and "RANK" not in os.environ:
        # a single process still goes through the reference's distributed set-up (FSDP over a group of one)
        os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE="1", LOCAL_WORLD_SIZE="1", NUM_NODES="1",
                          MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
    os.environ.setdefault("LOCAL_WORLD_SIZE", str(world))
    os.environ.setdefault("NUM_NODES", "1")
    os.environ.setdefault("OLMO_SHARED_FS", "1")
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

    try:
        import torch
        import torch.distributed as dist

        import olmo_core
        from olmo_core.config import DType
        from olmo_core.data.data_loader import DataLoaderBase
        from olmo_core.distributed.parallel import DataParallelType
        from olmo_core.nn.attention import AttentionBackendName
        from olmo_core.nn.transformer import TransformerConfig
        from olmo_core.optim import CosWithWarmup, OptimGroupOverride, SkipStepAdamWConfig
        from olmo_core.train import Duration, TrainerConfig, prepare_training_environment, teardown_training_environment
        from olmo_core.train.callbacks import Callback, CheckpointerCallback
        from olmo_core.train.train_module import (
            TransformerActivationCheckpointingConfig,
            TransformerActivationCheckpointingMode,
            TransformerDataParallelConfig,
            TransformerDataParallelWrappingStrategy,
            TransformerTrainModuleConfig,
        )
    except Exception as e:  # the reference could not be imported on this box
        _unavailable(f"reference import failed: {type(e).__name__}: {e}")
        return
    if "baseline/_ref" not in olmo_core.__file__.replace(os.sep, "/"):
        _unavailable(f"'olmo_core' resolved to {olmo_core.__file__}, not to the reference install under baseline/_ref")

    # Wall-clock budget of the whole arm, restarts included. A box with several GPUs is running a sweep over N with a
    # limit of 870 s per run; a one-GPU box runs this arm alone with a longer limit.
    chain_t0 = float(os.environ.setdefault("OCB_REF_T0", repr(time.time())))
    time_budget_s = float(os.environ.get("OCB_BENCH_TIME_BUDGET_S", 845 if torch.cuda.device_count() > 1 else 1700))

    prepare_training_environment(seed=1234)
    rank = dist.get_rank()
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)

    try:
        import flash_attn  # noqa: F401

        backend = AttentionBackendName.flash_2
    except Exception:
        backend = AttentionBackendName.torch
    kwargs: Dict[str, Any] = {}
    if args.layers is not None:
        kwargs["n_layers"] = args.layers
    model_config = getattr(TransformerConfig, args.model)(vocab_size=args.vocab_size, attn_backend=backend, **kwargs)
    model = model_config.build(init_device="meta")
    flops_per_token = model.num_flops_per_token(args.seq_len)

    tm_config = TransformerTrainModuleConfig(
        rank_microbatch_size=args.micro_batch * args.seq_len,
        max_sequence_length=args.seq_len,
        optim=SkipStepAdamWConfig(lr=3e-4, weight_decay=0.1, betas=(0.9, 0.95), foreach=not args.no_foreach,
                                  group_overrides=[OptimGroupOverride(params=["embeddings.weight"], opts=dict(weight_decay=0.0))]),
        compile_model=not args.no_compile,
        dp_config=TransformerDataParallelConfig(name=DataParallelType.fsdp, param_dtype=DType.bfloat16,
                                                reduce_dtype=DType.float32,
                                                wrapping_strategy=TransformerDataParallelWrappingStrategy.blocks),
        ac_config=(TransformerActivationCheckpointingConfig(mode=TransformerActivationCheckpointingMode.full)
                   if args.ac == "full" else None),
        z_loss_multiplier=1e-5,
        max_grad_norm=1.0,
        scheduler=CosWithWarmup(warmup_steps=2000),
    )
    train_module = tm_config.build(model, device=device)

    seqs, seq_len = args.seqs_per_gpu, args.seq_len
    total_steps = args.warmup + args.steps
    h2d_bytes = seqs * seq_len * 8

    class SyntheticLoader(DataLoaderBase):
        """Uniform-random token ids, generated once into pinned host memory and served in rotation."""

        def __init__(self):
            super().__init__(work_dir=tempfile.mkdtemp(), global_batch_size=seqs * seq_len * world,
                             dp_world_size=world, dp_rank=rank, fs_local_rank=rank)
            gen = torch.Generator().manual_seed(1234 + rank)
            self.pool = [torch.randint(0, args.vocab_size, (seqs, seq_len), generator=gen, dtype=torch.int64).pin_memory()
                         for _ in range(4)]

        @property
        def total_batches(self) -> Optional[int]:
            return total_steps

        def state_dict(self) -> Dict[str, Any]:
            return {"batches_processed": self.batches_processed}

        def load_state_dict(self, state_dict: Dict[str, Any]):
            self.batches_processed = state_dict["batches_processed"]

        def reshuffle(self, epoch: Optional[int] = None, **kw):
            self._epoch = epoch or 1

        def _iter_batches(self) -> Iterable[Dict[str, Any]]:
            for i in range(self.batches_processed, total_steps):
                yield {"input_ids": self.pool[i % len(self.pool)]}

        def get_mock_batch(self) -> Dict[str, Any]:
            return {"input_ids": self.pool[0][: args.micro_batch]}

        def global_num_tokens_in_batch(self, batch: Dict[str, Any]) -> Optional[int]:
            return batch["input_ids"].numel() * world

    result: Dict[str, Any] = {}

    @dataclass
    class Timer(Callback):
        """Brackets steps ``warmup+1 .. warmup+steps`` with barrier + synchronize and CUDA events."""

        def pre_step(self, batch):
            if self.step == 2 and total_steps > 4:
                torch.cuda.synchronize()
                result["probe_t0"] = time.perf_counter()
            if self.step == args.warmup + 1:
                dist.barrier()
                torch.cuda.synchronize()
                result["clocks"] = _Clocks(local_rank)
                result["clocks"].start()
                result["t0"] = time.perf_counter()
                result["start"] = torch.cuda.Event(enable_timing=True)
                result["end"] = torch.cuda.Event(enable_timing=True)
                result["start"].record()

        def post_step(self):
            if self.step == 2 and "probe_t0" in result:
                # Project the end of the run from the second step (the first one includes compilation). A run that
                # cannot end inside the time budget stops here with an `unavailable` line instead of being killed
                # at the limit, which would also end whatever the caller runs after this arm.
                torch.cuda.synchronize()
                step_s = time.perf_counter() - result.pop("probe_t0")
                projected = torch.tensor([time.time() - chain_t0 + step_s * (total_steps - 2) + 10.0], device=device)
                dist.all_reduce(projected, op=dist.ReduceOp.MAX)
                if projected.item() > time_budget_s:
                    raise _OverBudget(f"{step_s:.1f} s per step, projected {projected.item():.0f} s for "
                                      f"{total_steps} steps")
            if self.step == args.warmup + args.steps:
                result["end"].record()
                dist.barrier()
                torch.cuda.synchronize()
                result["wall"] = time.perf_counter() - result["t0"]
                result["clocks"] = result["clocks"].stop()
                result["ms"] = result["start"].elapsed_time(result["end"])

        def log_metrics(self, step, metrics):
            if "train/CE loss" in metrics:
                result["last_loss"] = metrics["train/CE loss"]

    save_folder = tempfile.mkdtemp(prefix="ref-bench-")
    trainer = TrainerConfig(
        save_folder=save_folder, save_overwrite=True, metrics_collect_interval=1, cancel_check_interval=1000,
        max_duration=Duration.steps(total_steps), no_checkpoints=True, no_evals=True,
    ).with_callback("checkpointer", CheckpointerCallback(enabled=False)).with_callback("bench_timer", Timer()).build(
        train_module, SyntheticLoader())
    try:
        trainer.fit()
    except _OverBudget as e:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": (
                f"the reference runs this config (activation_checkpointing={args.ac}, foreach={not args.no_foreach}) "
                f"but too slowly for the time budget of {time_budget_s:.0f} s per run: {e}")}), flush=True)
        sys.stdout.flush()
        os._exit(0)
    except torch.OutOfMemoryError as e:
        if world == 1 and args.ac == "none":
            # fp32 parameters, gradients and Adam moments of 7.3 B parameters take 117 GB unsharded; with the activations
            # of 32 layers that exceeds one GPU. Start over in a fresh process with the reference's own full activation
            # checkpointing, which is how the reference fits such a run.
            print("reference ran out of memory on one GPU; retrying with full activation checkpointing", flush=True)
            sys.stdout.flush()
            os.execv(sys.executable, [sys.executable] + sys.argv + ["--ac", "full"])
        if world == 1 and not args.no_foreach:
            # Last attempt: the multi-tensor AdamW update allocates temporaries as large as the parameters; the
            # reference's own foreach=False option updates one tensor at a time.
            print("reference ran out of memory again; retrying with SkipStepAdamWConfig(foreach=False)", flush=True)
            sys.stdout.flush()
            os.execv(sys.executable, [sys.executable] + sys.argv + ["--no-foreach"])
        _unavailable(f"reference ran out of device memory on this config: {e}")
        return

    ms = torch.tensor([result["ms"], result["wall"] * 1e3], device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = ms[0].item() / args.steps
    tokens_per_step = seqs * seq_len * world
    value = tokens_per_step / (ms_per_step / 1e3)
    if rank == 0:
        print(json.dumps({
            "metric": "tokens/sec/GPU + MFU, OLMo-2 7B FSDP bf16 at 1/2/4/8 B200, device-timed (value = whole-job tokens/s)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random token ids, random-init weights",
            "tokens_per_sec_per_gpu": value / world, "mfu": value / world * flops_per_token / PEAK_BF16_FLOPS,
            "config": {"model": args.model, "n_layers": model_config.n_layers, "global_batch": seqs * world,
                       "seq_len": seq_len, "micro_batch": args.micro_batch, "parallelism": f"fsdp{world}",
                       "optimizer": "SkipStepAdamW, clip 1.0", "attention_backend": str(backend),
                       "compile_model": not args.no_compile, "activation_checkpointing": args.ac, "foreach": not args.no_foreach,
                       "l2": "working set per step is far larger than the 126 MB L2"},
            "clocks": result["clocks"],
            "e2e": {"value": tokens_per_step * args.steps / (ms[1].item() / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "last_loss": result.get("last_loss")},
            "gpu_launches": None, "impl": "reference", "reference_version": getattr(olmo_core, "__version__", None),
        }), flush=True)
    teardown_training_environment()


if __name__ == "__main__":
    main()
