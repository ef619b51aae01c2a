"""
Headline benchmark: OLMo-2 7B pre-training throughput (tokens/s, whole job) with sharded data parallelism
in bf16 on N B200 GPUs of one node, synthetic uniform-random token ids, random-init weights.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

``--impl reference`` runs the unmodified reference implementation installed under ``baseline/_ref`` through
its own public API on the same config and prints the same JSON line.

A *step* is one optimizer step on the named config: micro-batch 2 x 4096 tokens per GPU, 128 sequences per
GPU per step (global batch 1024 sequences at 8 GPUs), AdamW with gradient clipping at 1.0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))
PEAK_BF16_FLOPS = 2.25e15  # dense bf16 peak the reference's MFU meter uses for B200


# The benchmark configurations: the headline one (OLMo-2 7B, sharded data parallel) and the other model / parallelism
# combinations the same step function is measured on. Each entry overrides command-line defaults; an explicit flag wins.
CONFIGS = {
    "olmo2_7B_fsdp": dict(model="olmo2_7B", seq_len=4096, micro_batch=2, seqs_per_gpu=128, vocab_size=100352),
    # OLMo-2 32B, tensor parallel 2 (sequence parallel) x sharded data parallel N/2, row-wise fp8 linear layers
    "olmo2_32B_tp2_fsdp4_fp8": dict(model="olmo2_32B", seq_len=4096, micro_batch=1, seqs_per_gpu=8, vocab_size=100352,
                                    tp=2, fp8="rowwise"),
    # the headline model with 8-bit linear layers: row-wise scaled e4m3, and block-scaled MX (32-element E8M0 scales)
    "olmo2_7B_fsdp_fp8": dict(model="olmo2_7B", seq_len=4096, micro_batch=2, seqs_per_gpu=128, vocab_size=100352, fp8="rowwise"),
    "olmo2_7B_fsdp_mxfp8": dict(model="olmo2_7B", seq_len=4096, micro_batch=2, seqs_per_gpu=128, vocab_size=100352, fp8="mx"),
    # OLMoE-1B-7B, experts spread over all N GPUs, the rest sharded data parallel
    "olmoe_1B_7B_ep8": dict(model="olmoe_1B_7B", seq_len=4096, micro_batch=4, seqs_per_gpu=32, vocab_size=50304, ep=0),
    # OLMo-3 7B long context: ONE 65536-token sequence per context-parallel group of all N GPUs
    "olmo3_7B_cp8": dict(model="olmo3_7B", seq_len=65536, micro_batch=1, seqs_per_gpu=1, vocab_size=100352, cp=0),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", default="olmo2_7B")
    ap.add_argument("--layers", type=int, default=None, help="override the number of layers (debugging only)")
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=2, help="sequences per micro-batch per GPU")
    ap.add_argument("--seqs-per-gpu", type=int, default=128, help="sequences per GPU per optimizer step")
    ap.add_argument("--vocab-size", type=int, default=100352)
    ap.add_argument("--no-e2e", action="store_true", help="accepted for compatibility; both numbers come from one loop")
    ap.add_argument("--config", default="olmo2_7B_fsdp", choices=sorted(CONFIGS),
                    help="which of the benchmark configurations to run (default: the headline one)")
    a = ap.parse_args()
    cfg = CONFIGS[a.config]
    given = {x.split("=")[0] for x in sys.argv[1:] if x.startswith("--")}
    for key, flag in (("model", "--model"), ("seq_len", "--seq-len"), ("micro_batch", "--micro-batch"),
                      ("seqs_per_gpu", "--seqs-per-gpu"), ("vocab_size", "--vocab-size")):
        if flag not in given:
            setattr(a, key, cfg[key])
    a.tp, a.fp8 = cfg.get("tp"), cfg.get("fp8")
    a.ep = a.gpus if cfg.get("ep") == 0 else cfg.get("ep")  # 0: all GPUs of the job
    a.cp = a.gpus if cfg.get("cp") == 0 else cfg.get("cp")
    return a


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i",
                 str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(maxc) if maxc else None,
                "reasons": sorted(reasons), "samples": len(clocks)}


def run_ours(args):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, REPO)
    from olmo_core_b200.config import DType
    from olmo_core_b200.nn.lm_head import LMLossImplementation
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.optim import AdamWConfig, OptimGroupOverride
    from olmo_core_b200.train.train_module import TransformerDataParallelConfig, TransformerTrainModuleConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N>1")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        from olmo_core_b200.distributed.utils import init_distributed

        init_distributed(backend="cpu:gloo,cuda:nccl")
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

    kwargs = {}
    if args.layers is not None:
        kwargs["n_layers"] = args.layers
    cfg = getattr(TransformerConfig, args.model)(vocab_size=args.vocab_size, **kwargs)
    cfg.lm_head.loss_implementation = LMLossImplementation.fused_linear
    model = cfg.build(init_device="meta")
    flops_per_token = model.num_flops_per_token(args.seq_len)
    extra = {}
    parallelism = f"fsdp{world}"
    if args.tp and args.tp > 1:
        from olmo_core_b200.train.train_module import TransformerTensorParallelConfig

        extra["tp_config"] = TransformerTensorParallelConfig(degree=args.tp)
        parallelism = f"tp{args.tp} x fsdp{world // args.tp}"
    if args.ep and args.ep > 1:
        from olmo_core_b200.train.train_module import TransformerExpertParallelConfig

        extra["ep_config"] = TransformerExpertParallelConfig(degree=args.ep)
        # expert parallelism rides on the shard dimension of hybrid sharding (one replica group here)
        extra["dp_config"] = TransformerDataParallelConfig(name="hsdp", param_dtype=DType.bfloat16, reduce_dtype=DType.float32,
                                                           shard_degree=args.ep)
        parallelism = f"ep{args.ep} + hsdp(shard {args.ep})"
    if args.cp and args.cp > 1:
        from olmo_core_b200.train.train_module import TransformerContextParallelConfig

        # contiguous shards: the layout that works with sliding-window layers (the published long-context recipe uses it)
        extra["cp_config"] = TransformerContextParallelConfig.llama3(degree=args.cp)
        parallelism = f"cp{args.cp} (llama3 layout) x dp{world // args.cp}"
    if args.fp8:
        from olmo_core_b200.float8 import AOFloat8LinearConfig, AOMXLinearConfig, Float8Config

        # quantised weights are kept for all micro-batches of a step (dropped after the parameter update)
        ao = AOFloat8LinearConfig(enable_fsdp_float8_all_gather=True)
        if args.fp8 == "mx":
            f8 = Float8Config(enabled=True, ao_mx=AOMXLinearConfig.mxfp8_cublas_rceil(), cache_weight_casts=True)
            parallelism += ", MX fp8 (e4m3, E8M0 scale per 32) linear layers"
        else:
            f8 = Float8Config(enabled=True, ao=ao)
            parallelism += ", fp8 row-wise linear layers"
        extra["float8_config"] = f8
    tm = TransformerTrainModuleConfig(
        rank_microbatch_size=args.micro_batch * args.seq_len,
        max_sequence_length=args.seq_len,
        optim=AdamWConfig(lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1,
                          group_overrides=[OptimGroupOverride(params=["embeddings.weight"], opts=dict(weight_decay=0.0))]),
        max_grad_norm=1.0,
        z_loss_multiplier=1e-5,
        dp_config=extra.pop("dp_config", None) or TransformerDataParallelConfig(
            name="fsdp", param_dtype=DType.bfloat16, reduce_dtype=DType.float32),
        **extra,
    ).build(model, device=device)

    seqs = args.seqs_per_gpu
    dp_ranks = world // (args.cp or 1) // (args.tp or 1)  # ranks of a context- / tensor-parallel group share their batch
    tokens_per_step_global = seqs * args.seq_len * dp_ranks
    gen = torch.Generator().manual_seed(1234 + rank // ((args.cp or 1) * (args.tp or 1)))  # one batch per data-parallel rank
    n_host_batches = args.warmup + args.steps
    host_batches = [torch.randint(0, args.vocab_size, (seqs, args.seq_len), generator=gen, dtype=torch.int64).pin_memory()
                    for _ in range(min(n_host_batches, 4))]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step(ids_host):
        """One optimizer step through the public train-module API: pinned host ids in, loss read back to the host."""
        tm.zero_grads()
        tm.train_batch({"input_ids": ids_host})  # copies ids and labels host -> device, micro-batch by micro-batch
        tm.optim_step()
        return tm.latest_ce_loss.item()  # device -> host read of the step's result

    for i in range(args.warmup):
        step(host_batches[i % len(host_batches)])
    _lib.check_device_status(device)

    # ONE timed loop gives both numbers: CUDA events on the launching stream bracket exactly the `steps` steps
    # (value), the wall clock around the same loop gives the end-to-end figure (e2e). Every step copies its inputs
    # from pinned host memory and reads its loss back.
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    launches0 = _lib.launch_count
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h2d = d2h = 0
    t0 = time.perf_counter()
    start.record()
    for i in range(args.steps):
        ids = host_batches[i % len(host_batches)]
        loss = step(ids)
        h2d += ids.numel() * ids.element_size() * 2  # input ids and labels of every micro-batch
        d2h += 4
    end.record()
    barrier()
    wall_s = time.perf_counter() - t0
    clocks = sampler.stop()
    launches = _lib.launch_count - launches0
    t = torch.tensor([start.elapsed_time(end), wall_s * 1e3], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = t[0].item() / args.steps
    _lib.check_device_status(device)
    e2e = {"value": tokens_per_step_global * args.steps / (t[1].item() / 1e3), "unit": "tokens/s",
           "h2d_bytes_per_step": h2d // max(args.steps, 1), "d2h_bytes_per_step": d2h // max(args.steps, 1),
           "last_loss": loss, "timed": "wall clock around the same loop as the CUDA events, max over ranks"}

    value = tokens_per_step_global / (ms_per_step / 1e3)
    if rank == 0:
        out = {
            "metric": ("tokens/sec/GPU + MFU, OLMo-2 7B FSDP bf16 at 1/2/4/8 B200, device-timed (value = whole-job tokens/s)"
                       if args.config == "olmo2_7B_fsdp" else f"tokens/sec, {args.config}, device-timed (value = whole-job tokens/s)"),
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16 (fp8 e4m3 linear layers)" if args.fp8 else "bf16",
            "data": "synthetic uniform-random token ids, random-init weights",
            "tokens_per_sec_per_gpu": value / world,
            "mfu": value / world * flops_per_token / PEAK_BF16_FLOPS,
            "config": {"name": args.config, "model": args.model, "n_layers": cfg.n_layers, "global_batch": seqs * dp_ranks,
                       "seq_len": args.seq_len, "micro_batch": args.micro_batch, "parallelism": parallelism,
                       "optimizer": "AdamW, clip 1.0",
                       "l2": "working set per step (14.6 GB bf16 weights + activations) is far larger than the 126 MB L2"},
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": launches,
            "impl": "ours",
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_reference(args):
    """Replace this process with ``baseline/run_reference.py`` running against ``baseline/_ref`` (never our package)."""
    ref = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "olmo_core")):
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is missing: the offline install of the "
                              "reference has not been done on this machine"}), flush=True)
        return
    env = dict(os.environ)
    env.setdefault("OCB_REF_T0", repr(time.time()))
    env["PYTHONPATH"] = os.pathsep.join([os.path.join(REPO, "baseline", "shims"), ref])
    script = os.path.join(REPO, "baseline", "run_reference.py")
    os.chdir(os.path.join(REPO, "baseline"))  # keep the repo root (and its 'olmo_core' alias package) off sys.path
    os.execve(sys.executable, [sys.executable, script] + sys.argv[1:], env)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
