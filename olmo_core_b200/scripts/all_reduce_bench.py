"""
All-reduce bandwidth over the GPUs of this job (role of src/scripts/train/all_reduce_bench.py)::

    torchrun --nproc-per-node=8 -m olmo_core_b200.scripts.all_reduce_bench [--gib 1.0] [--trials 5]

Reports, per payload, the algorithm bandwidth (payload / time) and the bus bandwidth (x 2(n-1)/n, the figure that is
comparable across rank counts) of ``torch.distributed.all_reduce`` (NCCL), and of this package's own gradient reduction
kernel over peer memory (every rank reduces its shard by loading it from all peers: a reduce-scatter, bus factor
(n-1)/n). Times are CUDA events on the launching stream, maximum over ranks.
"""

import argparse
import ctypes
import json

import torch
import torch.distributed as dist

from ..train import prepare_training_environment, teardown_training_environment


def _timed(fn, trials: int) -> float:
    for _ in range(2):
        fn()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    dist.barrier()
    start.record()
    for _ in range(trials):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(end) / trials], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms) / 1e3


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--gib", type=float, nargs="*", default=[0.0625, 0.25, 1.0], help="payload sizes in GiB (fp32)")
    p.add_argument("--trials", type=int, default=5)
    args = p.parse_args(argv)
    prepare_training_environment()
    n, rank = dist.get_world_size(), dist.get_rank()
    rows = []
    for gib in args.gib:
        numel = int(gib * 2**30 / 4) // (n * 1024) * (n * 1024)
        payload = numel * 4
        x = torch.rand(numel, device="cuda")
        t = _timed(lambda: dist.all_reduce(x), args.trials)
        row = {"payload_gib": payload / 2**30, "ranks": n, "nccl_all_reduce_algbw_gbs": payload / t / 1e9,
               "nccl_all_reduce_busbw_gbs": payload / t / 1e9 * 2 * (n - 1) / n}
        if n > 1:
            try:
                from ..ops import _lib
                from ..parallel.symmetric import SymmetricBuffer

                buf = SymmetricBuffer(numel, torch.float32, x.device)
                buf.tensor.copy_(x)
                shard = numel // n
                out = torch.empty(shard, device="cuda")
                scratch = torch.empty(_lib.lib().ocb_fused_partials(), device="cuda")
                sumsq = torch.zeros(1, device="cuda")

                def fused():
                    buf.barrier()
                    rc = _lib.lib().ocb_peer_reduce_sumsq(buf.peer_ptrs, buf.multicast_ptr, n, rank * shard, shard,
                                                          ctypes.c_float(1.0), out.data_ptr(), scratch.data_ptr(),
                                                          sumsq.data_ptr(), _lib.stream_ptr())
                    _lib.check(rc, "ocb_peer_reduce_sumsq")

                tf = _timed(fused, args.trials)
                row["peer_reduce_scatter_algbw_gbs"] = payload / tf / 1e9
                row["peer_reduce_scatter_busbw_gbs"] = payload / tf / 1e9 * (n - 1) / n
            except Exception as e:  # peer memory not available on this machine
                row["peer_reduce_scatter"] = f"unavailable: {e}"
        rows.append(row)
    if rank == 0:
        print(json.dumps(rows, indent=1))
    teardown_training_environment()


if __name__ == "__main__":
    main()
