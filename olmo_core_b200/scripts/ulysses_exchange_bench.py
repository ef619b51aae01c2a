"""
Time the Ulysses sequence <-> head exchange of q, k, v (``cp2hp``) plus the output's way back (``hp2cp``), forward and
backward, with the peer-memory kernel and with the NCCL all-to-all path, on the ranks of a ``torchrun`` job (one node):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m olmo_core_b200.scripts.ulysses_exchange_bench

Device time by CUDA events after warm-up, maximum over ranks; rank 0 prints one JSON line per path.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--seq", type=int, default=65536, help="length of the whole sequence")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=32)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()

    from olmo_core_b200.distributed.parallel.context_parallel import all_to_all_cp2hp, all_to_all_single_hp2cp
    from olmo_core_b200.ops import _lib

    dist.init_process_group("cpu:gloo,cuda:nccl")
    rank, cp = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    t = args.seq // cp
    q = torch.randn(1, t, args.heads, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(1, t, args.kv_heads, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(1, t, args.kv_heads, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        qh, kh, vh = all_to_all_cp2hp([q, k, v], dist.group.WORLD)
        out = all_to_all_single_hp2cp(qh, dist.group.WORLD)  # attention's output has the shape of q
        torch.autograd.backward([out, kh, vh], [out.detach(), kh.detach(), vh.detach()])

    for path, flag in (("peer_memory_kernel", "1"), ("nccl_all_to_all", "0")):
        os.environ["OLMO_CORE_B200_ULYSSES_PEER"] = flag
        for _ in range(3):
            step()
        times = []
        for _ in range(args.iters):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        tm = torch.tensor(sorted(times)[len(times) // 2], device=dev)
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        _lib.check_device_status()
        if rank == 0:
            moved = 2 * (2 * args.heads + 2 * args.kv_heads) * t * 128 * 2 * (cp - 1) / cp  # bytes sent per rank, fwd + bwd
            print(json.dumps({"path": path, "ranks": cp, "seq": args.seq, "heads": args.heads, "kv_heads": args.kv_heads,
                              "ms_max_over_ranks": round(float(tm), 3),
                              "nvlink_gb_per_s_per_rank": round(moved / float(tm) / 1e6, 1)}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
