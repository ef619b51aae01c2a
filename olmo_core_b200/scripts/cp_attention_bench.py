"""
Time context-parallel attention (forward + backward) of one layer three ways -- K / V pushed once into every rank's
sequence-ordered buffer by a peer-memory kernel, K / V tiles read from the owning GPU inside the attention kernels, and
the NCCL all-gather of K / V in front of the same kernels -- on the ranks of a ``torchrun`` job (one node):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m olmo_core_b200.scripts.cp_attention_bench

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
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--layout", choices=["zig_zag", "llama3"], default="zig_zag")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()

    from olmo_core_b200.nn.attention.ring import RingAttentionLoadBalancerType
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.attention import attention
    from olmo_core_b200.parallel import context

    dist.init_process_group("cpu:gloo,cuda:nccl")
    rank, cp = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    window = args.window or None

    class Style:
        load_balancer = RingAttentionLoadBalancerType(args.layout)

    class Backend:
        scale = None

        def _local(self, q_, k_, v_, causal=True):
            return attention(q_, k_, v_, causal=causal, window_size=window)

    Backend.window = window
    T_local = args.seq // cp
    gen = torch.Generator().manual_seed(1 + rank)
    q = torch.randn(1, T_local, args.heads, 128, generator=gen).to(dev, torch.bfloat16).requires_grad_(True)
    k = torch.randn(1, T_local, args.kv_heads, 128, generator=gen).to(dev, torch.bfloat16).requires_grad_(True)
    v = torch.randn(1, T_local, args.kv_heads, 128, generator=gen).to(dev, torch.bfloat16).requires_grad_(True)
    dout = torch.randn(1, T_local, args.heads, 128, generator=gen).to(dev, torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        context.ring_attention(Backend(), q, k, v, group=dist.group.WORLD, style=Style()).backward(dout)

    for path, flag, mode in (("kv_pushed_once_over_peer_memory", "1", "push"),
                             ("kv_tiles_read_from_peers_in_kernel", "1", "direct"),
                             ("nccl_all_gather_then_kernels", "0", "push")):
        os.environ["OLMO_CORE_B200_CP_IN_KERNEL"] = flag
        os.environ["OLMO_CORE_B200_CP_KV"] = mode
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
        t = torch.tensor(sorted(times)[len(times) // 2], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        _lib.check_device_status()
        if rank == 0:
            print(json.dumps({"path": path, "ranks": cp, "seq": args.seq, "heads": args.heads, "kv_heads": args.kv_heads,
                              "window": args.window, "layout": args.layout,
                              "fwd_bwd_ms_max_over_ranks": round(float(t), 3)}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
