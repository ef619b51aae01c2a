"""
Time one expert-parallel dropless MoE MLP (forward + backward) with the peer-memory exchange kernel and with the NCCL
all-to-all path, on the ranks of a ``torchrun`` job (one node):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m olmo_core_b200.scripts.moe_exchange_bench

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
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=8192, help="tokens per rank")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()

    from torch.distributed.device_mesh import init_device_mesh

    from olmo_core_b200.nn.moe.mlp import DroplessMoEMLP
    from olmo_core_b200.nn.moe.parallel_mlp import ParallelDroplessMLP
    from olmo_core_b200.ops import _lib

    dist.init_process_group("cpu:gloo,cuda:nccl")
    rank, ws = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    layer = ParallelDroplessMLP(
        mlp=DroplessMoEMLP(d_model=args.d_model, hidden_size=args.hidden, num_experts=args.experts, dtype=torch.bfloat16,
                           init_device="cpu"), top_k=args.top_k).to(dev)
    layer.apply_ep(init_device_mesh("cuda", (ws,), mesh_dim_names=("ep",)))
    gen = torch.Generator().manual_seed(1 + rank)
    x = torch.randn(1, args.tokens, args.d_model, generator=gen).to(dev, torch.bfloat16).requires_grad_(True)
    weights, idx = torch.softmax(torch.randn(args.tokens, args.experts, generator=gen), -1).topk(args.top_k, dim=-1)
    weights = weights.view(1, args.tokens, args.top_k).to(dev).requires_grad_(True)
    idx = idx.view(1, args.tokens, args.top_k).to(dev)
    counts = torch.bincount(idx.reshape(-1), minlength=args.experts)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        layer(x, weights, idx, counts).backward(x.detach().view_as(x))

    for path, flag in (("peer_memory_kernel", "1"), ("nccl_all_to_all", "0")):
        os.environ["OLMO_CORE_B200_EP_PEER"] = flag
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
            print(json.dumps({"path": path, "ranks": ws, "tokens_per_rank": args.tokens, "d_model": args.d_model,
                              "experts": args.experts, "top_k": args.top_k, "fwd_bwd_ms_max_over_ranks": round(float(t), 3)}),
                  flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
