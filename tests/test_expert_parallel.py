"""
Expert parallelism of the dropless MoE MLP: two ranks that each own half of the experts must produce the outputs and
gradients of a single rank that owns all of them. Runs on CPU (gloo: the NCCL-style all-to-all path) and, on two GPUs,
through the peer-memory exchange kernel as well.
"""

import os

import pytest
import torch

from olmo_core_b200.testing import requires_multi_gpu, run_distributed_test

D, HID, E, K, N = 64, 32, 4, 2, 96


def _ep_worker(device_type: str, peer: str):
    os.environ["OLMO_CORE_B200_EP_PEER"] = peer
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh

    from olmo_core_b200.nn.moe.mlp import DroplessMoEMLP
    from olmo_core_b200.nn.moe.parallel_mlp import ParallelDroplessMLP
    from olmo_core_b200.ops import moe_peer

    rank, ws = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", rank) if device_type == "cuda" else torch.device("cpu")
    dtype = torch.bfloat16 if device_type == "cuda" else torch.float32
    if device_type == "cuda":
        torch.cuda.set_device(dev)

    def build():
        torch.manual_seed(0)  # the same full set of experts everywhere
        return ParallelDroplessMLP(mlp=DroplessMoEMLP(d_model=D, hidden_size=HID, num_experts=E, dtype=dtype, init_device="cpu"),
                                   top_k=K).to(dev)

    full, sharded = build(), build()
    sharded.apply_ep(init_device_mesh(device_type, (ws,), mesh_dim_names=("ep",)))
    assert sharded.num_local_experts == E // ws

    gen = torch.Generator().manual_seed(10 + rank)  # every rank has its own tokens and routing
    for step in range(3):  # several rounds: the exchange buffers are double-buffered and reused
        x = torch.randn(1, N, D, generator=gen).to(dev, dtype)
        logits = torch.randn(N, E, generator=gen)
        weights, idx = torch.softmax(logits, -1).topk(K, dim=-1)
        weights = weights.view(1, N, K).to(dev, torch.float32)
        idx = idx.view(1, N, K).to(dev)
        counts = torch.bincount(idx.reshape(-1).cpu(), minlength=E).to(dev)
        outs, grads = [], []
        for mod in (full, sharded):
            xi = x.clone().requires_grad_(True)
            wi = weights.clone().requires_grad_(True)
            y = mod(xi, wi, idx, counts)
            y.float().square().sum().backward()
            outs.append(y.detach().float())
            grads.append((xi.grad.float(), wi.grad.float()))
        tol = dict(rtol=3e-2, atol=3e-2) if device_type == "cuda" else dict(rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(outs[1], outs[0], **tol)
        torch.testing.assert_close(grads[1][0], grads[0][0], **tol)
        torch.testing.assert_close(grads[1][1], grads[0][1], **tol)
    # expert weight gradients: this rank's experts saw the tokens of BOTH ranks
    for name in ("w1", "w2", "w3"):
        g_full = getattr(full.mlp, name).grad.float().clone()
        dist.all_reduce(g_full)
        rows = g_full.shape[0] // ws
        tol = dict(rtol=5e-2, atol=5e-2) if device_type == "cuda" else dict(rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(getattr(sharded.mlp, name).grad.float(), g_full[rank * rows:(rank + 1) * rows], **tol)
    if device_type == "cuda":
        from olmo_core_b200.ops import _lib

        _lib.check_device_status()
        used = sum(ex.transfers for ex in moe_peer.PeerExpertExchange._cache.values())
        assert (used > 0) == (peer == "1"), "the peer-memory exchange must be the path that ran iff it is enabled"


def test_expert_parallel_matches_single_rank_on_cpu():
    run_distributed_test(_ep_worker, world_size=2, backend="gloo", func_args=("cpu", "0"))


@pytest.mark.gpu
@requires_multi_gpu
@pytest.mark.parametrize("peer", ["1", "0"])
def test_expert_parallel_peer_exchange_matches_single_rank(peer):
    run_distributed_test(_ep_worker, world_size=2, backend="cuda:nccl,cpu:gloo", func_args=("cuda", peer))
