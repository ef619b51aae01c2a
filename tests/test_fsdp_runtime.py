"""
Sharded-parameter runtime on CPU / gloo: the streamed memory mode (per-block gather and gradient reduction through a
two-slot ring) must train exactly like the resident mode; parameters whose leading dimension does not divide by the
world size are padded, not replicated, and survive a checkpoint round trip; hybrid sharding with a shard group of one
still averages gradients over the replicas; an unsharded (DDP-style) run agrees with a sharded one.
"""

import os

import pytest
import torch
import torch.distributed as dist

from olmo_core_b200.nn.transformer import TransformerConfig
from olmo_core_b200.optim import AdamWConfig
from olmo_core_b200.testing import run_distributed_test


def _build(vocab=512, layers=3, streamed=None, shard=True, group=None, seed=0):
    from olmo_core_b200.parallel.fsdp import ShardedParamRuntime

    torch.manual_seed(seed)
    model = TransformerConfig.olmo2_30M(vocab_size=vocab, n_layers=layers).build(init_device="cpu")
    model._sharding_runtime = ShardedParamRuntime(model, group=group, param_dtype=None, reduce_dtype=torch.float32,
                                                  shard=shard, streamed=streamed)
    rt = model._sharding_runtime
    rt.materialize(torch.device("cpu"))
    model.init_weights(max_seq_len=64, device=torch.device("cpu"))
    rt.sync_lowp()
    return model, rt


def _steps(model, rt, optim, n=3, micro=2, vocab=512, seed=0):
    g = torch.Generator().manual_seed(100 + seed)
    losses = []
    for _ in range(n):
        rt.zero_grad()
        for _ in range(micro):
            ids = torch.randint(0, vocab, (2, 16), generator=g)
            out = model(ids, labels=ids)
            out.loss.backward()
            losses.append(float(out.loss))
        rt.reduce_gradients()
        optim.step()
    return losses


def _assert_same_params(p1, p0):
    # Adam turns a gradient element that is rounding noise into a +-lr step, and the two modes sum micro-batches and
    # ranks in different orders, so single elements may differ; the tensors as a whole must not.
    for name in p0:
        err = (p1[name] - p0[name]).norm() / p0[name].norm().clamp(min=1e-12)
        assert err < 2e-3, (name, float(err))


def _full_params(rt):
    """Every parameter in full, gathered from the fp32 master shards."""
    out = {}
    for s in rt.slots:
        local = s.param.data
        if s.sharded and rt.world_size > 1:
            parts = [torch.empty_like(local) for _ in range(rt.world_size)]
            dist.all_gather(parts, local.contiguous(), group=rt.group)
            local = torch.cat(parts, 0)[: s.full_shape[0]]
        out[s.name] = local.clone()
    return out


def _streamed_vs_resident(tmp):
    rank = dist.get_rank()
    results = {}
    for mode in (False, True):
        model, rt = _build(streamed=mode)
        assert rt.streamed == mode
        if mode:
            assert len(rt.units) == 3 and all(s.unit >= 0 for u in rt.units for s in u)
            assert rt.lowp_shard is not None and rt._ring_lowp[0].numel() == rt._unit_numel
            # full copies exist only for the resident part (embeddings, final norm, LM head) and two blocks
            assert rt.lowp.numel() < sum(s.flat_numel for s in rt.slots if s.aware) / 2
        optim = AdamWConfig(lr=1e-2, weight_decay=0.1).build(model)
        losses = _steps(model, rt, optim, seed=rank)
        results[mode] = (losses, _full_params(rt), float(rt.grad_norm_sq()))
    (l0, p0, n0), (l1, p1, n1) = results[False], results[True]
    assert l0 == pytest.approx(l1, rel=1e-5)
    assert n0 == pytest.approx(n1, rel=1e-4)
    _assert_same_params(p1, p0)


def test_streamed_mode_trains_like_resident_mode(tmp_path):
    run_distributed_test(_streamed_vs_resident, world_size=2, func_args=(str(tmp_path),))


def _streamed_with_checkpointing(tmp):
    """Activation checkpointing re-runs a block's forward inside the backward pass: the ring must cope."""
    from torch.utils.checkpoint import checkpoint

    rank = dist.get_rank()
    ref_model, ref_rt = _build(streamed=False)
    model, rt = _build(streamed=True)
    for block in model.blocks.values():
        inner = block.forward
        block.forward = (lambda *a, _f=inner, **k: checkpoint(_f, *a, use_reentrant=False, **k))
    o0 = AdamWConfig(lr=1e-2).build(ref_model)
    o1 = AdamWConfig(lr=1e-2).build(model)
    l0 = _steps(ref_model, ref_rt, o0, n=2, seed=rank)
    l1 = _steps(model, rt, o1, n=2, seed=rank)
    assert l0 == pytest.approx(l1, rel=1e-5)


def test_streamed_mode_with_activation_checkpointing(tmp_path):
    run_distributed_test(_streamed_with_checkpointing, world_size=2, func_args=(str(tmp_path),))


def _padded(tmp):
    from olmo_core_b200.distributed.checkpoint import load_model_and_optim_state, save_model_and_optim_state

    rank = dist.get_rank()
    vocab = 515  # not a multiple of 2: rank 0 owns 258 rows, rank 1 owns 257 and one row of padding
    model, rt = _build(vocab=vocab, layers=2)
    emb = rt.slot_for(model.embeddings.weight)
    assert emb.sharded and emb.padded_rows == 516 and emb.local_rows == 258
    assert emb.real_local_rows == (258 if rank == 0 else 257)
    assert tuple(model.embeddings.weight._lowp.shape) == (vocab, model.embeddings.weight._lowp.shape[1])
    optim = AdamWConfig(lr=1e-2).build(model)
    _steps(model, rt, optim, n=2, vocab=vocab, seed=rank)
    if rank == 1:
        assert model.embeddings.weight.data[257:].abs().max() == 0  # padding rows never move
    # a single-process run on the concatenated batches gives the same parameters
    full = _full_params(rt)
    assert full["embeddings.weight"].shape[0] == vocab
    path = os.path.join(tmp, "ckpt")
    save_model_and_optim_state(path, model, optim)
    model2, rt2 = _build(vocab=vocab, layers=2, seed=7)
    optim2 = AdamWConfig(lr=1e-2).build(model2)
    load_model_and_optim_state(path, model2, optim2)
    full2 = _full_params(rt2)
    for n in full:
        assert torch.equal(full[n], full2[n]), n
    if rank == 0:
        torch.save(full, os.path.join(tmp, "full.pt"))


def test_uneven_leading_dimension_is_padded_and_checkpoints(tmp_path):
    from olmo_core_b200.distributed.checkpoint import load_model_and_optim_state

    run_distributed_test(_padded, world_size=2, func_args=(str(tmp_path),))
    # the two-rank checkpoint with uneven shards loads into a single process
    full = torch.load(tmp_path / "full.pt", weights_only=False)
    torch.manual_seed(3)
    model = TransformerConfig.olmo2_30M(vocab_size=515, n_layers=2).build(init_device="cpu")
    model.init_weights(max_seq_len=64, device=torch.device("cpu"))
    optim = AdamWConfig(lr=1e-2).build(model)
    load_model_and_optim_state(str(tmp_path / "ckpt"), model, optim)
    for n, p in model.named_parameters():
        assert torch.equal(p.data, full[n]), n


def _hsdp_shard_one(tmp):
    """A 2-D mesh (replicate=2, shard=1): each replica holds everything; gradients must still be averaged."""
    from torch.distributed.device_mesh import init_device_mesh

    rank = dist.get_rank()
    mesh = init_device_mesh("cpu", (2, 1), mesh_dim_names=("replicate", "shard"))
    model, rt = _build(group=mesh, layers=2)
    assert rt.world_size == 1 and rt.replicate_group is not None and rt.grad_shard is not None
    optim = AdamWConfig(lr=1e-2).build(model)
    _steps(model, rt, optim, n=2, seed=rank)  # different data on the two replicas
    mine = torch.cat([s.param.data.reshape(-1) for s in rt.slots])
    both = [torch.empty_like(mine) for _ in range(2)]
    dist.all_gather(both, mine)
    assert torch.equal(both[0], both[1]), "replicas drifted apart: gradients were not synchronised"


def test_hsdp_with_shard_degree_one_synchronises_replicas(tmp_path):
    run_distributed_test(_hsdp_shard_one, world_size=2, func_args=(str(tmp_path),))


def _ddp_vs_fsdp(tmp):
    rank = dist.get_rank()
    m0, r0 = _build(shard=False, layers=2)
    m1, r1 = _build(shard=True, layers=2)
    assert not any(s.sharded for s in r0.slots) and any(s.sharded for s in r1.slots)
    o0 = AdamWConfig(lr=1e-2).build(m0)
    o1 = AdamWConfig(lr=1e-2).build(m1)
    l0 = _steps(m0, r0, o0, n=2, seed=rank)
    l1 = _steps(m1, r1, o1, n=2, seed=rank)
    assert l0 == pytest.approx(l1, rel=1e-5)
    p0, p1 = _full_params(r0), _full_params(r1)
    _assert_same_params(p1, p0)


def test_replicated_and_sharded_runs_agree(tmp_path):
    run_distributed_test(_ddp_vs_fsdp, world_size=2, func_args=(str(tmp_path),))
