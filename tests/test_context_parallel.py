"""Context-parallel attention (zig-zag and contiguous layouts, Ulysses head exchange) on gloo ranks vs one device."""

import pytest
import torch

from olmo_core_b200.testing import run_distributed_test

B, T, H, HKV, D = 2, 64, 4, 2, 16


def _full(seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, D, generator=g)
    k = torch.randn(B, T, HKV, D, generator=g)
    v = torch.randn(B, T, HKV, D, generator=g)
    return q, k, v


def _ring_worker(layout: str):
    import torch.distributed as dist

    from olmo_core_b200.nn.attention.backend import TorchAttentionBackend
    from olmo_core_b200.nn.attention.ring import (
        RingAttentionLlama3LoadBalancer,
        RingAttentionZigZagLoadBalancer,
        RingContextParallelStyle,
    )
    from olmo_core_b200.ops.attention import attention_reference
    from olmo_core_b200.parallel.context import ring_attention

    rank, ws = dist.get_rank(), dist.get_world_size()
    q, k, v = _full()
    want = attention_reference(q, k, v, causal=True)
    if layout == "zig_zag":
        lb, style = RingAttentionZigZagLoadBalancer(cp_rank=rank, cp_world_size=ws), RingContextParallelStyle.zig_zag()
    else:
        lb, style = RingAttentionLlama3LoadBalancer(cp_rank=rank, cp_world_size=ws), RingContextParallelStyle.llama3()
    ql, kl, vl, wl = lb.batch_shard(inputs=[q, k, v, want], seq_dims=[1, 1, 1, 1])
    ql, kl, vl = (t.clone().requires_grad_(True) for t in (ql, kl, vl))
    backend = TorchAttentionBackend(head_dim=D, n_heads=H, n_kv_heads=HKV)
    out = ring_attention(backend, ql, kl, vl, group=dist.group.WORLD, style=style)
    torch.testing.assert_close(out, wl, rtol=1e-4, atol=1e-5)
    # gradients: d(sum of all outputs)/dk on the owners must equal the single-device gradient shard
    out.sum().backward()
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    attention_reference(qf, kf, vf, causal=True).sum().backward()
    (kg,) = lb.batch_shard(inputs=[kf.grad], seq_dims=[1])
    torch.testing.assert_close(kl.grad, kg, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("layout", ["zig_zag", "llama3"])
def test_ring_attention_matches_single_device(layout):
    run_distributed_test(_ring_worker, world_size=2, func_args=(layout,))


def _ulysses_worker():
    import torch.distributed as dist

    from olmo_core_b200.distributed.parallel.context_parallel import all_to_all_cp2hp, all_to_all_single_hp2cp
    from olmo_core_b200.ops.attention import attention_reference

    rank, ws = dist.get_rank(), dist.get_world_size()
    q, k, v = _full(1)
    want = attention_reference(q, k, v, causal=True)
    sl = slice(rank * T // ws, (rank + 1) * T // ws)
    qh, kh, vh = all_to_all_cp2hp([q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous()], dist.group.WORLD)
    assert qh.shape == (B, T, H // ws, D)  # full sequence, a slice of the heads
    out = all_to_all_single_hp2cp(attention_reference(qh, kh, vh, causal=True), dist.group.WORLD)
    torch.testing.assert_close(out, want[:, sl], rtol=1e-4, atol=1e-5)


def test_ulysses_head_exchange_matches_single_device():
    run_distributed_test(_ulysses_worker, world_size=2)


# -- packed documents under ring context parallelism ------------------------------------------------------------------
def _ring_docs_worker(layout: str):
    import torch.distributed as dist

    from olmo_core_b200.nn.attention.backend import TorchAttentionBackend
    from olmo_core_b200.nn.attention.ring import (
        RingAttentionLlama3LoadBalancer,
        RingAttentionZigZagLoadBalancer,
        RingContextParallelStyle,
    )
    from olmo_core_b200.ops.attention import attention_reference
    from olmo_core_b200.parallel.context import ring_attention

    rank, ws = dist.get_rank(), dist.get_world_size()
    q, k, v = _full(2)
    # documents of uneven length that straddle the shard boundaries, counted over the flattened [B * T] sequence
    cu = torch.tensor([0, 10, 37, 64, 64 + 5, 64 + 50, 128], dtype=torch.int32)
    want = attention_reference(q, k, v, causal=True, cu_seqlens=cu)
    if layout == "zig_zag":
        lb, style = RingAttentionZigZagLoadBalancer(cp_rank=rank, cp_world_size=ws), RingContextParallelStyle.zig_zag()
    else:
        lb, style = RingAttentionLlama3LoadBalancer(cp_rank=rank, cp_world_size=ws), RingContextParallelStyle.llama3()
    ql, kl, vl, wl = lb.batch_shard(inputs=[q, k, v, want], seq_dims=[1, 1, 1, 1])
    ql, kl, vl = (t.clone().requires_grad_(True) for t in (ql, kl, vl))
    backend = TorchAttentionBackend(head_dim=D, n_heads=H, n_kv_heads=HKV)
    out = ring_attention(backend, ql, kl, vl, group=dist.group.WORLD, style=style, cu_doc_lens=cu)
    torch.testing.assert_close(out, wl, rtol=1e-4, atol=1e-5)
    out.sum().backward()
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    attention_reference(qf, kf, vf, causal=True, cu_seqlens=cu).sum().backward()
    (vg,) = lb.batch_shard(inputs=[vf.grad], seq_dims=[1])
    torch.testing.assert_close(vl.grad, vg, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("layout", ["zig_zag", "llama3"])
def test_ring_attention_with_packed_documents(layout):
    run_distributed_test(_ring_docs_worker, world_size=2, func_args=(layout,))


def _model_docs_worker(layout: str):
    """A whole model: position-sharded tokens + the documents' boundaries give the unsharded model's loss and gradients
    (attention masks AND rotary positions restart at every document)."""
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh

    from olmo_core_b200.nn.attention.ring import RingContextParallelStyle
    from olmo_core_b200.nn.transformer import TransformerConfig

    cfg = TransformerConfig.olmo2_30M(vocab_size=256, n_layers=2)
    torch.manual_seed(3)
    ref_model = cfg.build(init_device="cpu")
    ref_model.init_weights(device=torch.device("cpu"), max_seq_len=64)
    model = cfg.build(init_device="cpu")
    model.init_weights(device=torch.device("cpu"), max_seq_len=64)
    model.load_state_dict(ref_model.state_dict())
    mesh = init_device_mesh("cpu", (dist.get_world_size(),), mesh_dim_names=("cp",))
    model.apply_cp(mesh, ring=getattr(RingContextParallelStyle, layout)())
    ids = torch.randint(0, 256, (1, 64), generator=torch.Generator().manual_seed(4))
    labels = torch.roll(ids, -1, 1)
    doc_lens = torch.tensor([[9, 30, 25]])
    kw = dict(doc_lens=doc_lens, max_doc_lens=[30])
    want = ref_model(ids, labels=labels, loss_reduction="sum", **kw)
    plain = ref_model(ids, labels=labels, loss_reduction="sum")
    assert abs(float(want.loss) - float(plain.loss)) > 1e-3  # the documents do change the result
    got = model(ids, labels=labels, loss_reduction="sum", **kw)
    total = got.loss.detach().clone()
    dist.all_reduce(total)
    torch.testing.assert_close(total, want.loss.detach(), rtol=1e-4, atol=1e-4)
    got.loss.backward()
    want.loss.backward()
    for name in ("blocks.0.attention.w_k.weight", "blocks.1.feed_forward.w2.weight", "embeddings.weight"):
        g = dict(model.named_parameters())[name].grad.clone()
        dist.all_reduce(g)
        torch.testing.assert_close(g, dict(ref_model.named_parameters())[name].grad, rtol=1e-3, atol=1e-5, msg=name)


@pytest.mark.parametrize("layout", ["zig_zag", "llama3"])
def test_transformer_with_packed_documents_under_context_parallelism(layout):
    run_distributed_test(_model_docs_worker, world_size=2, func_args=(layout,))


def _gdn_ulysses_worker():
    """Gated DeltaNet with its heads split over the ranks (Ulysses) against the same layer on the whole sequence."""
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh

    from olmo_core_b200.nn.attention.recurrent import GatedDeltaNet
    from olmo_core_b200.nn.attention.ring import UlyssesContextParallelStyle

    rank, ws = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    layer = GatedDeltaNet(d_model=64, n_heads=4, n_v_heads=8, head_dim=16, init_device="cpu")
    layer.init_weights(std=0.05)
    ref = GatedDeltaNet(d_model=64, n_heads=4, n_v_heads=8, head_dim=16, init_device="cpu")
    ref.load_state_dict(layer.state_dict())
    x = torch.randn(2, 32, 64, generator=torch.Generator().manual_seed(1))
    want = ref(x)
    want.pow(2).sum().backward()
    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("cp",))
    layer.apply_cp(mesh, uly=UlyssesContextParallelStyle())
    sl = slice(rank * 32 // ws, (rank + 1) * 32 // ws)
    got = layer(x[:, sl].contiguous())
    torch.testing.assert_close(got, want[:, sl], rtol=1e-4, atol=1e-5)
    got.pow(2).sum().backward()
    for (n, p), q in zip(layer.named_parameters(), ref.parameters()):
        g = p.grad.clone()
        dist.all_reduce(g)  # every rank saw its tokens (projections) or its heads (decay, convolutions) only
        torch.testing.assert_close(g, q.grad, rtol=1e-3, atol=1e-5, msg=n)
    with pytest.raises(NotImplementedError):
        GatedDeltaNet(d_model=64, n_heads=4, head_dim=16, init_device="cpu").apply_cp(mesh, ring=object())


def test_gated_delta_net_under_ulysses_context_parallelism():
    run_distributed_test(_gdn_ulysses_worker, world_size=2)
