"""Tensor + sequence parallelism on two gloo ranks must reproduce the single-process losses (CPU)."""

import json
from pathlib import Path

import pytest
import torch

from olmo_core_b200.testing import run_distributed_test

VOCAB, SEQ = 256, 32


def _losses(tp: bool, steps: int = 3, mx: bool = False, tie: bool = False):
    from olmo_core_b200.float8 import AOMXLinearConfig, Float8Config
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.optim import AdamWConfig
    from olmo_core_b200.train.train_module import (
        TransformerDataParallelConfig,
        TransformerTensorParallelConfig,
        TransformerTrainModule,
    )

    torch.manual_seed(0)
    model = TransformerConfig.olmo2_30M(vocab_size=VOCAB, n_layers=2, tie_word_embeddings=tie).build(init_device="cpu")
    if tie:
        assert model.lm_head.w_out.weight is model.embeddings.weight
    torch.manual_seed(0)
    model.init_weights(max_seq_len=SEQ, device=torch.device("cpu"))
    # both layouts start from these weights: the train module must not re-initialise (sliced) parameters
    model.init_weights = lambda *a, **k: None
    tm = TransformerTrainModule(
        model=model, optim=AdamWConfig(lr=1e-3, weight_decay=0.0), rank_microbatch_size=4 * SEQ, max_sequence_length=SEQ,
        max_grad_norm=1.0, device=torch.device("cpu"),
        tp_config=TransformerTensorParallelConfig(degree=2) if tp else None,
        dp_config=TransformerDataParallelConfig(name="ddp") if tp else None,
        float8_config=Float8Config(ao_mx=AOMXLinearConfig.mxfp8_cublas_rceil()) if mx else None,
    )
    if mx:
        assert any(getattr(m, "float8", None) is not None for m in tm.model.modules())
    gen = torch.Generator().manual_seed(7)
    out = []
    for _ in range(steps):
        ids = torch.randint(0, VOCAB, (4, SEQ), generator=gen)
        tm.zero_grads()
        tm.train_batch({"input_ids": ids})
        tm.optim_step()
        out.append(float(tm.latest_ce_loss))
    return out


def _tp_worker(path: str, mx: bool = False, tie: bool = False):
    import torch.distributed as dist

    losses = _losses(tp=True, mx=mx, tie=tie)
    if dist.get_rank() == 0:
        Path(path).write_text(json.dumps(losses))


def test_tensor_parallel_matches_single_process(tmp_path):
    want = _losses(tp=False)
    out = tmp_path / "tp.json"
    run_distributed_test(_tp_worker, world_size=2, func_args=(str(out),))
    got = json.loads(out.read_text())
    assert got == pytest.approx(want, rel=2e-4), (got, want)


def test_tensor_parallel_with_tied_embeddings(tmp_path):
    """The shared weight gets a partial gradient from the sequence-parallel head AND from the embedding lookup."""
    want = _losses(tp=False, tie=True)
    assert want != _losses(tp=False)
    out = tmp_path / "tp_tied.json"
    run_distributed_test(_tp_worker, world_size=2, func_args=(str(out), False, True))
    got = json.loads(out.read_text())
    assert got == pytest.approx(want, rel=2e-4), (got, want)


def test_tensor_parallel_with_mx_quantised_projections(tmp_path):
    """Block-scaled 8-bit projections under tensor parallelism: the sliced weights quantise in the same 32-element blocks
    as the whole ones, so the losses follow the single-process run up to the order of the partial sums."""
    want = _losses(tp=False, mx=True)
    plain = _losses(tp=False)
    assert want != plain  # the quantised layers are really in use
    out = tmp_path / "tp_mx.json"
    run_distributed_test(_tp_worker, world_size=2, func_args=(str(out), True))
    got = json.loads(out.read_text())
    assert got == pytest.approx(want, rel=5e-3), (got, want)


def _head_worker():
    """Sequence-parallel LM head on two ranks against the whole-sequence head: every reduction, both loss forms."""
    import copy

    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh

    from olmo_core_b200.nn.layer_norm import LayerNormConfig
    from olmo_core_b200.nn.lm_head import LMHeadConfig, LMLossImplementation

    rank, ws = dist.get_rank(), dist.get_world_size()
    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("tp",))
    B, T, d, V = 2, 16, 32, 64
    torch.manual_seed(3)
    x = torch.randn(B, T, d)
    labels = torch.randint(0, V, (B, T))
    labels[0, :3] = -100
    for impl in (LMLossImplementation.default, LMLossImplementation.fused_linear):
        torch.manual_seed(4)
        whole = LMHeadConfig(layer_norm=LayerNormConfig(), bias=False, loss_implementation=impl).build(
            d_model=d, vocab_size=V, init_device="cpu")
        with torch.no_grad():
            for p in whole.parameters():
                p.copy_(torch.randn_like(p) * 0.2 + (1.0 if p.dim() == 1 else 0.0))
        for reduction, div in (("sum", 7.0), ("mean", None), ("none", 2.0)):
            ref_head, tp_head = copy.deepcopy(whole), copy.deepcopy(whole)
            tp_head.apply_tp(mesh)
            assert all(getattr(p, "_tp_partial_grad", None) is not None for p in tp_head.parameters())
            xr = x.clone().requires_grad_(True)
            want = ref_head(xr, labels=labels, loss_reduction=reduction, z_loss_multiplier=1e-3, loss_div_factor=div)
            want.loss.sum().backward()
            xl = x.chunk(ws, dim=1)[rank].clone().requires_grad_(True)
            got = tp_head(xl, labels=labels, loss_reduction=reduction, z_loss_multiplier=1e-3, loss_div_factor=div,
                          tp_sequence_sharded=True)
            got.loss.sum().backward()
            torch.testing.assert_close(got.loss, want.loss, rtol=1e-5, atol=1e-6)
            torch.testing.assert_close(got.ce_loss, want.ce_loss, rtol=1e-5, atol=1e-6)
            torch.testing.assert_close(got.z_loss, want.z_loss, rtol=1e-5, atol=1e-7)
            torch.testing.assert_close(xl.grad, xr.grad.chunk(ws, dim=1)[rank], rtol=1e-5, atol=1e-7)
            for (name, p), q in zip(tp_head.named_parameters(), ref_head.parameters()):
                g = p.grad.clone()
                dist.all_reduce(g)  # partial sums over the sequence shards
                torch.testing.assert_close(g, q.grad, rtol=1e-4, atol=1e-6, msg=f"{impl} {reduction} {name}")
        # logits: whole-sequence output from the shards; and "keep the last n" (gathered evaluation)
        with torch.no_grad():
            tp_head = copy.deepcopy(whole)
            tp_head.apply_tp(mesh)
            xl = x.chunk(ws, dim=1)[rank]
            torch.testing.assert_close(tp_head(xl, tp_sequence_sharded=True), whole(x))
            torch.testing.assert_close(tp_head(xl, logits_to_keep=3, tp_sequence_sharded=True), whole(x, logits_to_keep=3))
            out = tp_head(xl, labels=labels, return_logits=True, loss_reduction="sum", tp_sequence_sharded=True)
            torch.testing.assert_close(out.logits, whole(x))


def test_sequence_parallel_lm_head():
    run_distributed_test(_head_worker, world_size=2)
