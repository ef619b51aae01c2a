"""
Multi-GPU paths (2 ranks, NCCL): the optimizer step fused with its collectives over peer memory must give the same
parameters as the NCCL reduce-scatter / all-gather path, with plain peer loads and with NVSwitch multimem.
"""

import os

import pytest
import torch

from olmo_core_b200.testing import requires_multi_gpu, run_distributed_test

VOCAB, SEQ = 512, 128


def _train(out_path: str, symmetric: str, multimem: str, steps: int = 3, streamed: str = "0", early: str = "1"):
    os.environ["OLMO_CORE_B200_SYMMETRIC"] = symmetric
    os.environ["OLMO_CORE_B200_FSDP_EARLY_REDUCE"] = early
    os.environ["OLMO_CORE_B200_MULTIMEM"] = multimem
    os.environ["OLMO_CORE_B200_FSDP_STREAMED"] = streamed
    import torch.distributed as dist

    from olmo_core_b200.config import DType
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.optim import AdamWConfig
    from olmo_core_b200.train.train_module import TransformerDataParallelConfig, TransformerTrainModule

    rank = dist.get_rank()
    device = torch.device("cuda", rank)
    torch.manual_seed(0)
    model = TransformerConfig.olmo2_30M(vocab_size=VOCAB, n_layers=2).build(init_device="meta")
    tm = TransformerTrainModule(
        model=model, optim=AdamWConfig(lr=1e-3, weight_decay=0.1), rank_microbatch_size=2 * SEQ, max_sequence_length=SEQ,
        max_grad_norm=1.0, device=device,
        dp_config=TransformerDataParallelConfig(name="fsdp", param_dtype=DType.bfloat16, reduce_dtype=DType.float32),
    )
    rt = tm.runtime
    if streamed == "1":
        assert rt.streamed and (rt._sym_ring_grad is not None) == (symmetric == "1")
        norms = []
        gen = torch.Generator().manual_seed(100 + rank)
        for _ in range(steps):
            ids = torch.randint(0, VOCAB, (4, SEQ), generator=gen)
            tm.zero_grads()
            tm.train_batch({"input_ids": ids})
            tm.optim_step()
            norms.append(float(rt.grad_norm_sq().sqrt()))
        torch.cuda.synchronize()
        from olmo_core_b200.ops import _lib

        _lib.check_device_status(device)
        full = {}
        for s in rt.slots:
            if not s.aware:
                continue
            local = s.param.data.contiguous()
            parts = [torch.empty_like(local) for _ in range(dist.get_world_size())]
            dist.all_gather(parts, local)
            full[s.name] = torch.cat(parts, 0)[: s.full_shape[0]].to(torch.bfloat16).float().cpu().reshape(-1)
        if rank == 0:
            torch.save({"params": full, "norms": norms}, out_path)
        return
    assert rt.symmetric == (symmetric == "1"), (rt.symmetric, symmetric)
    if symmetric == "1" and multimem == "1" and rt._sym_grad.multicast_ptr is None:
        if rank == 0:
            torch.save({"skipped": "no multicast support"}, out_path)
        return
    gen = torch.Generator().manual_seed(100 + rank)
    norms = []
    for _ in range(steps):
        ids = torch.randint(0, VOCAB, (4, SEQ), generator=gen)
        tm.zero_grads()
        tm.train_batch({"input_ids": ids})
        tm.optim_step()
        norms.append(float(rt.grad_norm_sq().sqrt()))
    torch.cuda.synchronize()
    if early == "1" and symmetric == "1":
        assert rt.early_reduce_blocks == 2 * steps, rt.early_reduce_blocks  # both blocks, every step
    # every rank's resident bf16 copy must hold ALL parameters, including the rows owned by the peer
    full = {s.name: rt.lowp[s.full_offset: s.full_offset + s.full_numel].float().cpu() for s in rt.slots if s.aware}
    gathered = [None] * dist.get_world_size()
    dist.all_gather_object(gathered, {k: v.sum().item() for k, v in full.items()})
    assert gathered[0] == gathered[1], "ranks disagree about the gathered parameters"
    if rank == 0:
        torch.save({"params": full, "norms": norms}, out_path)


def _run(tmp_path, name: str, symmetric: str, multimem: str, streamed: str = "0", early: str = "1"):
    out = str(tmp_path / f"{name}.pt")
    run_distributed_test(_train, world_size=2, backend="cuda:nccl,cpu:gloo",
                         func_args=(out, symmetric, multimem, 3, streamed, early))
    return torch.load(out, weights_only=False)


@pytest.mark.gpu
@requires_multi_gpu
@pytest.mark.parametrize("symmetric", ["0", "1"])
def test_streamed_blocks_match_resident_parameters(tmp_path, symmetric):
    """Per-block gather / gradient reduction (NCCL, and the peer-memory kernels) against the resident NCCL path."""
    ref = _run(tmp_path, "nccl", "0", "0")
    got = _run(tmp_path, f"streamed{symmetric}", symmetric, "0", streamed="1")
    for a, b in zip(ref["norms"], got["norms"]):
        assert a == pytest.approx(b, rel=2e-3)
    for name, want in ref["params"].items():
        # both sides are bf16 roundings of fp32 masters that differ in the last bits: allow one bf16 ulp
        torch.testing.assert_close(got["params"][name], want, rtol=1e-2, atol=1e-2, msg=name)


@pytest.mark.gpu
@requires_multi_gpu
@pytest.mark.parametrize("multimem", ["0", "1"])
def test_fused_optimizer_collectives_match_nccl(tmp_path, multimem):
    ref = _run(tmp_path, "nccl", "0", "0")
    got = _run(tmp_path, f"fused{multimem}", "1", multimem)
    if "skipped" in got:
        pytest.skip(got["skipped"])
    for a, b in zip(ref["norms"], got["norms"]):
        # two bf16 training runs whose gradient sums are formed in different orders: agreement to bf16-level noise
        assert a == pytest.approx(b, rel=1e-3)
    for name, want in ref["params"].items():
        torch.testing.assert_close(got["params"][name], want, rtol=0, atol=1e-2, msg=name)


@pytest.mark.gpu
@requires_multi_gpu
def test_gradient_reduction_behind_the_last_backward_matches_the_one_shot_reduction(tmp_path):
    """Resident parameters: blocks reduced on a side stream while the last micro-batch's backward still runs give the
    same gradients as the reduction after the backward (the squared norm is summed in another order, so the clipping
    factor may differ in its last bits)."""
    ref = _run(tmp_path, "oneshot", "1", "0", early="0")
    got = _run(tmp_path, "early", "1", "0", early="1")
    assert ref["norms"][0] == pytest.approx(got["norms"][0], rel=1e-6)  # first step: same gradients, other summing order
    for a, b in zip(ref["norms"], got["norms"]):
        assert a == pytest.approx(b, rel=1e-3)  # later steps inherit bf16 rounding flips from the last bits of the clip factor
    for name, want in ref["params"].items():
        torch.testing.assert_close(got["params"][name], want, rtol=0, atol=1e-2, msg=name)


def _tp_fused_worker():
    """All-gather -> GEMM and GEMM -> reduce-scatter kernels against NCCL collectives around a plain GEMM, with grads."""
    import torch.distributed as dist

    from olmo_core_b200.ops import _lib
    from olmo_core_b200.parallel.tp_fused import fused_tp_available, gather_linear, linear_reduce_scatter

    rank, ws = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", rank)
    group = dist.group.WORLD
    m, K, N = 256, 320, 384  # rows per rank, model width, width of this rank's weight slice
    gen = torch.Generator().manual_seed(7)
    x_all = torch.randn(ws, m, K, generator=gen)
    w_cols = torch.randn(ws, N, K, generator=gen) * 0.05  # column-parallel slices (one per rank)
    w_rows = torch.randn(ws, K, N, generator=gen) * 0.05  # row-parallel slices: rank r holds [K, N_r]
    x = x_all[rank].to(dev, torch.bfloat16).requires_grad_(True)
    assert fused_tp_available(x, group, m)

    # --- gather_linear: y = [x_0; x_1; ...] @ W_r^T ---------------------------------------------------------
    w1 = w_cols[rank].to(dev, torch.bfloat16).requires_grad_(True)
    y = gather_linear(x, w1, group, "t1")
    ref_x = x_all.to(torch.bfloat16).float().reshape(ws * m, K)
    ref_y = ref_x @ w_cols[rank].to(torch.bfloat16).float().t()
    torch.testing.assert_close(y.float().cpu(), ref_y, rtol=2e-2, atol=2e-2)
    g = torch.randn(ws * m, N, generator=torch.Generator().manual_seed(20 + rank))
    y.backward(g.to(dev, torch.bfloat16))
    # dx_r = sum over ranks q of (g_q @ W_q)[rows of r]
    gb = g.to(torch.bfloat16).float()
    partial = (gb @ w_cols[rank].to(torch.bfloat16).float()).to(dev)
    dist.all_reduce(partial)
    torch.testing.assert_close(x.grad.float(), partial[rank * m:(rank + 1) * m], rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(w1.grad.float().cpu(), gb.t() @ ref_x, rtol=3e-2, atol=6e-2)

    # --- linear_reduce_scatter: y_r = sum_q (h_q @ V_q^T)[rows of r] ---------------------------------------
    h = torch.randn(ws * m, N, generator=torch.Generator().manual_seed(40 + rank))
    hq = h.to(dev, torch.bfloat16).requires_grad_(True)
    v = w_rows[rank].to(dev, torch.bfloat16).requires_grad_(True)  # [K, N]: y = h @ v^T
    out = linear_reduce_scatter(hq, v, group, "t2")
    full = (h.to(torch.bfloat16).float() @ w_rows[rank].to(torch.bfloat16).float().t()).to(dev)
    dist.all_reduce(full)
    torch.testing.assert_close(out.float(), full[rank * m:(rank + 1) * m], rtol=3e-2, atol=3e-2)
    go = torch.randn(m, K, generator=torch.Generator().manual_seed(60 + rank)).to(dev, torch.bfloat16)
    out.backward(go)
    go_all = [torch.empty_like(go) for _ in range(ws)]
    dist.all_gather(go_all, go)
    go_full = torch.cat(go_all).float()
    torch.testing.assert_close(hq.grad.float(), go_full @ v.detach().float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(v.grad.float(), go_full.t() @ hq.detach().float(), rtol=3e-2, atol=6e-2)
    _lib.check_device_status()


@pytest.mark.gpu
@requires_multi_gpu
def test_tensor_parallel_fused_collective_gemms():
    run_distributed_test(_tp_fused_worker, world_size=2, backend="cuda:nccl,cpu:gloo")


def _tp_multi_worker():
    """Several projections of one sharded input: one published shard, one reduction of the input gradient."""
    import torch.distributed as dist

    from olmo_core_b200.ops import _lib
    from olmo_core_b200.parallel.tp_fused import gather_linear_multi

    rank, ws = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", rank)
    m, K = 128, 256
    widths = (384, 128, 128)
    gen = torch.Generator().manual_seed(11)
    x_all = torch.randn(ws, m, K, generator=gen)
    w_all = [torch.randn(ws, n, K, generator=gen) * 0.05 for n in widths]
    x = x_all[rank].to(dev, torch.bfloat16).requires_grad_(True)
    weights = [w[rank].to(dev, torch.bfloat16).requires_grad_(True) for w in w_all]
    ys = gather_linear_multi(x, weights, dist.group.WORLD, "multi")
    ref_x = x_all.to(torch.bfloat16).float().reshape(ws * m, K)
    gs = [torch.randn(ws * m, n, generator=torch.Generator().manual_seed(30 + rank + i)) for i, n in enumerate(widths)]
    for y, w, n in zip(ys, w_all, widths):
        torch.testing.assert_close(y.float().cpu(), ref_x @ w[rank].to(torch.bfloat16).float().t(), rtol=2e-2, atol=2e-2)
    torch.autograd.backward(ys, [g.to(dev, torch.bfloat16) for g in gs])
    partial = sum(g.to(torch.bfloat16).float() @ w[rank].to(torch.bfloat16).float() for g, w in zip(gs, w_all)).to(dev)
    dist.all_reduce(partial)
    torch.testing.assert_close(x.grad.float(), partial[rank * m:(rank + 1) * m], rtol=3e-2, atol=5e-2)
    for wt, g in zip(weights, gs):
        torch.testing.assert_close(wt.grad.float().cpu(), g.to(torch.bfloat16).float().t() @ ref_x, rtol=3e-2, atol=8e-2)
    _lib.check_device_status()


@pytest.mark.gpu
@requires_multi_gpu
def test_tensor_parallel_shared_input_projections():
    run_distributed_test(_tp_multi_worker, world_size=2, backend="cuda:nccl,cpu:gloo")


def _tp_model_worker():
    """A tensor-parallel model (attention and MLP projections with the collectives inside their GEMMs) against the same
    model on one GPU: losses of three optimizer steps."""
    import torch.distributed as dist

    from olmo_core_b200.config import DType
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.optim import AdamWConfig
    from olmo_core_b200.parallel import tp_fused
    from olmo_core_b200.train.train_module import (
        TransformerDataParallelConfig,
        TransformerTensorParallelConfig,
        TransformerTrainModule,
    )

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    seq, vocab = 256, 512
    calls = {"n": 0}
    real = tp_fused._ag_gemm_multi

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    tp_fused._ag_gemm_multi = counting

    def losses(tp: bool):
        torch.manual_seed(0)
        model = TransformerConfig.olmo2_30M(vocab_size=vocab, n_layers=2).build(init_device="cpu")
        torch.manual_seed(0)
        model.init_weights(max_seq_len=seq, device=torch.device("cpu"))
        model.init_weights = lambda *a, **k: None
        model.to(dev)
        tm = TransformerTrainModule(
            model=model, optim=AdamWConfig(lr=1e-3, weight_decay=0.0), rank_microbatch_size=2 * seq, max_sequence_length=seq,
            max_grad_norm=1.0, device=dev,
            tp_config=TransformerTensorParallelConfig(degree=2) if tp else None,
            dp_config=TransformerDataParallelConfig(name="ddp", param_dtype=DType.bfloat16, reduce_dtype=DType.float32) if tp else None,
        )
        gen = torch.Generator().manual_seed(7)
        out = []
        for _ in range(3):
            ids = torch.randint(0, vocab, (2, seq), generator=gen)
            tm.zero_grads()
            tm.train_batch({"input_ids": ids})
            tm.optim_step()
            out.append(float(tm.latest_ce_loss))
        return out

    got = losses(True)
    assert calls["n"] >= 2 * 2 * 3, "the fused gather GEMMs did not run"  # (attention + MLP) x layers x steps, forward
    tp_fused._ag_gemm_multi = real
    # the same model without any parallelism: every rank trains its own copy on the same batches
    want = losses(False)
    assert got == pytest.approx(want, rel=2e-2), (got, want)


@pytest.mark.gpu
@requires_multi_gpu
def test_tensor_parallel_model_with_fused_projections():
    run_distributed_test(_tp_model_worker, world_size=2, backend="cuda:nccl,cpu:gloo")


def _cp_in_kernel_worker(zig_zag: bool, window, mode: str, docs: bool = False):
    """Context-parallel attention with K / V exchanged over peer memory (pushed once, or read tile by tile from the
    owning GPU inside the attention kernels), against attention over the whole sequence."""
    import torch.distributed as dist

    os.environ["OLMO_CORE_B200_CP_KV"] = mode

    from olmo_core_b200.nn.attention.ring import RingAttentionLoadBalancerType
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.attention import attention, attention_reference
    from olmo_core_b200.parallel import context

    rank, cp = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", rank)
    B, T, H, Hkv = 2, 2048, 4, 2
    gen = torch.Generator().manual_seed(11)
    q, k, v, dout = (torch.randn(B, T, h, 128, generator=gen).to(dev, torch.bfloat16) for h in (H, Hkv, Hkv, H))
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    cu = None
    if docs:  # packed documents across the shard boundaries, counted over the flattened [B * T] sequence
        cu = torch.tensor([0, 300, 1100, 1900, T, T + 777, T + 1500, 2 * T], dtype=torch.int32, device=dev)
    ref = attention_reference(qf, kf, vf, causal=True, window_size=window, cu_seqlens=cu)
    ref.backward(dout.float())

    class Style:
        load_balancer = RingAttentionLoadBalancerType.zig_zag if zig_zag else RingAttentionLoadBalancerType.llama3

    class Backend:
        scale = None

        def _local(self, q_, k_, v_, causal=True):
            return attention(q_, k_, v_, causal=causal, window_size=window)

    Backend.window = window
    rows = torch.cat([torch.arange(a, b, device=dev) for a, b in context.local_position_ranges(T // cp, rank, cp, zig_zag)])
    for _ in range(3):  # several calls: the two slots of the exchange buffer are reused
        ql, kl, vl = (t[:, rows].contiguous().requires_grad_(True) for t in (q, k, v))
        assert context._sharded_kernels_usable(ql, kl, dist.group.WORLD, zig_zag)
        out = context.ring_attention(Backend(), ql, kl, vl, group=dist.group.WORLD, style=Style(), cu_doc_lens=cu)
        out.backward(dout[:, rows].contiguous())
        torch.cuda.synchronize()
        _lib.check_device_status(dev)
        torch.testing.assert_close(out.float(), ref[:, rows], rtol=2e-2, atol=2e-2)
        for got, want in ((ql.grad, qf.grad), (kl.grad, kf.grad), (vl.grad, vf.grad)):
            want = want[:, rows]
            torch.testing.assert_close(got.float(), want, rtol=3e-2, atol=3e-2 * float(want.abs().max()) / 2 + 3e-2)


@pytest.mark.gpu
@requires_multi_gpu
@pytest.mark.parametrize("zig_zag,window,mode,docs", [
    (False, None, "push", False), (True, None, "push", False), (False, 300, "push", False), (True, None, "direct", False),
    (False, 300, "direct", False), (True, None, "push", True), (False, 300, "push", True),
])
def test_context_parallel_attention_over_peer_memory(zig_zag, window, mode, docs):
    run_distributed_test(_cp_in_kernel_worker, world_size=2, backend="cuda:nccl,cpu:gloo",
                         func_args=(zig_zag, window, mode, docs))


def _ulysses_peer_worker():
    """Sequence <-> head exchange by the peer-memory kernel against the all-to-all path, values and gradients."""
    import torch.distributed as dist

    from olmo_core_b200.distributed.parallel.context_parallel import all_to_all_cp2hp, all_to_all_single_hp2cp
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.parallel import ulysses

    rank, cp = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", rank)
    B, t, D = 2, 1500, 128  # more tokens than one segment piece
    gen = torch.Generator().manual_seed(5 + rank)
    results = {}
    for flag in ("1", "0"):
        os.environ["OLMO_CORE_B200_ULYSSES_PEER"] = flag
        q = torch.randn(B, t, 4 * cp, D, generator=torch.Generator().manual_seed(5 + rank)).to(dev, torch.bfloat16).requires_grad_(True)
        k = torch.randn(B, t, 2 * cp, D, generator=torch.Generator().manual_seed(50 + rank)).to(dev, torch.bfloat16).requires_grad_(True)
        assert ulysses.peer_exchange_usable(q, dist.group.WORLD) == (flag == "1")
        for _ in range(3):  # both halves of the receive buffer get reused
            qh, kh = all_to_all_cp2hp([q, k], dist.group.WORLD)
            assert qh.shape == (B, cp * t, 4, D) and kh.shape == (B, cp * t, 2, D)
            back = all_to_all_single_hp2cp(qh * 2, dist.group.WORLD)
            assert back.shape == q.shape
        q.grad = k.grad = None
        w = torch.randn(back.shape, generator=torch.Generator().manual_seed(9)).to(dev, torch.bfloat16)
        ((back * w).float().sum() + (kh.float() ** 2).sum()).backward()
        torch.cuda.synchronize()
        _lib.check_device_status(dev)
        results[flag] = [t_.detach().float().cpu() for t_ in (qh, kh, back, q.grad, k.grad)]
    del gen
    for a, b in zip(results["1"], results["0"]):
        torch.testing.assert_close(a, b, rtol=0, atol=0)
    torch.testing.assert_close(results["1"][2], 2 * q.detach().float().cpu(), rtol=0, atol=0)


@pytest.mark.gpu
@requires_multi_gpu
def test_ulysses_exchange_over_peer_memory():
    run_distributed_test(_ulysses_peer_worker, world_size=2, backend="cuda:nccl,cpu:gloo")


def _model_cp_worker(style_name: str):
    """A small transformer with its sequence split over two GPUs against the same model on the whole sequence."""
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh

    from olmo_core_b200.config import DType
    from olmo_core_b200.nn.attention.ring import RingContextParallelStyle, UlyssesContextParallelStyle
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.ops import _lib

    rank, cp = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    cfg = TransformerConfig.llama_like(vocab_size=512, d_model=512, n_layers=2, n_heads=4, dtype=DType.bfloat16)
    torch.manual_seed(3)
    ref_model = cfg.build(init_device="cpu")
    ref_model.init_weights(device=dev, max_seq_len=1024)
    model = cfg.build(init_device="cpu")
    model.init_weights(device=dev, max_seq_len=1024)
    model.load_state_dict(ref_model.state_dict())
    mesh = init_device_mesh("cuda", (cp,), mesh_dim_names=("cp",))
    if style_name == "ulysses":
        model.apply_cp(mesh, uly=UlyssesContextParallelStyle())
    else:
        model.apply_cp(mesh, ring=getattr(RingContextParallelStyle, style_name)())
    ids = torch.randint(0, 512, (2, 1024), generator=torch.Generator().manual_seed(4)).to(dev)
    labels = torch.roll(ids, -1, 1)
    want = ref_model(ids, labels=labels, loss_reduction="sum")
    got = model(ids, labels=labels, loss_reduction="sum")
    total = got.loss.detach().float().clone()
    dist.all_reduce(total)
    torch.cuda.synchronize()
    _lib.check_device_status(dev)
    torch.testing.assert_close(total, want.loss.detach().float(), rtol=2e-2, atol=2e-2 * float(want.loss.abs()))
    got.loss.backward()
    want.loss.backward()
    g = model.blocks["0"].attention.w_k.weight.grad.float().clone()
    dist.all_reduce(g)
    w = ref_model.blocks["0"].attention.w_k.weight.grad.float()
    torch.testing.assert_close(g, w, rtol=5e-2, atol=5e-2 * float(w.abs().max()))
    _lib.check_device_status(dev)


@pytest.mark.gpu
@requires_multi_gpu
@pytest.mark.parametrize("style_name", ["zig_zag", "llama3", "ulysses"])
def test_transformer_under_context_parallelism(style_name):
    run_distributed_test(_model_cp_worker, world_size=2, backend="cuda:nccl,cpu:gloo", func_args=(style_name,))
