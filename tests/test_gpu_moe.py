"""Mixture-of-experts kernels (grouped GEMM, counting sort, row movement, fused router) against PyTorch fp32 references."""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


def _offsets(sizes):
    off = torch.zeros(len(sizes) + 1, dtype=torch.int32)
    off[1:] = torch.tensor(sizes).cumsum(0)
    return off.to(DEV)


SIZES = [
    [128, 256, 128],  # whole tiles
    [100, 0, 333, 7, 1],  # ragged, with an empty group
    [1000, 37, 0, 0, 513, 64, 65, 2],
]


@pytest.mark.parametrize("sizes", SIZES)
@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("K,N", [(256, 512), (320, 264)])
def test_grouped_gemm_rows(sizes, trans_b, K, N):
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.gemm import grouped_gemm

    torch.manual_seed(0)
    G, R = len(sizes), sum(sizes)
    x = torch.randn(R, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(G * N, K, device=DEV, dtype=torch.bfloat16) if trans_b else \
        torch.randn(G * K, N, device=DEV, dtype=torch.bfloat16)
    out = torch.full((R, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    grouped_gemm(x, w, _offsets(sizes), trans_b=trans_b, out=out)
    _lib.check_device_status()
    ref, r = [], 0
    for g, n in enumerate(sizes):
        wg = w.view(G, -1, w.shape[1])[g].float()
        ref.append(x[r:r + n].float() @ (wg.t() if trans_b else wg))
        r += n
    ref = torch.cat(ref)
    assert torch.isfinite(out.float()).all()  # every row of every group was written
    assert _rel_err(out, ref) < 5e-3


@pytest.mark.parametrize("sizes", SIZES)
@pytest.mark.parametrize("M,N", [(128, 256), (200, 264)])
@pytest.mark.parametrize("accumulate", [False, True])
def test_grouped_gemm_wgrad(sizes, M, N, accumulate):
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.gemm import grouped_gemm_wgrad

    torch.manual_seed(1)
    G, R = len(sizes), sum(sizes)
    a = torch.randn(R, M, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(R, N, device=DEV, dtype=torch.bfloat16)
    base = torch.randn(G * M, N, device=DEV, dtype=torch.float32)
    out = base.clone() if accumulate else torch.full((G * M, N), float("nan"), device=DEV, dtype=torch.float32)
    grouped_gemm_wgrad(a, b, _offsets(sizes), out, accumulate=accumulate)
    _lib.check_device_status()
    ref, r = [], 0
    for n in sizes:  # the reduction of a group ends mid-tile: rows of the NEXT group must not leak in
        ref.append(a[r:r + n].float().t() @ b[r:r + n].float())
        r += n
    ref = torch.cat(ref)
    if accumulate:
        ref = ref + base
    assert torch.isfinite(out).all()
    assert _rel_err(out, ref) < 5e-3
    empty = [g for g, n in enumerate(sizes) if n == 0]
    for g in empty:
        torch.testing.assert_close(out[g * M:(g + 1) * M], ref[g * M:(g + 1) * M])


@pytest.mark.parametrize("n,E,k", [(10, 4, 2), (5000, 64, 8), (70000, 128, 1)])
def test_counting_sort_matches_stable_sort(n, E, k):
    from olmo_core_b200.ops.moe import indices_and_bins

    torch.manual_seed(2)
    top = torch.randint(0, E, (n, k), device=DEV)
    indices, bin_ids, bins = indices_and_bins(top, E)
    want_ids, want_idx = torch.sort(top.reshape(-1), stable=True)
    assert torch.equal(indices.long(), want_idx) and torch.equal(bin_ids.long(), want_ids)
    assert torch.equal(bins.long(), torch.bincount(top.reshape(-1), minlength=E).cumsum(0))
    dest = indices._dest.long()
    assert torch.equal(dest[indices.long()], torch.arange(n * k, device=DEV))
    assert bins._offsets[0] == 0 and torch.equal(bins._offsets[1:], bins)


def test_gather_scatter_autograd():
    from olmo_core_b200.ops import moe as ops

    torch.manual_seed(3)
    N, d, E, k = 300, 256, 16, 4
    x = torch.randn(N, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.rand(N, k, device=DEV, dtype=torch.float32, requires_grad=True)
    top = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(N)])
    indices, bin_ids, bins = ops.indices_and_bins(top, E)
    xs = ops.gather(x, indices, bin_ids, bins, k)
    ys = xs * 1.5  # stand-in for the experts
    out = ops.scatter(ys, indices, bin_ids, w, bins, k)
    g = torch.randn_like(out)
    out.backward(g)

    xf = x.detach().float().cpu().requires_grad_(True)
    wf = w.detach().cpu().requires_grad_(True)
    idx = indices.cpu().long()
    xs_ref = xf[idx // k]
    torch.testing.assert_close(xs.float().cpu(), xs_ref.detach(), rtol=0, atol=0)
    ys_ref = xs_ref * 1.5
    contrib = ys_ref * wf.reshape(-1)[idx][:, None]
    out_ref = torch.zeros(N, d).index_add(0, idx // k, contrib)
    assert _rel_err(out.cpu(), out_ref) < 1e-2
    out_ref.backward(g.float().cpu())
    assert _rel_err(x.grad.cpu(), xf.grad) < 2e-2
    assert _rel_err(w.grad.cpu(), wf.grad) < 2e-2


@pytest.mark.parametrize("E,k", [(8, 2), (64, 8), (200, 5)])
def test_fused_router(E, k):
    from olmo_core_b200.nn.moe.router import _FusedSoftmaxTopK

    torch.manual_seed(4)
    n = 777
    logits = torch.randn(n, E, device=DEV, requires_grad=True)
    scores, weights, ids, counts = _FusedSoftmaxTopK.apply(logits, k)
    ref_logits = logits.detach().clone().requires_grad_(True)
    ref_scores = ref_logits.softmax(-1)
    ref_w, ref_ids = torch.topk(ref_scores, k, dim=-1)
    torch.testing.assert_close(scores, ref_scores.detach(), rtol=1e-5, atol=1e-6)
    assert torch.equal(ids, ref_ids)
    torch.testing.assert_close(weights, ref_w.detach(), rtol=1e-5, atol=1e-6)
    assert torch.equal(counts.long(), torch.bincount(ref_ids.reshape(-1), minlength=E))
    gs, gw = torch.randn_like(scores), torch.randn_like(weights)
    (scores * gs).sum().add((weights * gw).sum()).backward()
    (ref_scores * gs).sum().add((ref_w * gw).sum()).backward()
    torch.testing.assert_close(logits.grad, ref_logits.grad, rtol=1e-4, atol=1e-6)


def test_dropless_moe_block_matches_cpu_reference():
    """Whole MoE feed-forward (router -> sort -> gather -> grouped SwiGLU experts -> weighted scatter) on the kernels."""
    from olmo_core_b200.nn.moe import MoEConfig, MoERouterConfig, MoEType

    torch.manual_seed(5)
    d, hidden, E, k = 256, 512, 8, 2
    cfg = MoEConfig(name=MoEType.dropless, num_experts=E, hidden_size=hidden, router=MoERouterConfig(top_k=k),
                    lb_loss_weight=0.01, z_loss_weight=0.001)
    ref = cfg.build(d_model=d, init_device="cpu")
    gpu = cfg.build(d_model=d, init_device="cpu")
    gpu.load_state_dict(ref.state_dict())
    gpu = gpu.to(DEV)
    x = torch.randn(2, 96, d)
    xr = x.clone().requires_grad_(True)
    xg = x.to(DEV, torch.bfloat16).requires_grad_(True)
    ref.train(), gpu.train()
    routed = {}
    ref.router.register_forward_hook(lambda m, i, o: routed.__setitem__("ref", o[1].sort(-1).values.cpu()))
    gpu.router.register_forward_hook(lambda m, i, o: routed.__setitem__("gpu", o[1].sort(-1).values.cpu()))
    yr = ref(xr)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        yg = gpu(xg)
    # bf16 logits can flip a near-tie of the top-k; compare the tokens that both sides routed identically
    same = (routed["ref"] == routed["gpu"]).all(-1)
    assert same.float().mean() > 0.9
    assert _rel_err(yg.cpu()[same], yr[same]) < 3e-2
    g = torch.randn_like(yr)
    yr.backward(g)
    yg.backward(g.to(DEV, yg.dtype))
    assert _rel_err(xg.grad.cpu()[same], xr.grad[same]) < 6e-2
    flips = 1.0 - same.float().mean().item()
    for (name, pr), (_, pg) in zip(ref.named_parameters(), gpu.named_parameters()):
        if pr.grad is not None and pr.grad.abs().sum() > 0:
            grad = pg.grad if pg.grad is not None else getattr(pg, "main_grad", None)
            assert grad is not None, name
            assert _rel_err(grad.cpu(), pr.grad) < 6e-2 + 2.0 * flips ** 0.5, name


def test_grouped_kernels_ignore_rows_past_the_last_group():
    """Buffers sized for a capacity hold rows that belong to no group (here NaN and infinity on purpose). The grouped
    kernels must neither read them as data nor let them leak through the ragged tail of the last reduction block."""
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.gemm import grouped_gemm, grouped_gemm_wgrad

    torch.manual_seed(5)
    sizes = [70, 0, 133, 40]  # 243 rows used, a tail block of the last group that is far from full
    used, capacity, M, N = sum(sizes), 512, 128, 264
    offsets = _offsets(sizes)
    a = torch.randn(capacity, M, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(capacity, N, device=DEV, dtype=torch.bfloat16)
    a[used:] = float("nan")
    b[used:] = float("inf")
    got = torch.zeros(len(sizes) * M, N, device=DEV, dtype=torch.float32)
    grouped_gemm_wgrad(a, b, offsets, got, accumulate=False)
    ref = torch.zeros_like(got)
    grouped_gemm_wgrad(a[:used].contiguous(), b[:used].contiguous(), offsets, ref, accumulate=False)
    _lib.check_device_status()
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, ref, rtol=1e-5, atol=1e-4)
    # rows-grouped mode: outputs of the used rows do not depend on what follows them
    w = torch.randn(len(sizes) * N, M, device=DEV, dtype=torch.bfloat16)
    y = grouped_gemm(a, w, offsets, trans_b=True)
    y_ref = grouped_gemm(a[:used].contiguous(), w, offsets, trans_b=True)
    assert torch.isfinite(y[:used].float()).all() and torch.equal(y[:used], y_ref)
