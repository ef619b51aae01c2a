"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same ops."""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


@pytest.mark.parametrize(
    "M,N,K",
    [(128, 256, 64), (256, 512, 256), (384, 768, 4096), (1000, 520, 264), (4096, 4096, 4096), (64, 64, 64), (8, 100352 // 8, 128)],
)
def test_gemm_nt(M, N, K):
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.gemm import gemm

    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    out = gemm(a, b, trans_b=True)
    _lib.check_device_status()
    ref = a.float() @ b.float().t()
    assert _rel_err(out, ref) < 5e-3


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (512, 768, 320), (1000, 520, 264), (2048, 4096, 1024)])
def test_gemm_nn_and_tn(M, N, K):
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.gemm import gemm

    torch.manual_seed(1)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    out = gemm(a, b, trans_b=False)
    ref = a.float() @ b.float()
    assert _rel_err(out, ref) < 5e-3
    # TN: a stored [K, M]
    at = torch.randn(K, M, device=DEV, dtype=torch.bfloat16)
    out32 = gemm(at, b, trans_a=True, trans_b=False, out_dtype=torch.float32)
    ref = at.float().t() @ b.float()
    assert _rel_err(out32, ref) < 1e-3
    # accumulate into fp32
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    expect = acc + ref
    gemm(at, b, trans_a=True, trans_b=False, out=acc, accumulate=True)
    assert _rel_err(acc, expect) < 1e-3
    # TN with K-major B (a^T @ b2^T)
    b2 = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    out = gemm(at, b2, trans_a=True, trans_b=True)
    assert _rel_err(out, at.float().t() @ b2.float().t()) < 5e-3
    _lib.check_device_status()


def test_gemm_strided_views():
    from olmo_core_b200.ops.gemm import gemm

    torch.manual_seed(2)
    big = torch.randn(512, 1024, device=DEV, dtype=torch.bfloat16)
    a = big[:, 256:768]  # row stride 1024, 512 columns
    w = torch.randn(384, 512, device=DEV, dtype=torch.bfloat16)
    outbuf = torch.zeros(512, 1024, device=DEV, dtype=torch.bfloat16)
    gemm(a, w, trans_b=True, out=outbuf[:, 128:512])
    ref = a.float() @ w.float().t()
    assert _rel_err(outbuf[:, 128:512], ref) < 5e-3
    assert outbuf[:, :128].abs().max().item() == 0 and outbuf[:, 512:].abs().max().item() == 0


def test_linear_autograd_matches_reference():
    from olmo_core_b200.ops.gemm import linear

    torch.manual_seed(3)
    x = torch.randn(4, 96, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(512, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 5e-3
    assert _rel_err(x.grad, xr.grad) < 5e-3
    assert _rel_err(w.grad, wr.grad) < 5e-3


def test_linear_main_grad_accumulation():
    from olmo_core_b200.ops.gemm import linear

    torch.manual_seed(4)
    x = torch.randn(300, 128, device=DEV, dtype=torch.bfloat16)
    w = torch.nn.Parameter(torch.randn(256, 128, device=DEV, dtype=torch.float32))
    w._lowp = w.detach().to(torch.bfloat16)
    w.main_grad = torch.zeros_like(w)
    for _ in range(2):
        y = linear(x, w)
        y.float().sum().backward()
    assert w.grad is None
    ref = 2 * (torch.ones(300, 256, device=DEV).t() @ x.float())
    assert _rel_err(w.main_grad, ref) < 1e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,cols,group", [(64, 4096, 4096), (37, 1024, 128), (300, 512, 512), (5, 8192, 8192)])
def test_rms_norm(dtype, rows, cols, group):
    from olmo_core_b200.ops.elementwise import rms_norm, rms_norm_reference

    torch.manual_seed(5)
    x = torch.randn(rows, cols, device=DEV, dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(group, device=DEV)).to(dtype).requires_grad_(True)
    res = torch.randn(rows, cols, device=DEV, dtype=dtype, requires_grad=True)
    y = rms_norm(x, w, 1e-6, residual=res, group=group)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, rr = (t.detach().float().requires_grad_(True) for t in (x, w, res))
    yr = rms_norm_reference(xr, wr, 1e-6, rr, group)
    yr.backward(g.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert _rel_err(y, yr) < tol
    assert _rel_err(x.grad, xr.grad) < tol
    assert _rel_err(res.grad, rr.grad) < tol
    assert _rel_err(w.grad, wr.grad) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("norm_mode", [0, 1, 2])
@pytest.mark.parametrize("B,S,H,hd", [(2, 64, 32, 128), (1, 33, 8, 64), (2, 16, 40, 128)])
def test_norm_rope(dtype, norm_mode, B, S, H, hd):
    from olmo_core_b200.ops.elementwise import norm_rope, norm_rope_reference

    torch.manual_seed(6)
    x = torch.randn(B, S, H * hd, device=DEV, dtype=dtype, requires_grad=True)
    wn = H * hd if norm_mode == 1 else hd
    w = (1 + 0.1 * torch.randn(wn, device=DEV)).to(dtype).requires_grad_(True) if norm_mode else None
    inv = 500000.0 ** (-torch.arange(0, hd, 2, device=DEV).float() / hd)
    fr = torch.outer(torch.arange(128, device=DEV).float(), inv)
    pos = torch.cat([fr, fr], -1)
    sin, cos = pos.sin(), pos.cos()
    y = norm_rope(x, w, sin, cos, H, 1e-6, norm_mode, None, 3)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True) if norm_mode else None
    yr = norm_rope_reference(xr, wr, sin, cos, H, 1e-6, norm_mode, None, 3)
    yr.backward(g.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert _rel_err(y, yr) < tol
    assert _rel_err(x.grad, xr.grad) < tol
    if norm_mode:
        assert _rel_err(w.grad, wr.grad) < tol
    # explicit position ids
    ids = torch.randint(0, 128, (B, S), device=DEV)
    y2 = norm_rope(x, w, sin, cos, H, 1e-6, norm_mode, ids, 0)
    y2r = norm_rope_reference(xr, wr, sin, cos, H, 1e-6, norm_mode, ids, 0)
    assert _rel_err(y2, y2r) < tol


@pytest.mark.parametrize("cols", [2048, 4096])
@pytest.mark.parametrize("with_residual", [False, True])
@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
def test_rms_norm_many_rows_per_block(cols, with_residual, wdtype):
    """More rows than resident blocks: every block walks several rows through its copy ring (ragged last round)."""
    from olmo_core_b200.ops.elementwise import rms_norm, rms_norm_reference

    torch.manual_seed(11)
    rows = 3001
    wide = torch.randn(rows, cols + 64, device=DEV, dtype=torch.bfloat16)
    x = wide[:, :cols].detach().requires_grad_(True)  # a strided view: leading dimension cols + 64
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).to(wdtype).requires_grad_(True)
    res = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16, requires_grad=True) if with_residual else None
    y = rms_norm(x, w, 1e-6, residual=res)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    rr = res.detach().float().requires_grad_(True) if with_residual else None
    yr = rms_norm_reference(xr, wr, 1e-6, rr, cols)
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=3e-2)
    assert _rel_err(y, yr) < 1e-2 and _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2
    if with_residual:
        assert _rel_err(res.grad, rr.grad) < 1e-2


@pytest.mark.parametrize("norm_mode", [0, 1, 2])
@pytest.mark.parametrize("H", [32, 8])
@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
def test_norm_rope_many_rows_per_block(norm_mode, H, wdtype):
    """Rows of a fused projection output (strided), several rows per block, offsets and explicit position ids."""
    from olmo_core_b200.ops.elementwise import norm_rope, norm_rope_reference

    torch.manual_seed(12)
    B, S, hd = 2, 1500, 128
    fused = torch.randn(B, S, H * hd + 256, device=DEV, dtype=torch.bfloat16)
    x = fused[..., 128:128 + H * hd].detach().requires_grad_(True)
    wn = H * hd if norm_mode == 1 else hd
    w = (1 + 0.1 * torch.randn(wn, device=DEV)).to(wdtype).requires_grad_(True) if norm_mode else None
    inv = 500000.0 ** (-torch.arange(0, hd, 2, device=DEV).float() / hd)
    fr = torch.outer(torch.arange(2048, device=DEV).float(), inv)
    pos = torch.cat([fr, fr], -1)
    sin, cos = pos.sin(), pos.cos()
    for ids, offset in ((None, 5), (torch.randint(0, 2048, (B, S), device=DEV), 0)):
        x.grad = None
        if w is not None:
            w.grad = None
        y = norm_rope(x, w, sin, cos, H, 1e-6, norm_mode, ids, offset)
        g = torch.randn_like(y)
        y.backward(g)
        xr = x.detach().float().requires_grad_(True)
        wr = w.detach().float().requires_grad_(True) if norm_mode else None
        yr = norm_rope_reference(xr, wr, sin, cos, H, 1e-6, norm_mode, ids, offset)
        yr.backward(g.float())
        torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=4e-2)
        torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=4e-2)
        assert _rel_err(y, yr) < 1e-2 and _rel_err(x.grad, xr.grad) < 1e-2
        if norm_mode:
            assert _rel_err(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu(dtype):
    from olmo_core_b200.ops.elementwise import swiglu

    torch.manual_seed(7)
    a = torch.randn(3, 50, 1024, device=DEV, dtype=dtype, requires_grad=True)
    b = torch.randn(3, 50, 1024, device=DEV, dtype=dtype, requires_grad=True)
    y = swiglu(a, b)
    g = torch.randn_like(y)
    y.backward(g)
    ar, br = a.detach().float().requires_grad_(True), b.detach().float().requires_grad_(True)
    yr = torch.nn.functional.silu(ar) * br
    yr.backward(g.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert _rel_err(y, yr) < tol and _rel_err(a.grad, ar.grad) < tol and _rel_err(b.grad, br.grad) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("V", [1024, 50304, 1003])
def test_cross_entropy(dtype, V):
    from olmo_core_b200.ops.loss import cross_entropy_with_z_loss

    torch.manual_seed(8)
    logits = (3 * torch.randn(4, 37, V, device=DEV)).to(dtype).requires_grad_(True)
    labels = torch.randint(0, V, (4, 37), device=DEV)
    labels[0, :5] = -100
    ce, z = cross_entropy_with_z_loss(logits, labels, reduction="sum", compute_z_loss=True, z_loss_multiplier=1e-3)
    (ce + z).backward()
    lr = logits.detach().float().requires_grad_(True)
    cer = torch.nn.functional.cross_entropy(lr.view(-1, V), labels.view(-1), ignore_index=-100, reduction="sum")
    mask = (labels.view(-1) != -100).float()
    zr = 1e-3 * (torch.logsumexp(lr.view(-1, V), -1).pow(2) * mask).sum()
    (cer + zr).backward()
    assert abs(ce.item() - cer.item()) / cer.item() < 1e-4
    assert abs(z.item() - zr.item()) / zr.item() < 1e-4
    assert _rel_err(logits.grad, lr.grad) < (2e-2 if dtype == torch.bfloat16 else 1e-4)


def test_fused_linear_cross_entropy():
    from olmo_core_b200.ops.loss import fused_linear_cross_entropy

    torch.manual_seed(9)
    N, d, V = 700, 256, 2048
    h = torch.randn(N, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(V, d, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    labels = torch.randint(0, V, (N,), device=DEV)
    labels[:9] = -100
    scale = torch.tensor(1.0 / 691, device=DEV)
    ce, z = fused_linear_cross_entropy(h, w, labels, z_loss_multiplier=1e-4, scale=scale, chunk_rows=256)
    (ce + z).backward()
    hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    lg = (hr @ wr.t()).to(torch.bfloat16).float()
    lg_live = hr @ wr.t()
    cer = torch.nn.functional.cross_entropy(lg_live, labels, ignore_index=-100, reduction="sum") / 691
    zr = 1e-4 * (torch.logsumexp(lg_live, -1).pow(2) * (labels != -100).float()).sum() / 691
    (cer + zr).backward()
    assert abs(ce.item() - cer.item()) / cer.item() < 2e-3
    assert abs(z.item() - zr.item()) / zr.item() < 2e-3
    assert _rel_err(h.grad, hr.grad) < 3e-2
    assert _rel_err(w.grad, wr.grad) < 3e-2


def test_embedding():
    from olmo_core_b200.ops.elementwise import embedding

    torch.manual_seed(10)
    w = torch.randn(1000, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 1000, (4, 77), device=DEV)
    y = embedding(ids, w)
    g = torch.randn_like(y)
    y.backward(g)
    wr = w.detach().float().requires_grad_(True)
    yr = torch.nn.functional.embedding(ids, wr)
    yr.backward(g.float())
    assert torch.equal(y.float(), yr)
    assert _rel_err(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_adamw_and_sumsq(gdtype):
    from olmo_core_b200.ops.optim import adamw_step_, adamw_step_reference_, sumsq

    torch.manual_seed(11)
    n = 100003 * 4
    p = torch.randn(n, device=DEV)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    lowp = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    step = torch.zeros((), device=DEV)
    sf = torch.ones((), device=DEV)
    gs = torch.tensor(0.5, device=DEV)
    for i in range(3):
        g = torch.randn(n, device=DEV).to(gdtype)
        kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, step=step, step_factor=sf, grad_scale=gs)
        adamw_step_(p, m, v, g, lowp=lowp, **kw)
        adamw_step_reference_(pr, mr, vr, g, **kw)
        step += sf
    assert _rel_err(p, pr) < 1e-5 and _rel_err(m, mr) < 1e-5 and _rel_err(v, vr) < 1e-5
    assert torch.equal(lowp, p.to(torch.bfloat16))
    # a skipped step leaves everything untouched
    before = p.clone()
    adamw_step_(p, m, v, g, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, step=step,
                step_factor=torch.zeros((), device=DEV))
    assert torch.equal(before, p)
    x = torch.randn(1 << 20, device=DEV).to(gdtype)
    s = sumsq(x)
    assert abs(s.item() - x.float().pow(2).sum().item()) / s.item() < 1e-4


def test_multi_linear_sums_input_gradients_in_the_epilogue():
    from olmo_core_b200.nn.feed_forward import Linear
    from olmo_core_b200.ops.gemm import multi_linear

    torch.manual_seed(11)
    x = torch.randn(2, 256, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    projs = [Linear(512, n, False, torch.bfloat16, DEV) for n in (512, 256, 768)]
    outs = multi_linear(x, projs)
    grads = [torch.randn_like(o) for o in outs]
    torch.autograd.backward(outs, grads)
    xf = x.detach().float().requires_grad_(True)
    ref = [xf @ p.weight.detach().float().t() for p in projs]
    torch.autograd.backward(ref, [g.float() for g in grads])
    for o, r in zip(outs, ref):
        assert _rel_err(o, r) < 5e-3
    assert _rel_err(x.grad, xf.grad) < 1e-2
    for p, g, in zip(projs, grads):
        want = g.float().reshape(-1, g.shape[-1]).t() @ x.detach().float().reshape(-1, 512)
        assert _rel_err(p.weight.grad, want) < 5e-3


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 8192), (4096, 11008, 2048), (19072, 256, 1024)])
def test_gemm_last_wave_split_matches_reference(M, N, K):
    """Tile counts that leave a thin last wave: those tiles are split along the reduction and summed in fixed order."""
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.gemm import gemm

    torch.manual_seed(12)
    a = torch.randn(K, M, device=DEV, dtype=torch.bfloat16)  # wgrad layout: both operands reduction-major
    b = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    base = torch.randn(M, N, device=DEV, dtype=torch.float32)
    out = base.clone()
    gemm(a, b, trans_a=True, trans_b=False, out=out, accumulate=True)
    again = base.clone()
    gemm(a, b, trans_a=True, trans_b=False, out=again, accumulate=True)
    _lib.check_device_status()
    assert torch.equal(out, again)  # deterministic
    ref = base + a.float().t() @ b.float()
    assert _rel_err(out, ref) < 5e-3
    y = gemm(a.t().contiguous(), b.t().contiguous(), trans_b=True)  # the same product through the bf16 epilogue
    assert _rel_err(y, a.float().t() @ b.float()) < 5e-3


def test_token_ids_and_labels_left_on_the_host_are_moved_not_dereferenced():
    """A model moved with ``.to()`` after construction, fed host tensors: ids and labels follow the parameters."""
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.ops.elementwise import embedding
    from olmo_core_b200.ops.loss import cross_entropy_with_z_loss

    table = torch.randn(64, 32, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 64, (3, 5))
    torch.testing.assert_close(embedding(ids, table), table[ids.cuda()])
    torch.testing.assert_close(embedding(ids.int().cuda(), table), table[ids.cuda()])
    logits = torch.randn(15, 64, device="cuda", dtype=torch.bfloat16)
    ce, _ = cross_entropy_with_z_loss(logits, ids.reshape(-1), reduction="sum")
    ref = torch.nn.functional.cross_entropy(logits.float(), ids.reshape(-1).cuda(), reduction="sum")
    torch.testing.assert_close(ce.float(), ref, rtol=2e-2, atol=2e-2)

    model = TransformerConfig.olmo2_30M(vocab_size=128, n_layers=1).build(init_device="cpu")
    model.init_weights(max_seq_len=16, device=torch.device("cpu"))
    assert model.device.type == "cpu"
    model.to("cuda")
    assert model.device.type == "cuda"
    out = model(torch.randint(0, 128, (2, 16)))
    assert out.is_cuda and torch.isfinite(out.float()).all()
