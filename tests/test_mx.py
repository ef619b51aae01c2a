"""MX (32-element block-scaled e4m3) quantisation, GEMM and linear layer: CPU emulation and the sm_100a kernels."""

import pytest
import torch

from olmo_core_b200.ops import mx


def _rand(shape, seed, scale=1.0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g) * scale
    # blocks with very different magnitudes: what block scaling is for
    x[:, : shape[1] // 4] *= 37.0
    x[: shape[0] // 3] *= 1e-3
    return x.to(torch.bfloat16).to(device)


def test_scale_layout_roundtrip():
    e = torch.randint(0, 254, (300, 512 // 32), dtype=torch.uint8)
    sf = mx.scales_from_matrix(e, 512)
    assert sf.numel() == 3 * 4 * 512
    assert torch.equal(mx.scales_as_matrix(sf, 300, 512), e)
    # row 33, block 5 -> 128-row group 0, 128-column group 1, byte (33 % 32) * 16 + (33 // 32) * 4 + 5 % 4
    assert sf[1 * 512 + 1 * 16 + 1 * 4 + 1] == e[33, 5]


@pytest.mark.parametrize("mode", ["rceil", "floor", "ceil", "even"])
def test_quantize_emulation_error(mode):
    x = _rand((256, 384), 0)
    q, sf = mx.quantize_mx_rowwise(x, mode)
    back = mx.dequantize_mx(q, sf)
    err = (back - x.float()).abs()
    blocks = x.float().view(256, -1, 32).abs().amax(-1, keepdim=True).expand(-1, -1, 32).reshape(256, 384)
    # e4m3 keeps 3 mantissa bits: the error is below 2^-3 of the block maximum after power-of-two scaling
    assert (err <= blocks * 2.0 ** -3 + 1e-30).all()
    if mode in ("rceil", "ceil"):
        assert (q.view(torch.float8_e4m3fn).float().abs() <= 448).all()
        assert (x.float().view(256, -1, 32).abs().amax(-1) <= 448 * torch.exp2(mx.scales_as_matrix(sf, 256, 384).float() - 127)).all()
    qt, sft = mx.quantize_mx_colwise_transposed(x.t().contiguous(), mode)
    assert torch.equal(qt, q) and torch.equal(sft, sf)


def test_linear_emulation_gradients():
    x = _rand((256, 256), 1).float().requires_grad_(True)
    w = (_rand((384, 256), 2).float() * 0.05).requires_grad_(True)
    y = mx.mx_linear(x, w)
    y.float().pow(2).mean().backward()
    xr, wr = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    yr = xr @ wr.t()
    yr.pow(2).mean().backward()

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm()).item()

    assert rel(y, yr) < 0.05
    assert rel(x.grad, xr.grad) < 0.08
    assert rel(w.grad, wr.grad) < 0.08


def test_linear_falls_back_on_odd_shapes():
    x = torch.randn(24, 96)
    w = torch.randn(40, 96)
    assert torch.allclose(mx.mx_linear(x, w), x @ w.t(), atol=1e-4, rtol=1e-4)


def test_config_routes_linear_through_mx():
    from olmo_core_b200.float8 import AOMXLinearConfig, Float8Config
    from olmo_core_b200.nn.feed_forward import FeedForward

    ff = FeedForward(d_model=128, hidden_size=256, bias=False, dtype=torch.float32)
    ref = FeedForward(d_model=128, hidden_size=256, bias=False, dtype=torch.float32)
    ref.load_state_dict(ff.state_dict())
    Float8Config(ao_mx=AOMXLinearConfig.mxfp8_cublas_rceil()).apply_float8_linear(ff)
    assert ff.w1.float8["mx"] is not None
    x = torch.randn(128, 128)
    y, yr = ff(x), ref(x)
    assert not torch.equal(y, yr)  # quantised
    assert ((y - yr).norm() / yr.norm()).item() < 0.08


# ----------------------------------------------------------------------------------------------------------------- GPU


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["rceil", "floor", "ceil", "even"])
@pytest.mark.parametrize("shape", [(256, 512), (1000, 384), (128, 4096)])
def test_gpu_quantize_rowwise_matches_emulation(shape, mode):
    x = _rand(shape, 3, device="cuda")
    q, sf = mx.quantize_mx_rowwise(x, mode)
    q_ref, sf_ref = mx.quantize_mx_rowwise(x.cpu(), mode)
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(mx.scales_as_matrix(sf.cpu(), *shape), mx.scales_as_matrix(sf_ref, *shape))


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["rceil", "floor", "ceil", "even"])
@pytest.mark.parametrize("shape", [(256, 512), (384, 1000), (4096, 136)])
def test_gpu_quantize_colwise_transposed_matches_emulation(shape, mode):
    x = _rand(shape, 4, device="cuda")
    q, sf = mx.quantize_mx_colwise_transposed(x, mode)
    q_ref, sf_ref = mx.quantize_mx_colwise_transposed(x.cpu(), mode)
    assert q.shape == (shape[1], shape[0])
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(mx.scales_as_matrix(sf.cpu(), shape[1], shape[0]), mx.scales_as_matrix(sf_ref, shape[1], shape[0]))


@pytest.mark.gpu
@pytest.mark.parametrize("mnk", [(128, 192, 128), (256, 384, 512), (300, 200, 256), (1024, 4096, 1024), (8192, 1000, 384)])
def test_gpu_gemm_mx_matches_dequantised_product(mnk):
    M, N, K = mnk
    a = _rand((M, K), 5, device="cuda")
    b = _rand((N, K), 6, 0.05, device="cuda")
    aq, sa = mx.quantize_mx_rowwise(a)
    bq, sb = mx.quantize_mx_rowwise(b)
    ref = mx.dequantize_mx(aq.cpu(), sa.cpu()).double() @ mx.dequantize_mx(bq.cpu(), sb.cpu()).double().t()
    out = mx.gemm_mx(aq, sa, bq, sb, out_dtype=torch.float32)
    torch.cuda.synchronize()
    from olmo_core_b200.ops import _lib

    _lib.check_device_status()
    torch.testing.assert_close(out.cpu().double(), ref, rtol=1e-4, atol=1e-4 * ref.abs().max().item())
    out_bf16 = mx.gemm_mx(aq, sa, bq, sb)
    torch.testing.assert_close(out_bf16.cpu().double(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())
    acc = torch.ones((M, N), dtype=torch.float32, device="cuda")
    mx.gemm_mx(aq, sa, bq, sb, out=acc, accumulate=True)
    torch.testing.assert_close(acc.cpu().double(), ref + 1.0, rtol=1e-4, atol=1e-4 * ref.abs().max().item() + 1e-5)
    # every launch gives the same bits
    assert torch.equal(out, mx.gemm_mx(aq, sa, bq, sb, out_dtype=torch.float32))


@pytest.mark.gpu
def test_gpu_mx_linear_forward_backward():
    torch.manual_seed(0)
    x = (torch.randn(512, 256, device="cuda") * 2).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(384, 256, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    y = mx.mx_linear(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    xc, wc = x.detach().cpu().requires_grad_(True), w.detach().cpu().requires_grad_(True)
    yc = mx.mx_linear(xc, wc)
    yc.backward(dy.cpu())
    torch.testing.assert_close(y.cpu().float(), yc.float(), rtol=2e-2, atol=2e-2 * yc.float().abs().max().item())
    torch.testing.assert_close(x.grad.cpu().float(), xc.grad.float(), rtol=2e-2, atol=2e-2 * xc.grad.float().abs().max().item())
    torch.testing.assert_close(w.grad.cpu().float(), wc.grad.float(), rtol=2e-2, atol=2e-2 * wc.grad.float().abs().max().item())


def test_weight_cast_cache_lives_for_one_optimizer_step():
    from olmo_core_b200.float8 import AOFloat8LinearConfig, AOMXLinearConfig, Float8Config, refresh_float8_scales
    from olmo_core_b200.nn.feed_forward import FeedForward

    ff = FeedForward(d_model=128, hidden_size=256, bias=False, dtype=torch.float32)
    cfg = Float8Config(ao_mx=AOMXLinearConfig())
    assert cfg.ao_mx.scale_rounding == "floor" and AOMXLinearConfig.mxfp8_cublas_rceil().scale_rounding == "rceil"
    with pytest.raises(Exception):
        AOMXLinearConfig(elem_dtype="float4_e2m1fn_x2")
    cfg.apply_float8_linear(ff)
    assert ff.w1.float8["weight_cache"] is None  # off unless asked for
    ff2 = FeedForward(d_model=128, hidden_size=256, bias=False, dtype=torch.float32)
    c2 = Float8Config(ao=AOFloat8LinearConfig.recommended())
    c2.apply_float8_linear(ff2)
    for m in (ff2.w1, ff2.w2, ff2.w3):  # force the MX op on CPU through the same cache
        m.float8["mx"] = AOMXLinearConfig()
    x = torch.randn(128, 128, requires_grad=True)
    ff2(x).sum().backward()
    cache = ff2.w1.float8["weight_cache"]
    assert set(cache) == {"mx_row", "mx_col_t"}
    first = cache["mx_row"][1][0]
    ff2(x).sum().backward()
    assert cache["mx_row"][1][0] is first  # second micro-batch reuses the cast
    with torch.no_grad():
        ff2.w1.weight.mul_(2.0)  # an ordinary in-place update is noticed through the version counter
    y_new = ff2(x)
    assert cache["mx_row"][1][0] is not first
    refresh_float8_scales(ff2)
    assert len(cache) == 0
    assert torch.isfinite(y_new).all()
