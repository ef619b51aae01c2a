"""
CTA-pair GEMM (``csrc/gemm_pair_sm100.cu``) against fp32 PyTorch references: every operand layout and epilogue on shapes
with ragged tile edges, element-wise (a wrong row or tile must not hide in a norm), run-to-run bit equality, and the
gated-MLP path with the activation in the GEMM epilogues against the unfused path.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _pair(M, N, K, a, b, out, a_mn, b_mn, epi):
    from olmo_core_b200.ops import _lib

    def ld(t):
        return t.stride(0)

    rc = _lib.lib().ocb_gemm_bf16_pair(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, ld(a), ld(b), ld(out), a_mn, b_mn,
                                       epi, _lib.status_buffer(a.device).data_ptr(), _lib.stream_ptr())
    assert rc == 0, rc
    _lib.check_device_status()


def _close(got, ref, K):
    # bf16 operands are exact in fp32; the error is the output rounding plus fp32 accumulation order
    tol = 2e-2 if got.dtype == torch.bfloat16 else 1e-3
    torch.testing.assert_close(got.float(), ref, atol=tol * K ** 0.5, rtol=tol)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (1000, 520, 264), (2088, 2376, 520), (304, 8, 72)])
def test_pair_gemm_all_layouts_elementwise(M, N, K):
    from olmo_core_b200.ops import _lib

    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    at = a.t().contiguous()
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    wt = w.t().contiguous()
    ref = a.float() @ w.float().t()
    for a_op, a_mn in ((a, 0), (at, 1)):
        for b_op, b_mn in ((w, 0), (wt, 1)):
            out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
            _pair(M, N, K, a_op, b_op, out, a_mn, b_mn, _lib.EPI_BF16)
            _close(out, ref, K)
    out32 = torch.empty(M, N, device=DEV, dtype=torch.float32)
    _pair(M, N, K, a, w, out32, 0, 0, _lib.EPI_F32)
    _close(out32, ref, K)
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    expect = acc + ref
    _pair(M, N, K, at, wt, acc, 1, 1, _lib.EPI_F32_ACC)
    _close(acc, expect, K)
    accb = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    expect = accb.float() + ref
    _pair(M, N, K, a, w, accb, 0, 0, _lib.EPI_BF16_ACC)
    _close(accb, expect, K)


def test_pair_gemm_writes_nothing_outside_its_output():
    from olmo_core_b200.ops import _lib

    torch.manual_seed(1)
    M, N, K = 700, 392, 136
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    buf = torch.full((M + 64, 512), 7.0, device=DEV, dtype=torch.bfloat16)
    out = buf[:M, 64:64 + N]
    _pair(M, N, K, a, w, out, 0, 0, _lib.EPI_BF16)
    _close(out, a.float() @ w.float().t(), K)
    assert (buf[:, :64] == 7).all() and (buf[:, 64 + N:] == 7).all() and (buf[M:] == 7).all()


def test_gemm_is_bit_reproducible():
    from olmo_core_b200.ops.gemm import gemm

    torch.manual_seed(2)
    for M, N, K in ((4096, 4096, 1024), (2500, 4096, 512), (8192, 1024, 512)):  # pair kernel, split last wave, one-CTA tiles
        a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
        assert torch.equal(gemm(a, w), gemm(a, w))
        g = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
        d1 = torch.zeros(N, K, device=DEV, dtype=torch.float32)
        d2 = torch.zeros(N, K, device=DEV, dtype=torch.float32)
        gemm(g, a, trans_a=True, trans_b=False, out=d1, accumulate=True)
        gemm(g, a, trans_a=True, trans_b=False, out=d2, accumulate=True)
        assert torch.equal(d1, d2)


@pytest.mark.parametrize("M,H,K", [(1024, 1408, 512), (1000, 1416, 520)])
def test_swiglu_epilogue_kernels(M, H, K):
    from olmo_core_b200.ops import _lib

    torch.manual_seed(3)
    L = _lib.lib()
    st = _lib.status_buffer(torch.device(DEV)).data_ptr()
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16) * 0.5
    w13 = torch.randn(2 * H, K, device=DEV, dtype=torch.bfloat16) * 0.1
    ab = torch.empty(M, 2 * H, device=DEV, dtype=torch.bfloat16)
    h = torch.empty(M, H, device=DEV, dtype=torch.bfloat16)
    assert L.ocb_gemm_swiglu_fwd(x.data_ptr(), w13.data_ptr(), ab.data_ptr(), h.data_ptr(), M, H, K, K, K, 2 * H, H, st,
                                 _lib.stream_ptr()) == 0
    _close(ab, x.float() @ w13.float().t(), K)
    ra, rb = ab[:, :H].float(), ab[:, H:].float()
    torch.testing.assert_close(h.float(), torch.nn.functional.silu(ra) * rb, atol=2e-2, rtol=2e-2)
    D = K + 8
    dy = torch.randn(M, D, device=DEV, dtype=torch.bfloat16) * 0.5
    w2 = torch.randn(D, H, device=DEV, dtype=torch.bfloat16) * 0.1
    dab = torch.empty(M, 2 * H, device=DEV, dtype=torch.bfloat16)
    h2 = torch.empty(M, H, device=DEV, dtype=torch.bfloat16)
    for hout in (h2, None):
        assert L.ocb_gemm_swiglu_bwd(dy.data_ptr(), w2.data_ptr(), ab.data_ptr(), dab.data_ptr(),
                                     None if hout is None else hout.data_ptr(), M, H, D, D, H, 2 * H, 2 * H, H, st,
                                     _lib.stream_ptr()) == 0
        dh = dy.float() @ w2.float()
        s = torch.sigmoid(ra)
        torch.testing.assert_close(dab[:, :H].float(), dh * rb * s * (1 + ra * (1 - s)), atol=4e-2, rtol=3e-2)
        torch.testing.assert_close(dab[:, H:].float(), dh * ra * s, atol=4e-2, rtol=3e-2)
    torch.testing.assert_close(h2.float(), torch.nn.functional.silu(ra) * rb, atol=2e-2, rtol=2e-2)
    _lib.check_device_status()


def test_feed_forward_fused_matches_unfused():
    """A FeedForward under the sharded-parameter runtime takes the fused path; its result and gradients match the
    projection-by-projection path on the same weights."""
    from olmo_core_b200.nn.feed_forward import FeedForward
    from olmo_core_b200.ops import gemm as gemm_ops
    from olmo_core_b200.parallel.fsdp import ShardedParamRuntime

    torch.manual_seed(4)
    d, H, T = 512, 1408, 768
    ff = FeedForward(d_model=d, hidden_size=H, bias=False, dtype=torch.float32, init_device=DEV)
    rt = ShardedParamRuntime(ff, param_dtype=torch.bfloat16, device=torch.device(DEV))
    rt.materialize(torch.device(DEV))
    rt.sync_lowp()
    assert gemm_ops.stacked_pair(ff.w1.weight._lowp, ff.w3.weight._lowp) is not None
    x = (torch.randn(2, T // 2, d, device=DEV) * 0.5).to(torch.bfloat16)
    dy = (torch.randn(2, T // 2, d, device=DEV) * 0.1).to(torch.bfloat16)

    calls = []
    real = gemm_ops.SwiGLUMLPFunction.apply

    def run(fused):
        rt.zero_grad()
        xi = x.clone().requires_grad_(True)
        if fused:
            y = ff(xi)
        else:
            orig = gemm_ops.swiglu_mlp
            import olmo_core_b200.nn.feed_forward as ffmod

            ffmod.swiglu_mlp = lambda *a, **k: None
            try:
                y = ff(xi)
            finally:
                ffmod.swiglu_mlp = orig
        y.backward(dy)
        grads = {n: p.main_grad.clone() for n, p in ff.named_parameters()}
        return y.detach().float(), xi.grad.float(), grads

    y1, dx1, g1 = run(True)
    y0, dx0, g0 = run(False)
    # 'selected_ops' activation checkpointing: the gated activation is not kept, the backward kernel re-derives it
    ff.recompute_activation = True
    y2, dx2, g2 = run(True)
    ff.recompute_activation = False
    assert torch.equal(y2, y1) and torch.equal(dx2, dx1)
    for n in g1:
        assert torch.equal(g2[n], g1[n]), n
    torch.testing.assert_close(y1, y0, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(dx1, dx0, atol=2e-2, rtol=2e-2)
    for n in g0:
        assert g0[n].abs().max() > 0
        torch.testing.assert_close(g1[n], g0[n], atol=3e-2, rtol=3e-2)
