"""tcgen05 flash-attention kernels (forward, dK/dV, dQ) against a plain fp32 PyTorch reference."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(q, k, v, causal):
    B, T, H, D = q.shape
    Hkv = k.shape[2]
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    if Hkv != H:
        kf = kf.repeat_interleave(H // Hkv, 1)
        vf = vf.repeat_interleave(H // Hkv, 1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool, device=q.device), 1), float("-inf"))
    return (torch.softmax(s, -1) @ vf).permute(0, 2, 1, 3)


@pytest.mark.parametrize("B,T,H,Hkv,causal", [
    (1, 128, 1, 1, True),     # a single diagonal tile
    (2, 1024, 4, 2, True),    # several tiles, grouped-query heads
    (1, 512, 2, 1, False),    # bidirectional, multi-query
    (1, 2048, 2, 2, True),
])
def test_flash_attention_forward_and_backward(B, T, H, Hkv, causal):
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.attention import attention, has_flash_kernel

    assert has_flash_kernel(), "the kernel library must export the attention entry points on a GPU box"
    torch.manual_seed(T + H)
    dev = torch.device("cuda")
    q = torch.randn(B, T, H, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, T, Hkv, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, T, Hkv, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    dout = torch.randn(B, T, H, 128, device=dev, dtype=torch.bfloat16)

    launches = _lib.launch_count
    out = attention(q, k, v, causal=causal)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.check_device_status(dev)
    assert _lib.launch_count == launches + 2  # the in-tree kernels ran, not the PyTorch path

    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = _reference(qf, kf, vf, causal)
    ref.backward(dout.float())
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    for got, want in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        torch.testing.assert_close(got.float(), want, rtol=3e-2, atol=3e-2 * float(want.abs().max()) / 2 + 2e-2)


def test_flash_attention_reads_strided_qkv_views():
    """q, k, v as column slices of one fused projection output: no copies, the row stride goes to the tensor maps."""
    from olmo_core_b200.ops.attention import attention

    B, T, H, D = 1, 256, 2, 128
    fused = torch.randn(B, T, 3 * H * D, device="cuda", dtype=torch.bfloat16)
    q, k, v = (fused[..., i * H * D:(i + 1) * H * D].view(B, T, H, D) for i in range(3))
    out = attention(q, k, v, causal=True)
    ref = _reference(q, k, v, True)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)


def test_unsupported_shapes_take_the_masked_path():
    from olmo_core_b200.ops.attention import attention, attention_reference

    q = torch.randn(1, 100, 2, 64, device="cuda", dtype=torch.bfloat16)
    out = attention(q, q, q, causal=True, window_size=16)
    ref = attention_reference(q, q, q, causal=True, window_size=16)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


def _doc_boundaries(total: int, seed: int, B: int, T: int) -> torch.Tensor:
    """Random document boundaries over B * T tokens; every multiple of T is a boundary."""
    g = torch.Generator().manual_seed(seed)
    cuts = set(range(0, total + 1, T))
    for b in range(B):
        n = int(torch.randint(1, 6, (1,), generator=g))
        cuts |= {b * T + int(c) for c in torch.randint(1, T, (n,), generator=g)}
    return torch.tensor(sorted(cuts), dtype=torch.int32)


@pytest.mark.parametrize("B,T,H,Hkv,window,docs", [
    (1, 512, 2, 2, 128, False),    # window of exactly one tile
    (2, 1024, 4, 2, 100, False),   # window smaller than a tile
    (1, 2048, 2, 1, 700, False),   # window spanning several tiles, not tile-aligned
    (2, 1024, 2, 2, None, True),   # packed documents
    (1, 2048, 4, 2, 300, True),    # documents and a window together
])
def test_flash_attention_windows_and_documents(B, T, H, Hkv, window, docs):
    """Sliding windows and document boundaries run in the flash kernels (skipped key tiles + element-wise masks)."""
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.attention import attention, attention_reference

    torch.manual_seed(T + (window or 0))
    dev = torch.device("cuda")
    cu = _doc_boundaries(B * T, seed=T, B=B, T=T).to(dev) if docs else None
    q = torch.randn(B, T, H, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, T, Hkv, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, T, Hkv, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    dout = torch.randn(B, T, H, 128, device=dev, dtype=torch.bfloat16)
    launches = _lib.launch_count
    out = attention(q, k, v, causal=True, window_size=window, cu_seqlens=cu)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.check_device_status(dev)
    assert _lib.launch_count == launches + 2  # forward and backward launchers of the in-tree kernels

    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = attention_reference(qf, kf, vf, causal=True, window_size=window, cu_seqlens=cu)
    ref.backward(dout.float())
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    for got, want in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        torch.testing.assert_close(got.float(), want, rtol=3e-2, atol=3e-2 * float(want.abs().max()) / 2 + 2e-2)


@pytest.mark.parametrize("B,Tq,Tk,H,Hkv,window", [
    (1, 128, 512, 2, 1, None),     # one query tile at the end of a longer key sequence
    (2, 256, 1024, 4, 2, None),
    (1, 512, 1536, 2, 2, 300),     # with a sliding window
])
def test_flash_attention_queries_at_the_end_of_longer_keys(B, Tq, Tk, H, Hkv, window):
    """Fewer queries than keys (causal masking aligned at the end) stays on the flash kernels."""
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.attention import attention, attention_reference

    torch.manual_seed(Tq + Tk)
    dev = torch.device("cuda")
    q = torch.randn(B, Tq, H, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, Tk, Hkv, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, Tk, Hkv, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    dout = torch.randn(B, Tq, H, 128, device=dev, dtype=torch.bfloat16)
    launches = _lib.launch_count
    out = attention(q, k, v, causal=True, window_size=window)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.check_device_status(dev)
    assert _lib.launch_count == launches + 2
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = attention_reference(qf, kf, vf, causal=True, window_size=window)
    ref.backward(dout.float())
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    for got, want in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        torch.testing.assert_close(got.float(), want, rtol=3e-2, atol=3e-2 * float(want.abs().max()) / 2 + 2e-2)


class _OneGpuExchange:
    """All shards of a context-parallel group on one GPU: the kernels only see addresses, so this exercises the sharded
    tile lookup (sources, chunks, zig-zag order) without peers."""

    def __init__(self, ks, vs):
        import ctypes

        self.world_size = len(ks)
        self.k_ptrs = (ctypes.c_void_p * len(ks))(*[t.data_ptr() for t in ks])
        self.v_ptrs = (ctypes.c_void_p * len(vs))(*[t.data_ptr() for t in vs])
        self.partials = None

    def publish(self, k, v, layout, window=None):
        return self.k_ptrs, self.v_ptrs, self.world_size, k.shape[1], layout.c_array

    def reduce_to_owners(self, dk_all, dv_all, window=None):
        self.partials = (dk_all, dv_all)
        n = dk_all.shape[1] // self.world_size
        return torch.zeros_like(dk_all[:, :n]), torch.zeros_like(dv_all[:, :n])


@pytest.mark.parametrize("cp,zig_zag,T,window", [
    (2, False, 512, None),
    (4, True, 2048, None),
    (4, False, 2048, 300),
    (2, True, 1024, 200),
])
def test_sharded_attention_reads_tiles_from_their_owners(cp, zig_zag, T, window):
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.attention import ShardedSequenceLayout, attention_reference, sharded_attention
    from olmo_core_b200.parallel.context import local_position_ranges

    torch.manual_seed(T + cp)
    dev = torch.device("cuda")
    B, H, Hkv = 2, 4, 2
    q = torch.randn(B, T, H, 128, device=dev, dtype=torch.bfloat16)
    k = torch.randn(B, T, Hkv, 128, device=dev, dtype=torch.bfloat16)
    v = torch.randn(B, T, Hkv, 128, device=dev, dtype=torch.bfloat16)
    dout = torch.randn(B, T, H, 128, device=dev, dtype=torch.bfloat16)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = attention_reference(qf, kf, vf, causal=True, window_size=window)
    ref.backward(dout.float())

    T_local = T // cp
    rows = [torch.cat([torch.arange(a, b, device=dev) for a, b in local_position_ranges(T_local, r, cp, zig_zag)])
            for r in range(cp)]
    ks = [k[:, idx].contiguous() for idx in rows]
    vs = [v[:, idx].contiguous() for idx in rows]
    dk_sum = torch.zeros_like(kf)
    dv_sum = torch.zeros_like(vf)
    for r in range(cp):
        ex = _OneGpuExchange(ks, vs)
        layout = ShardedSequenceLayout.for_rank(T_local, r, cp, zig_zag)
        ql = q[:, rows[r]].contiguous().requires_grad_(True)
        out = sharded_attention(ql, ks[r], vs[r], exchange=ex, layout=layout, window_size=window)
        out.backward(dout[:, rows[r]].contiguous())
        torch.cuda.synchronize()
        _lib.check_device_status(dev)
        torch.testing.assert_close(out.float(), ref[:, rows[r]], rtol=2e-2, atol=2e-2)
        want = qf.grad[:, rows[r]]
        torch.testing.assert_close(ql.grad.float(), want, rtol=3e-2, atol=3e-2 * float(want.abs().max()) / 2 + 2e-2)
        dk_sum += ex.partials[0].float()
        dv_sum += ex.partials[1].float()
    for got, want in ((dk_sum, kf.grad), (dv_sum, vf.grad)):
        torch.testing.assert_close(got, want, rtol=3e-2, atol=3e-2 * float(want.abs().max()) / 2 + 3e-2)
