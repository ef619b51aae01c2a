"""
``ocb_rmsnorm_bwd_static``: the RMSNorm backward entry point that uses the library's built-in scratch array
instead of a caller-provided buffer. Checked through the exported C symbol against the regular entry points
(``ocb_rmsnorm_bwd`` + ``ocb_reduce_partials``) and a plain fp32 PyTorch reference, on two calls in a row so
that a scratch array left dirty by the first call would show in the second.

The file name sorts last on purpose: the test must pass both on its own and after every other GPU test has
used the device.
"""

import ctypes
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_GROUP = 4096
ERR_TOO_SMALL = -6


def _bind():
    from olmo_core_b200.ops import _lib

    _lib.register_signature(
        "ocb_rmsnorm_bwd_static",
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
         c_longlong, c_longlong, c_int, c_int, c_int, c_void_p],
    )
    _lib.register_signature("ocb_rmsnorm_bwd_static_max_group", [])
    handle = _lib.lib()
    handle.ocb_rmsnorm_bwd_static_strerror.argtypes = [c_int]
    handle.ocb_rmsnorm_bwd_static_strerror.restype = ctypes.c_char_p
    return _lib, handle


def _reference(dy, x, w, group):
    """Plain fp32 autograd of y = x * rsqrt(mean(x^2) + eps) * w over groups of ``group`` channels."""
    xf = x.float().detach().requires_grad_(True)
    wf = w.float().detach().requires_grad_(True)
    xg = xf.view(x.shape[0], -1, group)
    y = xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    y.view_as(xf).backward(dy.float())
    return xf.grad, wf.grad


def _forward_rstd(_lib, handle, x, w, group):
    rows, cols = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows * (cols // group), dtype=torch.float32, device=x.device)
    rc = handle.ocb_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), rstd.data_ptr(), rows, cols, group,
                                cols, cols, 0, 1e-6, _lib.dt(x), _lib.dt(w), _lib.stream_ptr())
    assert rc == 0
    return rstd


def _existing(_lib, handle, dy, x, w, rstd, group):
    rows, cols = x.shape
    n_partial = handle.ocb_norm_bwd_partials()
    partial = torch.empty(n_partial, group, dtype=torch.float32, device=x.device)
    dx = torch.empty_like(x)
    dw = torch.empty(group, dtype=torch.float32, device=x.device)
    rc = handle.ocb_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                partial.data_ptr(), rows, cols, group, cols, cols, cols, _lib.dt(x), _lib.dt(w),
                                _lib.stream_ptr())
    assert rc == 0
    rc = handle.ocb_reduce_partials(partial.data_ptr(), dw.data_ptr(), n_partial, group, 0, _lib.DT_F32,
                                    _lib.stream_ptr())
    assert rc == 0
    return dx, dw


def _static(_lib, handle, dy, x, w, rstd, group, dx, dw, accumulate=0):
    rows, cols = x.shape
    return handle.ocb_rmsnorm_bwd_static(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                         dw.data_ptr(), accumulate, rows, cols, group, cols, cols, cols, _lib.dt(x),
                                         _lib.dt(w), _lib.dt(dw), _lib.stream_ptr())


@pytest.mark.parametrize("rows,cols,group", [(4096, 4096, 4096), (1000, 1024, 128), (37, 512, 512)])
def test_static_scratch_matches_existing_entry_point_twice(rows, cols, group):
    _lib, handle = _bind()
    assert handle.ocb_rmsnorm_bwd_static_max_group() == MAX_GROUP
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(1234 + rows)
    # every buffer the entry point touches exists before the calls; the calls themselves must not allocate
    dx = torch.empty(rows, cols, dtype=torch.bfloat16, device=dev)
    dw = torch.empty(group, dtype=torch.float32, device=dev)
    for call in range(2):
        x = torch.randn(rows, cols, device=dev, generator=gen).bfloat16()
        dy = (torch.randn(rows, cols, device=dev, generator=gen) * (1.0 + call)).bfloat16()
        w = (1.0 + 0.1 * torch.randn(group, device=dev, generator=gen)).float()
        rstd = _forward_rstd(_lib, handle, x, w, group)
        dx_old, dw_old = _existing(_lib, handle, dy, x, w, rstd, group)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        rc = _static(_lib, handle, dy, x, w, rstd, group, dx, dw)
        torch.cuda.synchronize()
        assert rc == 0, handle.ocb_rmsnorm_bwd_static_strerror(rc)
        assert torch.cuda.memory_allocated() == before
        if call == 1:
            # The caching allocator's counter cannot see a raw cudaMalloc inside the library; the driver's count of
            # free device memory can. The first call may still load the module, the second must leave it unchanged.
            assert torch.cuda.mem_get_info()[0] == free_before
        # same kernel, same inputs: dx is bitwise equal; dw differs only by the order of the fp32 atomics
        assert torch.equal(dx, dx_old)
        torch.testing.assert_close(dw, dw_old, rtol=1e-4, atol=1e-3)
        dx_ref, dw_ref = _reference(dy, x, w, group)
        torch.testing.assert_close(dx.float(), dx_ref, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(dw, dw_ref, rtol=2e-2, atol=2e-2 * (rows * cols / group) ** 0.5)


def test_static_scratch_accumulates_into_dw():
    _lib, handle = _bind()
    dev = torch.device("cuda")
    rows, cols = 512, 2048
    x = torch.randn(rows, cols, device=dev).bfloat16()
    dy = torch.randn(rows, cols, device=dev).bfloat16()
    w = torch.ones(cols, device=dev)
    rstd = _forward_rstd(_lib, handle, x, w, cols)
    dx = torch.empty_like(x)
    dw = torch.zeros(cols, dtype=torch.float32, device=dev)
    assert _static(_lib, handle, dy, x, w, rstd, cols, dx, dw, accumulate=0) == 0
    once = dw.clone()
    assert _static(_lib, handle, dy, x, w, rstd, cols, dx, dw, accumulate=1) == 0
    torch.testing.assert_close(dw, 2 * once, rtol=1e-4, atol=1e-3)


def test_static_scratch_empty_batch_zeroes_dw():
    _lib, handle = _bind()
    dev = torch.device("cuda")
    cols = 1024
    x = torch.empty(0, cols, dtype=torch.bfloat16, device=dev)
    w = torch.ones(cols, device=dev)
    rstd = torch.empty(0, device=dev)
    dw = torch.full((cols,), 3.0, device=dev)
    assert _static(_lib, handle, x, x, w, rstd, cols, x, dw, accumulate=1) == 0
    torch.cuda.synchronize()
    assert bool((dw == 3.0).all())
    assert _static(_lib, handle, x, x, w, rstd, cols, x, dw, accumulate=0) == 0
    torch.cuda.synchronize()
    assert bool((dw == 0.0).all())


def test_static_scratch_rejects_groups_beyond_its_size():
    _lib, handle = _bind()
    dev = torch.device("cuda")
    rows, cols = 8, 2 * MAX_GROUP
    x = torch.randn(rows, cols, device=dev).bfloat16()
    w = torch.ones(cols, device=dev)
    rstd = torch.ones(rows, device=dev)
    dx = torch.full_like(x, 7.0)
    dw = torch.full((cols,), 7.0, device=dev)
    rc = _static(_lib, handle, x, x, w, rstd, cols, dx, dw)
    torch.cuda.synchronize()
    assert rc == ERR_TOO_SMALL
    assert b"OCB_STATIC_SCRATCH_MAX_GROUP" in handle.ocb_rmsnorm_bwd_static_strerror(rc)
    # nothing was launched
    assert bool((dx == 7.0).all()) and bool((dw == 7.0).all())
