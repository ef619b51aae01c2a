"""
Pytest marks, parameter lists and capability probes (src/olmo_core/testing/utils.py:1-250). GPU tests carry the ``gpu``
mark; the capabilities that the reference gates on optional wheels are built in here, so each probe answers whether this
package's own kernel for that role can run on the current machine.
"""

from __future__ import annotations

import pytest
import torch

__all__ = [
    "BACKENDS",
    "DEVICES",
    "INIT_DEVICES",
    "LOW_PRECISION_DTYPES",
    "GPU_MARKS",
    "MULTI_GPU_MARKS",
    "MPS_MARKS",
    "has_cuda",
    "has_multiple_gpus",
    "has_mps",
    "has_te",
    "requires_gpu",
    "requires_multi_gpu",
    "requires_mps",
    "FLASH_2_MARKS",
    "FLASH_3_MARKS",
    "FLASH_4_MARKS",
    "GROUPED_GEMM_MARKS",
    "TE_MARKS",
    "has_flash_attn_2",
    "has_flash_attn_3",
    "has_flash_attn_4",
    "has_grouped_gemm",
    "has_torchao",
    "has_quack",
    "requires_flash_attn_2",
    "requires_flash_attn_3",
    "requires_flash_attn_4",
    "requires_grouped_gemm",
    "requires_fla",
    "requires_quack",
    "requires_dion",
    "requires_te",
    "requires_compute_capability",
]

has_cuda = torch.cuda.is_available()
has_multiple_gpus = has_cuda and torch.cuda.device_count() > 1

GPU_MARKS = (pytest.mark.gpu, pytest.mark.skipif(not has_cuda, reason="Requires a GPU"))
MULTI_GPU_MARKS = (pytest.mark.gpu, pytest.mark.skipif(not has_multiple_gpus, reason="Requires multiple GPUs"))


def _apply(marks, func):
    for mark in marks:
        func = mark(func)
    return func


def requires_gpu(func):
    return _apply(GPU_MARKS, func)


has_mps = bool(getattr(torch.backends, "mps", None)) and torch.backends.mps.is_available()
MPS_MARKS = (pytest.mark.skipif(not has_mps, reason="Requires MPS"),)


def requires_mps(func):
    return _apply(MPS_MARKS, func)


def requires_multi_gpu(func):
    return _apply(MULTI_GPU_MARKS, func)


def _kernels_available() -> bool:
    if not has_cuda:
        return False
    from ..ops.attention import has_flash_kernel

    return has_flash_kernel()


# The capabilities that the reference gates on optional wheels are built in here: each probe answers whether this
# package's own kernel for that role can run on the current machine.
has_flash_attn_2 = has_flash_attn_3 = has_flash_attn_4 = _kernels_available()
has_grouped_gemm = has_cuda
has_torchao = has_cuda  # float8 training uses this package's own GEMMs
has_quack = has_cuda  # fused RMSNorm / cross-entropy kernels are built in
has_te = False

FLASH_2_MARKS = FLASH_3_MARKS = FLASH_4_MARKS = (
    pytest.mark.gpu, pytest.mark.skipif(not has_flash_attn_2, reason="Requires the flash-attention kernels (B200)"))
GROUPED_GEMM_MARKS = GPU_MARKS
TE_MARKS = (pytest.mark.gpu, pytest.mark.skipif(True, reason="Transformer Engine is not used by this framework"))


def requires_flash_attn_2(func):
    return _apply(FLASH_2_MARKS, func)


requires_flash_attn_3 = requires_flash_attn_4 = requires_flash_attn_2


def requires_grouped_gemm(func):
    return _apply(GROUPED_GEMM_MARKS, func)


def requires_fla(func):  # the gated delta rule is built in and runs everywhere
    return func


def requires_quack(func):
    return _apply(GPU_MARKS, func)


def requires_dion(func):  # the Dion optimizer is built in
    return func


def requires_te(func):
    return _apply(TE_MARKS, func)


def requires_compute_capability(min_cc: int):
    """``min_cc`` as major * 10 + minor, e.g. 100 for sm_100."""
    def decorator(func):
        ok = has_cuda and (lambda c: c[0] * 10 + c[1])(torch.cuda.get_device_capability()) >= min_cc
        return _apply((pytest.mark.gpu, pytest.mark.skipif(not ok, reason=f"Requires compute capability >= {min_cc}")), func)

    return decorator


INIT_DEVICES = [
    pytest.param(torch.device("meta"), id="device=meta"),
    pytest.param(torch.device("cpu"), id="device=CPU"),
    pytest.param(torch.device("cuda"), id="device=CUDA", marks=GPU_MARKS),
]
DEVICES = [
    pytest.param(torch.device("cpu"), id="device=CPU"),
    pytest.param(torch.device("cuda"), id="device=CUDA", marks=GPU_MARKS),
]
BACKENDS = [
    pytest.param("gloo", id="backend=GLOO"),
    pytest.param("cuda:nccl,cpu:gloo", id="backend=NCCL", marks=MULTI_GPU_MARKS),
]
LOW_PRECISION_DTYPES = [
    pytest.param(torch.float16, id="dtype=float16"),
    pytest.param(torch.bfloat16, id="dtype=bfloat16", marks=GPU_MARKS),
]
