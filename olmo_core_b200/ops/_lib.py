"""
ctypes bindings for ``libocb_kernels.so`` (the hand-written sm_100a kernels).

The library is built in-tree by :mod:`olmo_core_b200.ops.build`. On a machine with a CUDA device the
library is mandatory: a missing or unloadable library raises instead of silently falling back to
PyTorch kernels. On CPU-only machines nothing is loaded and the ops use their PyTorch reference path.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .build import LIB_PATH

_lib: Optional["_Library"] = None
_lock = threading.Lock()

DT_BF16 = 0
DT_F32 = 1

EPI_BF16 = 0
EPI_F32_ACC = 1
EPI_F32 = 2
EPI_BF16_ACC = 3
EPI_F32_RED_PEER = 4


class KernelError(RuntimeError):
    """A kernel launcher rejected its arguments or a device-side wait reported a time-out."""


_SIGS = {
    "ocb_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                      c_int, c_int, c_void_p, c_void_p],
    "ocb_gemm_bf16_pair": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                           c_int, c_int, c_void_p, c_void_p],
    "ocb_gemm_set_pair_mode": [c_int],
    "ocb_gemm_swiglu_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                            c_longlong, c_void_p, c_void_p],
    "ocb_gemm_swiglu_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong,
                            c_longlong, c_longlong, c_longlong, c_void_p, c_void_p],
    "ocb_peer_gather_segments": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p],
    "ocb_peer_pull_reduce_segments": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_float, c_void_p],
    "ocb_peer_barrier_flag_words": [],
    "ocb_peer_barrier": [c_void_p, c_int, c_int, c_int, ctypes.c_uint, c_longlong, c_int, c_void_p, c_void_p],
    "ocb_grouped_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_longlong,
                              c_longlong, c_longlong, c_int, c_int, c_void_p, c_void_p],
    "ocb_gemm_bf16_tp": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_int,
                         c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "ocb_gemm_fp8": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong,
                     c_longlong, c_int, c_void_p, c_void_p],
    "ocb_quantize_e4m3_rowwise": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong, c_int, c_void_p],
    "ocb_quantize_e4m3_colwise_t": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong, c_int,
                                    c_void_p],
    "ocb_moe_router_topk": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                            c_longlong, c_int, c_void_p],
    "ocb_moe_sort": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ocb_moe_gather": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p],
    "ocb_moe_scatter": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p],
    "ocb_moe_rowdot": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p],
    "ocb_moe_push_rows": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                          c_longlong, c_int, c_longlong, c_longlong, c_void_p, c_void_p],
    "ocb_rmsnorm_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong,
                        c_longlong, c_float, c_int, c_int, c_void_p],
    "ocb_norm_bwd_partials": [],
    "ocb_rmsnorm_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong,
                        c_longlong, c_longlong, c_int, c_int, c_void_p],
    "ocb_reduce_partials": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "ocb_norm_rope_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_longlong, c_longlong, c_float, c_int, c_int, c_void_p],
    "ocb_norm_rope_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_int,
                          c_void_p],
    "ocb_swiglu_fwd": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_longlong, c_longlong, c_longlong, c_int,
                       c_void_p],
    "ocb_swiglu_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_longlong, c_longlong,
                       c_longlong, c_longlong, c_longlong, c_int, c_void_p],
    "ocb_cross_entropy_fwd_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong,
                                  c_longlong, c_longlong, c_float, c_void_p, c_int, c_void_p],
    "ocb_embedding_fwd": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_int, c_void_p],
    "ocb_embedding_bwd": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_int, c_void_p],
    "ocb_adamw_step": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_float, c_float, c_float,
                       c_float, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "ocb_sumsq_partials": [],
    "ocb_sumsq": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ocb_cast_f32_to_bf16": [c_void_p, c_void_p, c_longlong, c_void_p],
}

# Entry points that newer builds of the library add; bound when present.
_OPTIONAL_SIGS = {
    "ocb_attention_fwd": None,
    "ocb_attention_bwd": None,
}


class _Library:
    """
    The loaded kernel library. Entry points resolve once and are cached as plain attributes. With NVTX ranges switched
    on (:func:`set_nvtx`, or ``OLMO_CORE_B200_NVTX=1`` in the environment) every launcher call is bracketed by a range
    named after its entry point, so a timeline shows which op issued which kernels.
    """

    def __init__(self, handle: ctypes.CDLL):
        object.__setattr__(self, "_handle", handle)

    def __getattr__(self, name: str):
        fn = getattr(self._handle, name)
        if _nvtx_enabled and callable(fn):
            raw = fn

            def fn(*args, _raw=raw, _name=name):  # type: ignore[no-redef]
                torch.cuda.nvtx.range_push(_name)
                try:
                    return _raw(*args)
                finally:
                    torch.cuda.nvtx.range_pop()

            fn.argtypes, fn.restype = raw.argtypes, raw.restype  # type: ignore[attr-defined]
        object.__setattr__(self, name, fn)
        return fn


_nvtx_enabled = os.environ.get("OLMO_CORE_B200_NVTX", "0") not in ("0", "")


def set_nvtx(enabled: bool) -> None:
    """Switch NVTX ranges around the kernel launchers (and around transformer blocks) on or off."""
    global _nvtx_enabled
    _nvtx_enabled = bool(enabled)
    if isinstance(_lib, _Library):
        for name in [k for k in vars(_lib) if k != "_handle"]:
            object.__delattr__(_lib, name)


def nvtx_enabled() -> bool:
    return _nvtx_enabled


def available() -> bool:
    """True when the CUDA kernels should be used (a CUDA device is present)."""
    return torch.cuda.is_available()


def lib() -> "_Library":
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise KernelError(
                f"{LIB_PATH} is missing. Build it with `python -m olmo_core_b200.ops.build` "
                "(nvcc, sm_100a) before using CUDA tensors."
            )
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, argtypes in _SIGS.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        _lib = _Library(handle)
    return _lib


def register_signature(name: str, argtypes) -> None:
    """Declare the signature of an additional entry point (used by ops that live in their own .cu)."""
    fn = getattr(lib()._handle, name)
    fn.argtypes = argtypes
    fn.restype = c_int


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def dt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return DT_BF16
    if t.dtype == torch.float32:
        return DT_F32
    raise KernelError(f"unsupported dtype {t.dtype}: the sm_100a kernels take bfloat16 or float32")


launch_count = 0


def check(rc: int, what: str) -> None:
    """Validate a launcher's return code; also counts launcher calls (see ``launch_count``)."""
    global launch_count
    launch_count += 1
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


_status_bufs: dict = {}


def status_buffer(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write their error status to."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    buf = _status_bufs.get(key)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
        _status_bufs[key] = buf
    return buf


_STATUS_TEXT = {
    1: "TMA producer timed out waiting for a free shared-memory stage",
    2: "MMA issuer timed out waiting for operands or a free accumulator",
    3: "epilogue timed out waiting for an accumulator",
    4: "timed out waiting for a flag owned by another rank",
    5: "bad kernel argument",
}


def check_device_status(device: Optional[torch.device] = None) -> None:
    """Synchronising check of the device status word; raises if any kernel reported a time-out."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    buf = status_buffer(device)
    code = int(buf[0].item())
    if code != 0:
        buf.zero_()
        raise KernelError(f"device-side wait failed: {_STATUS_TEXT.get(code, code)}")
