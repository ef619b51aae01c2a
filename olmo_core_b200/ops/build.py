"""
Ahead-of-time build of the sm_100a kernel library.

``python -m olmo_core_b200.ops.build`` compiles every ``csrc/*.cu`` with ``nvcc`` for ``sm_100a`` and
links them into ``olmo_core_b200/ops/libocb_kernels.so`` next to this file. The library exposes plain C
entry points (``csrc/ocb_api.h``) that :mod:`olmo_core_b200.ops._lib` binds with :mod:`ctypes`, so no
PyTorch headers are involved and a full rebuild takes seconds. nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Optional

OPS_DIR = Path(__file__).resolve().parent
CSRC_DIR = OPS_DIR / "csrc"
BUILD_DIR = OPS_DIR / "_build"
LIB_PATH = OPS_DIR / "libocb_kernels.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
    "-cudart",
    "shared",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    if cand.exists():
        return str(cand)
    found = shutil.which("nvcc")
    if found is None:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


def _source_hash(path: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(path.read_bytes())
    for header in sorted(list(CSRC_DIR.glob("*.cuh")) + list(CSRC_DIR.glob("*.h"))):
        h.update(header.read_bytes())
    return h.hexdigest()


def sources() -> List[Path]:
    return sorted(CSRC_DIR.glob("*.cu"))


def _compile_one(src: Path, verbose: bool) -> Path:
    obj = BUILD_DIR / (src.stem + ".o")
    stamp = BUILD_DIR / (src.stem + ".hash")
    digest = _source_hash(src)
    if obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC_DIR), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = BUILD_DIR / (src.stem + ".ptxas.log")
    log.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(f"[ocb build] compiled {src.name}", file=sys.stderr)
    stamp.write_text(digest)
    return obj


def build(force: bool = False, verbose: bool = True) -> Path:
    """Compile (if stale) and link the kernel library. Returns the path of the shared object."""
    BUILD_DIR.mkdir(exist_ok=True)
    if force:
        for f in BUILD_DIR.glob("*.hash"):
            f.unlink()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile_one(s, verbose), srcs))
    link_stamp = BUILD_DIR / "link.hash"
    digest = hashlib.sha256(b"".join(o.read_bytes() for o in objs)).hexdigest()
    if LIB_PATH.exists() and link_stamp.exists() and link_stamp.read_text() == digest:
        return LIB_PATH
    tmp = BUILD_DIR / (LIB_PATH.name + ".tmp")  # linked aside and renamed: a reader never sees a half-written library
    cmd = [_nvcc(), "-shared", "-cudart", "shared", "-o", str(tmp), *map(str, objs)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, LIB_PATH)
    link_stamp.write_text(digest)
    if verbose:
        print(f"[ocb build] linked {LIB_PATH}", file=sys.stderr)
    return LIB_PATH


NATIVE_SRC_DIR = OPS_DIR.parent / "nn" / "_csrc"
NATIVE_LIB_PATH = OPS_DIR.parent / "nn" / "libocb_native.so"


def build_native(force: bool = False, verbose: bool = True) -> Path:
    """
    Compile the host-side C++ helpers that need PyTorch's headers (``nn/_csrc/*.cpp``: the storage rebinding used by
    ``OutputDiscardCheckpoint``) into ``nn/libocb_native.so``. They register dispatcher ops (``torch.ops.ocb_native.*``)
    and are loaded with ``torch.ops.load_library``.
    """
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths

    BUILD_DIR.mkdir(exist_ok=True)
    srcs = sorted(NATIVE_SRC_DIR.glob("*.cpp"))
    h = hashlib.sha256(torch.__version__.encode())
    for src in srcs:
        h.update(src.read_bytes())
    stamp = BUILD_DIR / "native.hash"
    if not force and NATIVE_LIB_PATH.exists() and stamp.exists() and stamp.read_text() == h.hexdigest():
        return NATIVE_LIB_PATH
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", *map(str, srcs), "-o", str(NATIVE_LIB_PATH)]
    for inc in include_paths():
        cmd += ["-isystem", inc]
    for lib_dir in library_paths():
        cmd += [f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}"]
    cmd += ["-ltorch", "-ltorch_cpu", "-lc10"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"native helper build failed:\n{proc.stdout}\n{proc.stderr}")
    stamp.write_text(h.hexdigest())
    if verbose:
        print(f"[ocb build] linked {NATIVE_LIB_PATH}", file=sys.stderr)
    return NATIVE_LIB_PATH


def is_built() -> bool:
    return LIB_PATH.exists()


def main(argv: Optional[List[str]] = None) -> None:
    argv = sys.argv[1:] if argv is None else argv
    build(force="--force" in argv)
    build_native(force="--force" in argv)


if __name__ == "__main__":
    main()
