"""Build and load ``libnvfp4_b200.so`` (the C ABI declared in ``include/nvfp4_b200.h``)."""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

_PKG = Path(__file__).resolve().parent
CSRC = _PKG / "csrc"
BUILT_SO = _PKG / "libnvfp4_b200.so"     # what build() makes
# what load() opens: NVFP4_B200_LIB names another build of the library (an instrumented one, say)
SO_PATH = Path(os.environ["NVFP4_B200_LIB"]).resolve() if os.environ.get("NVFP4_B200_LIB") else BUILT_SO
HEADER = _PKG.parent / "include" / "nvfp4_b200.h"

NVCC_FLAGS = [
    "-O3", "-std=c++17", "--threads", "4", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared", "--cudart=static",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not BUILT_SO.exists():
        return True
    t = BUILT_SO.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [HEADER]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel for sm_100a into one shared library next to this file (nvcc cross-compiles
    without a GPU)."""
    if not force and not _stale():
        return BUILT_SO
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(BUILT_SO), *map(str, sources())]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return BUILT_SO


class Group(ctypes.Structure):
    """Mirror of ``nvfp4_group_t``."""
    _fields_ = [("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("sfa_sw", ctypes.c_void_p),
                ("sfb_sw", ctypes.c_void_p), ("c", ctypes.c_void_p),
                ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("reserved", ctypes.c_int)]


_lib = None


def load() -> ctypes.CDLL:
    """Load the library; raises if it has not been built (there is no fallback path)."""
    global _lib
    if _lib is not None:
        return _lib
    if not SO_PATH.exists():
        raise RuntimeError(f"{SO_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                           "(the NVFP4 ops have no fallback implementation)")
    lib = ctypes.CDLL(str(SO_PATH))
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.nvfp4_gemv.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, f, vp]
    lib.nvfp4_gemm.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, f, vp]
    lib.nvfp4_dual_gemm.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, f, vp]
    lib.nvfp4_dual_gemm_nvfp4.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, f, vp]
    pp = ctypes.POINTER(ctypes.c_void_p)
    lib.nvfp4_gemm_allgather.argtypes = [vp, vp, vp, vp, pp, i, i, i, i, i, i, f, vp]
    lib.nvfp4_dual_gemm_allgather.argtypes = [vp, vp, vp, vp, vp, vp, pp, i, i, i, i, i, i, f, vp]
    lib.nvfp4_grouped_gemm.argtypes = [ctypes.POINTER(Group), i, f, vp]
    lib.nvfp4_grouped_gemm_noalloc.argtypes = [ctypes.POINTER(Group), i, f, vp]
    for q in (lib.nvfp4_quantize_f32, lib.nvfp4_quantize_f16, lib.nvfp4_quantize_bf16):
        q.argtypes = [vp, vp, vp, i, i, i, vp]
    lib.nvfp4_device_status.argtypes = [i, i]
    lib.nvfp4_wait_selftest.argtypes = [i, ctypes.POINTER(ctypes.c_double), vp]
    lib.nvfp4_strerror.argtypes = [i]
    lib.nvfp4_strerror.restype = ctypes.c_char_p
    for name in ("nvfp4_gemv", "nvfp4_gemm", "nvfp4_dual_gemm", "nvfp4_dual_gemm_nvfp4", "nvfp4_gemm_allgather", "nvfp4_dual_gemm_allgather", "nvfp4_grouped_gemm", "nvfp4_grouped_gemm_noalloc", "nvfp4_quantize_f32", "nvfp4_quantize_f16", "nvfp4_quantize_bf16", "nvfp4_device_status",
                 "nvfp4_wait_selftest", "nvfp4_abi_version", "nvfp4_shutdown"):
        getattr(lib, name).restype = i
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().nvfp4_strerror(code).decode()


def check(code: int, what: str) -> None:
    """Raise like the reference's kernels do (a Python exception fails the test, eval_base.py:224-225)."""
    if code != 0:
        raise RuntimeError(f"{what} failed: [{code}] {strerror(code)}")


def device_status(dev: int, clear: bool = True) -> int:
    return int(load().nvfp4_device_status(dev, 1 if clear else 0))
