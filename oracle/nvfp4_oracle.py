"""CPU oracle for the NVFP4 hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Two independent restatements of what the reference computes:

* ``c_*``  : ctypes bindings of ``nvfp4_oracle.c`` (exact integer block dot
  products, fp32 accumulation, OpenMP over rows).  Fast enough to be the timed
  CPU baseline.
* ``np_*`` : a numpy/torch-CPU "dequantise, then fp32 matmul" version written
  separately (table decode, fancy-index un-swizzle, ``torch.matmul``), i.e. the
  shape of computation the reference's oracle has on the GPU
  (eval/nvfp4_gemm/reference.py:16-27: ``_scaled_mm(a, b.T, to_blocked(sfa),
  to_blocked(sfb))``).

Only ``tests/``, the smoke check and the CPU-baseline / reference legs of the
bench may import this module.  The reference holds no stored golden vectors
for this path; the pins are the fixtures under ``tests/golden/`` (scale layout
from the reference's own ``to_blocked``; ``torch._scaled_mm`` outputs recorded
on a B200).

All functions take and return numpy arrays with the reference's memory
layouts: operands ``[L, rows, K/2]`` uint8 (two e2m1 per byte, element 2i in
the low nibble), scales as the flat swizzled byte buffer, outputs
``[L, M, N]`` float16.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "nvfp4_oracle.c"


def _cpu_tag() -> str:
    """The library is compiled with -march=native, so its file name carries a hash of this host's CPU
    flags: a prebuilt file brought over from another machine is not picked up by mistake."""
    import hashlib
    try:
        flags = next(l for l in open("/proc/cpuinfo") if l.startswith("flags"))
    except (OSError, StopIteration):
        flags = "unknown"
    return hashlib.sha1(flags.encode()).hexdigest()[:10]


_SO = _HERE / "_build" / f"libnvfp4_oracle.{_cpu_tag()}.so"

SF_VEC = 16
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                        -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def build(force: bool = False) -> Path:
    """Compile nvfp4_oracle.c into oracle/_build/ (gcc, OpenMP)."""
    if _SO.exists() and not force and _SO.stat().st_mtime >= _SRC.stat().st_mtime:
        return _SO
    _SO.parent.mkdir(exist_ok=True)
    cmd = ["gcc", "-O3", "-march=native", "-fopenmp", "-shared", "-fPIC", str(_SRC), "-o", str(_SO), "-lm"]
    try:
        subprocess.run(cmd, check=True, capture_output=True)
    except subprocess.CalledProcessError:
        cmd.remove("-march=native")
        subprocess.run(cmd, check=True)
    return _SO


_lib = None


def _load():
    global _lib
    if _lib is None:
        if not _SO.exists():
            build()
        lib = ctypes.CDLL(str(_SO))
        u8p, u16p = ctypes.c_void_p, ctypes.c_void_p
        i, f = ctypes.c_int, ctypes.c_float
        lib.oracle_gemm.argtypes = [u8p, u8p, u8p, u8p, u16p, i, i, i, i, f]
        lib.oracle_dual_gemm.argtypes = [u8p, u8p, u8p, u8p, u8p, u8p, u16p, i, i, i, i, f]
        lib.oracle_gemv.argtypes = [u8p, u8p, u8p, u8p, u16p, i, i, i, i, f]
        lib.oracle_sf_offset.argtypes = [i, i, i, i, i]
        lib.oracle_sf_offset.restype = ctypes.c_size_t
        lib.oracle_e4m3_decode.argtypes = [ctypes.c_uint]
        lib.oracle_e4m3_decode.restype = f
        lib.oracle_e2m1_decode.argtypes = [ctypes.c_uint]
        lib.oracle_e2m1_decode.restype = f
        lib.oracle_dequant.argtypes = [u8p, u8p, ctypes.c_void_p, i, i, i]
        lib.oracle_num_threads.restype = i
        lib.oracle_set_num_threads.argtypes = [i]
        _lib = lib
    return _lib


def num_threads() -> int:
    return int(_load().oracle_num_threads())


def set_num_threads(n: int) -> None:
    _load().oracle_set_num_threads(int(n))


def _u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint8, a.dtype
    return a


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def sf_bytes(rows: int, K: int, L: int) -> int:
    """Size of a swizzled scale buffer (rows padded to 128, K/16 padded to 4)."""
    return L * ((rows + 127) // 128) * ((K // SF_VEC + 3) // 4) * 512


# --------------------------------------------------------------------------- C oracle

def c_gemm(a, b, sfa_sw, sfb_sw, alpha: float = 1.0) -> np.ndarray:
    a, b, sfa_sw, sfb_sw = _u8(a), _u8(b), _u8(sfa_sw), _u8(sfb_sw)
    L, M, K2 = a.shape
    N = b.shape[1]
    K = 2 * K2
    assert b.shape == (L, N, K2)
    assert sfa_sw.size >= sf_bytes(M, K, L) and sfb_sw.size >= sf_bytes(N, K, L)
    c = np.empty((L, M, N), dtype=np.float16)
    rc = _load().oracle_gemm(_ptr(a), _ptr(b), _ptr(sfa_sw), _ptr(sfb_sw), _ptr(c), M, N, K, L, alpha)
    assert rc == 0, rc
    return c


def c_dual_gemm(a, b1, b2, sfa_sw, sfb1_sw, sfb2_sw, alpha: float = 1.0) -> np.ndarray:
    a, b1, b2 = _u8(a), _u8(b1), _u8(b2)
    sfa_sw, sfb1_sw, sfb2_sw = _u8(sfa_sw), _u8(sfb1_sw), _u8(sfb2_sw)
    L, M, K2 = a.shape
    N = b1.shape[1]
    K = 2 * K2
    c = np.empty((L, M, N), dtype=np.float16)
    rc = _load().oracle_dual_gemm(_ptr(a), _ptr(b1), _ptr(b2), _ptr(sfa_sw), _ptr(sfb1_sw), _ptr(sfb2_sw),
                                  _ptr(c), M, N, K, L, alpha)
    assert rc == 0, rc
    return c


def c_gemv(a, x, sfa_sw, sfx_sw, alpha: float = 1.0) -> np.ndarray:
    """a [L,M,K/2]; x [L,x_rows,K/2] (row 0 is the vector) -> [L, M] float16."""
    a, x, sfa_sw, sfx_sw = _u8(a), _u8(x), _u8(sfa_sw), _u8(sfx_sw)
    L, M, K2 = a.shape
    x_rows = x.shape[1]
    K = 2 * K2
    c = np.empty((L, M), dtype=np.float16)
    rc = _load().oracle_gemv(_ptr(a), _ptr(x), _ptr(sfa_sw), _ptr(sfx_sw), _ptr(c), M, K, L, x_rows, alpha)
    assert rc == 0, rc
    return c


def c_grouped_gemm(groups, alpha: float = 1.0) -> list[np.ndarray]:
    """groups: iterable of (a [M,K/2], b [N,K/2], sfa_sw, sfb_sw); empty groups (M = 0) give [0, N]."""
    out = []
    for a, b, sfa_sw, sfb_sw in groups:
        a, b = _u8(a), _u8(b)
        if a.shape[0] == 0:
            out.append(np.empty((0, b.shape[0]), dtype=np.float16))
            continue
        out.append(c_gemm(a[None], b[None], sfa_sw, sfb_sw, alpha)[0])
    return out


# --------------------------------------------------------------------------- numpy / torch-CPU oracle

def np_e4m3_decode(byte) -> np.ndarray:
    """e4m3fn bits -> float32, by field arithmetic (no library cast)."""
    b = np.asarray(byte).astype(np.int32)
    s, e, m = (b >> 7) & 1, (b >> 3) & 15, b & 7
    v = np.where(e == 0, m.astype(np.float32) * np.float32(2.0 ** -9),
                 (8 + m).astype(np.float32) * np.exp2((e - 10).astype(np.float32)))
    v = np.where((e == 15) & (m == 7), np.float32(np.nan), v)
    return np.where(s == 1, -v, v).astype(np.float32)


def np_unpack_e2m1(p) -> np.ndarray:
    """[..., K/2] uint8 -> [..., K] float32."""
    p = np.asarray(p, dtype=np.uint8)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.float32)
    out[..., 0::2] = E2M1_VALUES[p & 0xF]
    out[..., 1::2] = E2M1_VALUES[p >> 4]
    return out


def np_unswizzle_sf(sf_sw, rows: int, K: int, L: int) -> np.ndarray:
    """Flat swizzled bytes -> [L, rows, K/16] uint8 (gather by the offset formula)."""
    sf_sw = np.asarray(sf_sw, dtype=np.uint8).reshape(-1)
    kbs = K // SF_VEC
    R, Kb = (rows + 127) // 128, (kbs + 3) // 4
    l = np.arange(L, dtype=np.int64)[:, None, None]
    r = np.arange(rows, dtype=np.int64)[None, :, None]
    kb = np.arange(kbs, dtype=np.int64)[None, None, :]
    off = (l * R * Kb * 512 + (r // 128) * Kb * 512 + (kb // 4) * 512
           + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4)
    return sf_sw[off]


def np_dequant(p, sf_sw, rows: int, K: int, L: int) -> np.ndarray:
    """Packed operand + swizzled scales -> [L, rows, K] float32."""
    v = np_unpack_e2m1(np.asarray(p).reshape(L, -1, K // 2)[:, :rows])
    sf = np_e4m3_decode(np_unswizzle_sf(sf_sw, rows, K, L))
    return (v.reshape(L, rows, K // SF_VEC, SF_VEC) * sf[..., None]).reshape(L, rows, K)


def _mm(a32: np.ndarray, b32: np.ndarray) -> np.ndarray:
    import torch
    return torch.matmul(torch.from_numpy(a32), torch.from_numpy(b32).transpose(-1, -2)).numpy()


def np_gemm(a, b, sfa_sw, sfb_sw, alpha: float = 1.0) -> np.ndarray:
    L, M, K2 = a.shape
    N, K = b.shape[1], 2 * K2
    acc = _mm(np_dequant(a, sfa_sw, M, K, L), np_dequant(b, sfb_sw, N, K, L))
    return (np.float32(alpha) * acc).astype(np.float16)


def np_dual_gemm(a, b1, b2, sfa_sw, sfb1_sw, sfb2_sw, alpha: float = 1.0) -> np.ndarray:
    import torch
    L, M, K2 = a.shape
    N, K = b1.shape[1], 2 * K2
    A = np_dequant(a, sfa_sw, M, K, L)
    r1 = torch.from_numpy(np.float32(alpha) * _mm(A, np_dequant(b1, sfb1_sw, N, K, L)))
    r2 = torch.from_numpy(np.float32(alpha) * _mm(A, np_dequant(b2, sfb2_sw, N, K, L)))
    return (torch.nn.functional.silu(r1) * r2).to(torch.float16).numpy()


def np_gemv(a, x, sfa_sw, sfx_sw, alpha: float = 1.0) -> np.ndarray:
    L, M, K2 = a.shape
    K, x_rows = 2 * K2, x.shape[1]
    A = np_dequant(a, sfa_sw, M, K, L)
    X = np_dequant(x, sfx_sw, x_rows, K, L)[:, :1]
    return (np.float32(alpha) * _mm(A, X))[:, :, 0].astype(np.float16)


# --------------------------------------------------------------------------- dequantise (C, OpenMP) + library fp32 matmul
# The fastest CPU form of the reference's "dequantise, then matmul" computation: the C dequantiser on all cores, then
# torch.matmul in fp32.  Every function returns (result, seconds dequantising, seconds in the matmul and epilogue), so
# the CPU baseline of the bench can list the two phases apart.

def c_dequant(p, sf_sw, rows: int, K: int, L: int) -> np.ndarray:
    """Packed operand + swizzled scales -> [L, rows, K] float32 (oracle_dequant in nvfp4_oracle.c)."""
    p, sf_sw = _u8(p), _u8(sf_sw)
    assert p.size == L * rows * (K // 2) and sf_sw.size >= sf_bytes(rows, K, L)
    out = np.empty((L, rows, K), dtype=np.float32)
    rc = _load().oracle_dequant(_ptr(p), _ptr(sf_sw), _ptr(out), rows, K, L)
    assert rc == 0, rc
    return out


def dq_gemm(a, b, sfa_sw, sfb_sw, alpha: float = 1.0):
    import time
    L, M, K2 = a.shape
    N, K = b.shape[1], 2 * K2
    t0 = time.perf_counter()
    A, B = c_dequant(a, sfa_sw, M, K, L), c_dequant(b, sfb_sw, N, K, L)
    t1 = time.perf_counter()
    c = (np.float32(alpha) * _mm(A, B)).astype(np.float16)
    return c, t1 - t0, time.perf_counter() - t1


def dq_dual_gemm(a, b1, b2, sfa_sw, sfb1_sw, sfb2_sw, alpha: float = 1.0):
    import time
    import torch
    L, M, K2 = a.shape
    N, K = b1.shape[1], 2 * K2
    t0 = time.perf_counter()
    A, B1, B2 = c_dequant(a, sfa_sw, M, K, L), c_dequant(b1, sfb1_sw, N, K, L), c_dequant(b2, sfb2_sw, N, K, L)
    t1 = time.perf_counter()
    r1 = torch.from_numpy(_mm(A, B1)).mul_(float(alpha))
    r2 = torch.from_numpy(_mm(A, B2)).mul_(float(alpha))
    c = torch.nn.functional.silu(r1).mul_(r2).to(torch.float16).numpy()
    return c, t1 - t0, time.perf_counter() - t1


def dq_gemv(a, x, sfa_sw, sfx_sw, alpha: float = 1.0):
    import time
    L, M, K2 = a.shape
    K, x_rows = 2 * K2, x.shape[1]
    t0 = time.perf_counter()
    A, X = c_dequant(a, sfa_sw, M, K, L), c_dequant(x, sfx_sw, x_rows, K, L)[:, :1]
    t1 = time.perf_counter()
    c = (np.float32(alpha) * _mm(A, X))[:, :, 0].astype(np.float16)
    return c, t1 - t0, time.perf_counter() - t1


def dq_grouped_gemm(groups, alpha: float = 1.0):
    out, td, tm = [], 0.0, 0.0
    for a, b, sfa_sw, sfb_sw in groups:
        a, b = _u8(a), _u8(b)
        if a.shape[0] == 0:
            out.append(np.empty((0, b.shape[0]), dtype=np.float16))
            continue
        c, d, m = dq_gemm(a[None], b[None], sfa_sw, sfb_sw, alpha)
        out.append(c[0])
        td += d
        tm += m
    return out, td, tm
