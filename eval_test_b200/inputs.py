"""Seeded input generators for the four problems.

Two families:

* ``*_reference_style``: the value distributions of the harness's own generators - random bit patterns and
  small dyadic scales, chosen so that fp32 accumulation is exact
  (GEMM eval/nvfp4_gemm/reference.py:31-46, GEMV eval/nvfp4_gemv/reference.py:31-49, dual GEMM
  eval/nvfp4_dual_gemm/reference.py:48-73, grouped GEMM eval/nvfp4_grouped_gemm/reference.py:137-201).
  The reference draws on the CUDA generator; here the draw comes from a ``torch.Generator`` on the requested
  device, so the same seed gives the same tensors on any machine when ``device="cpu"``.
* ``*_quantized``: N(0,1) fp32 data pushed through the block-16 quantiser (``formats.quantize_nvfp4``).

Both return the reference's input tuples: packed operands ``[rows, K/2, L]`` (``float4_e2m1fn_x2``, batch
outermost in memory), row-major reference scales ``[rows, K/16, L]`` (``float8_e4m3fn``), the 6-D swizzled
``*_permuted`` views, and a pre-allocated fp16 output ``[M, N, L]`` filled with noise.
"""
from __future__ import annotations

import numpy as np
import torch

from . import formats as F

FP4X2 = torch.float4_e2m1fn_x2
E4M3 = torch.float8_e4m3fn


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def _operand(bytes_lrc: torch.Tensor) -> torch.Tensor:
    return F.batch_last(bytes_lrc.contiguous()).view(FP4X2)


def _out(L, M, N, g, device) -> torch.Tensor:
    c = torch.randn((L, M, N), generator=g, device=device, dtype=torch.float32).to(torch.float16)
    return F.batch_last(c)


def _scales_from_values(vals_full: torch.Tensor, rows: int, kbs: int):
    """vals_full: float32 ``[L, R*128, Kb*4]`` (padding included) -> (ref [rows, kbs, L] e4m3, permuted 6-D view)."""
    L = vals_full.shape[0]
    bits_full = vals_full.to(E4M3).view(torch.uint8)
    ref = bits_full[:, :rows, :kbs].contiguous()
    buf = F.swizzle_scales(ref, pad=bits_full)
    return F.batch_last(ref).view(E4M3), F.permuted_view(buf, rows, kbs * F.SF_VEC, L)


def _int_scales(L, rows, K, lo, hi, g, device):
    kbs = K // F.SF_VEC
    R, Kb = F.ceil_div(rows, 128), F.ceil_div(kbs, 4)
    v = torch.randint(lo, hi, (L, R * 128, Kb * 4), generator=g, device=device).float()
    return _scales_from_values(v, rows, kbs)


def _uniform_scales(L, rows, K, g, device):
    kbs = K // F.SF_VEC
    R, Kb = F.ceil_div(rows, 128), F.ceil_div(kbs, 4)
    v = torch.rand((L, R * 128, Kb * 4), generator=g, device=device, dtype=torch.float32)
    return _scales_from_values(v, rows, kbs)


def _rand_bytes(L, rows, K, g, device, lo=0, hi=256, mask=0xFF):
    b = torch.randint(lo, hi, (L, rows, K // 2), generator=g, device=device, dtype=torch.int16)
    return (b & mask).to(torch.uint8)


# ------------------------------------------------------------------------------------------ reference style
def gemm_reference_style(m: int, n: int, k: int, l: int, seed: int, device="cuda"):
    """All 256 byte patterns, scales in {0,1,2,3}."""
    g = _gen(seed, device)
    a = _operand(_rand_bytes(l, m, k, g, device))
    b = _operand(_rand_bytes(l, n, k, g, device))
    c = _out(l, m, n, g, device)
    sfa, sfa_p = _int_scales(l, m, k, 0, 4, g, device)
    sfb, sfb_p = _int_scales(l, n, k, 0, 4, g, device)
    return (a, b, sfa, sfb, sfa_p, sfb_p, c)


def gemv_reference_style(m: int, k: int, l: int, seed: int, device="cuda"):
    """Bytes in {0..3} (odd-k elements are zero), scales in {0,1,2}; the vector operand has 128 rows."""
    g = _gen(seed, device)
    a = _operand(_rand_bytes(l, m, k, g, device, 0, 4))
    b = _operand(_rand_bytes(l, 128, k, g, device, 0, 4))
    c = _out(l, m, 1, g, device)
    sfa, sfa_p = _int_scales(l, m, k, 0, 3, g, device)
    sfb, sfb_p = _int_scales(l, 128, k, 0, 3, g, device)
    return (a, b, sfa, sfb, sfa_p, sfb_p, c)


def dual_gemm_reference_style(m: int, n: int, k: int, l: int, seed: int, device="cuda"):
    """Bytes masked with 0xBB (|v| <= 1.5), scales U[0,1) rounded to e4m3."""
    g = _gen(seed, device)
    a = _operand(_rand_bytes(l, m, k, g, device, 0, 255, 0xBB))
    b1 = _operand(_rand_bytes(l, n, k, g, device, 0, 255, 0xBB))
    b2 = _operand(_rand_bytes(l, n, k, g, device, 0, 255, 0xBB))
    c = _out(l, m, n, g, device)
    sfa, sfa_p = _uniform_scales(l, m, k, g, device)
    sfb1, sfb1_p = _uniform_scales(l, n, k, g, device)
    sfb2, sfb2_p = _uniform_scales(l, n, k, g, device)
    return (a, b1, b2, sfa, sfb1, sfb2, sfa_p, sfb1_p, sfb2_p, c)


def grouped_gemm_reference_style(m, n, k, g: int, seed: int, device="cuda"):
    """Per group: bytes masked with 0xBB, scales in {1,2} (padding rows of the swizzled buffers too)."""
    gen = _gen(seed, device)
    abc, sfs, sfs_p, sizes = [], [], [], []
    for gi in range(g):
        mi, ni, ki = int(m[gi]), int(n[gi]), int(k[gi])
        a = _operand(_rand_bytes(1, mi, ki, gen, device, 0, 255, 0xBB))
        b = _operand(_rand_bytes(1, ni, ki, gen, device, 0, 255, 0xBB))
        c = _out(1, mi, ni, gen, device)
        sfa, sfa_p = _int_scales(1, mi, ki, 1, 3, gen, device)
        sfb, sfb_p = _int_scales(1, ni, ki, 1, 3, gen, device)
        abc.append((a, b, c))
        sfs.append((sfa, sfb))
        sfs_p.append((sfa_p, sfb_p))
        sizes.append((mi, ni, ki, 1))
    return (abc, sfs, sfs_p, sizes)


# ------------------------------------------------------------------------------------------ N(0,1) -> quantiser
def quantized_operand(L: int, rows: int, K: int, gen: torch.Generator, device, zero_rows_from: int | None = None):
    """N(0,1) ``[L, rows, K]`` -> (operand [rows,K/2,L], ref scales [rows,K/16,L], permuted view).
    Generated one batch at a time to bound temporary memory."""
    packed = torch.empty((L, rows, K // 2), dtype=torch.uint8, device=device)
    sf = torch.empty((L, rows, K // F.SF_VEC), dtype=torch.uint8, device=device)
    for l in range(L):
        x = torch.randn((rows, K), generator=gen, device=device, dtype=torch.float32)
        if zero_rows_from is not None:
            x[zero_rows_from:] = 0
        packed[l], sf[l] = F.quantize_nvfp4(x)
        del x
    buf = F.swizzle_scales(sf)
    return _operand(packed), F.batch_last(sf).view(E4M3), F.permuted_view(buf, rows, K, L)


def gemm_quantized(m: int, n: int, k: int, l: int, seed: int, device="cuda"):
    g = _gen(seed, device)
    a, sfa, sfa_p = quantized_operand(l, m, k, g, device)
    b, sfb, sfb_p = quantized_operand(l, n, k, g, device)
    return (a, b, sfa, sfb, sfa_p, sfb_p, _out(l, m, n, g, device))


def gemv_quantized(m: int, k: int, l: int, seed: int, device="cuda"):
    """The vector is row 0 of a 128-row operand whose other rows are zero."""
    g = _gen(seed, device)
    a, sfa, sfa_p = quantized_operand(l, m, k, g, device)
    b, sfb, sfb_p = quantized_operand(l, 128, k, g, device, zero_rows_from=1)
    return (a, b, sfa, sfb, sfa_p, sfb_p, _out(l, m, 1, g, device))


def dual_gemm_quantized(m: int, n: int, k: int, l: int, seed: int, device="cuda"):
    g = _gen(seed, device)
    a, sfa, sfa_p = quantized_operand(l, m, k, g, device)
    b1, sfb1, sfb1_p = quantized_operand(l, n, k, g, device)
    b2, sfb2, sfb2_p = quantized_operand(l, n, k, g, device)
    return (a, b1, b2, sfa, sfb1, sfb2, sfa_p, sfb1_p, sfb2_p, _out(l, m, n, g, device))


def poisson_group_sizes(g: int, mean: float, lo: int, hi: int, seed: int) -> list[int]:
    """Per-group M ~ Poisson(mean) clipped to [lo, hi], from ``numpy.random.default_rng(seed)``."""
    return [int(v) for v in np.clip(np.random.default_rng(seed).poisson(mean, g), lo, hi)]


def grouped_gemm_quantized(m, n, k, g: int, seed: int, device="cuda"):
    """Groups with ``m[i] == 0`` are empty: zero-row operands and outputs."""
    gen = _gen(seed, device)
    abc, sfs, sfs_p, sizes = [], [], [], []
    for gi in range(g):
        mi, ni, ki = int(m[gi]), int(n[gi]), int(k[gi])
        a, sfa, sfa_p = quantized_operand(1, mi, ki, gen, device)
        b, sfb, sfb_p = quantized_operand(1, ni, ki, gen, device)
        abc.append((a, b, _out(1, mi, ni, gen, device)))
        sfs.append((sfa, sfb))
        sfs_p.append((sfa_p, sfb_p))
        sizes.append((mi, ni, ki, 1))
    return (abc, sfs, sfs_p, sizes)
