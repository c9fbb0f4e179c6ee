"""NVFP4 number formats and layouts on the host side (encode direction): the block-16 quantiser, nibble
packing and the swizzled scale-factor layout.  Everything is plain torch ops, so it runs on CPU or on the GPU.

Formats: e2m1 nibble ``s e1 e0 m`` with magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}; element ``2i`` sits in bits
3..0 of byte ``i`` and element ``2i+1`` in bits 7..4; one e4m3fn scale per 16 consecutive K elements of a row
(block size as in eval/common/scale_helpers.py:3).  Scale layout: see ``swizzle_scales``.
"""
from __future__ import annotations

import torch

SF_VEC = 16
E2M1_MAX = 6.0
E4M3_MAX = 448.0


def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def sf_buffer_bytes(rows: int, K: int, L: int = 1) -> int:
    """Bytes of the swizzled scale buffer of a ``rows x K`` operand with ``L`` batches."""
    return L * ceil_div(rows, 128) * ceil_div(K // SF_VEC, 4) * 512


def round_to_e2m1_code(y: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even onto the e2m1 grid, saturating at +-6; returns uint8 codes ``s e1 e0 m``."""
    m = y.abs()
    code = ((m > 0.25).to(torch.uint8) + (m >= 0.75).to(torch.uint8) + (m > 1.25).to(torch.uint8)
            + (m >= 1.75).to(torch.uint8) + (m > 2.5).to(torch.uint8) + (m >= 3.5).to(torch.uint8)
            + (m > 5.0).to(torch.uint8))
    sign = torch.signbit(y).to(torch.uint8) << 3   # a negative value that rounds to zero keeps its sign (-0)
    return code | sign


def pack_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """``[..., K]`` uint8 codes -> ``[..., K/2]`` bytes (even element in the low nibble)."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()


def quantize_nvfp4(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``[..., K]`` -> (packed e2m1 ``[..., K/2]`` uint8, e4m3fn scale bits ``[..., K/16]`` uint8).

    Per 16-element block: scale = amax/6 rounded to e4m3 (RNE, clamped to 448), values = RNE(x / scale) on
    the e2m1 grid; a zero scale gives zero values.  Both divisions are done as products with a correctly rounded
    fp32 reciprocal - amax * fl32(1/6) and x * fl32(1/scale) - which gives the same bits on CPU, on CUDA and in
    the ``nvfp4_quantize_f32`` kernel (where an IEEE division per element would make the kernel compute-bound).
    """
    K = x.shape[-1]
    assert K % SF_VEC == 0
    xb = x.float().reshape(*x.shape[:-1], K // SF_VEC, SF_VEC)
    amax = xb.abs().amax(dim=-1)
    sf = (amax * (1.0 / E2M1_MAX)).clamp(max=E4M3_MAX).to(torch.float8_e4m3fn)
    s32 = sf.float().unsqueeze(-1)
    y = torch.where(s32 > 0, xb * torch.reciprocal(s32), torch.zeros_like(xb))
    codes = round_to_e2m1_code(y).reshape(*x.shape[:-1], K)
    return pack_e2m1(codes), sf.view(torch.uint8)


def swizzle_scales(sf: torch.Tensor, pad: torch.Tensor | None = None) -> torch.Tensor:
    """Row-major scale bytes ``[L, rows, K/16]`` (uint8) -> flat swizzled buffer.

    Layout (that of the reference's ``*_permuted`` tensors, eval/common/scale_helpers.py:41-68): 512-byte
    atoms of 128 rows x 4 k-blocks, ordered ``[L][ceil(rows/128)][ceil(K/64)]``; inside an atom the scale of
    row ``r`` and k-block ``kb`` is byte ``(r%32)*16 + ((r%128)//32)*4 + kb%4``.  Rows / k-blocks beyond the
    operand are filled from ``pad`` (a full ``[L, R*128, Kb*4]`` tensor) or with zeros.
    """
    assert sf.dtype == torch.uint8 and sf.dim() == 3
    L, rows, kbs = sf.shape
    R, Kb = ceil_div(rows, 128), ceil_div(kbs, 4)
    full = torch.zeros((L, R * 128, Kb * 4), dtype=torch.uint8, device=sf.device) if pad is None else pad.clone()
    assert full.shape == (L, R * 128, Kb * 4)
    full[:, :rows, :kbs] = sf
    # r = rb*128 + g*32 + i ; kb = q*4 + kk  ->  [L][rb][q][i][g][kk]
    return full.view(L, R, 4, 32, Kb, 4).permute(0, 1, 4, 3, 2, 5).contiguous().view(-1)


def unswizzle_scales(buf: torch.Tensor, rows: int, K: int, L: int) -> torch.Tensor:
    """Inverse of ``swizzle_scales`` (drops the padding): flat buffer -> ``[L, rows, K/16]`` uint8."""
    kbs = K // SF_VEC
    R, Kb = ceil_div(rows, 128), ceil_div(kbs, 4)
    t = buf.view(torch.uint8).reshape(L, R, Kb, 32, 4, 4).permute(0, 1, 4, 3, 2, 5).reshape(L, R * 128, Kb * 4)
    return t[:, :rows, :kbs].contiguous()


def permuted_view(buf: torch.Tensor, rows: int, K: int, L: int) -> torch.Tensor:
    """The 6-D ``[32, 4, R, 4, Kb, L]`` float8_e4m3fn view the reference passes to kernels
    (``mma_permute_order`` of eval/common/scale_helpers.py:52-55), aliasing the flat swizzled buffer."""
    R, Kb = ceil_div(rows, 128), ceil_div(K // SF_VEC, 4)
    assert buf.numel() == L * R * Kb * 512
    return torch.as_strided(buf.view(torch.float8_e4m3fn), (32, 4, R, 4, Kb, L),
                            (16, 4, Kb * 512, 1, 512, R * Kb * 512))


def permuted_strides(rows: int, K: int) -> tuple[int, ...]:
    R, Kb = ceil_div(rows, 128), ceil_div(K // SF_VEC, 4)
    return (16, 4, Kb * 512, 1, 512, R * Kb * 512)


def batch_last(t: torch.Tensor) -> torch.Tensor:
    """``[L, rows, cols]`` contiguous -> the reference's ``[rows, cols, L]`` view (batch outermost in memory)."""
    return t.permute(1, 2, 0)
