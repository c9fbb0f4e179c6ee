"""The harness's acceptance check, for runs on a GPU: each problem's reference result is what the reference's
``ref_kernel`` computes - ``torch._scaled_mm`` (cuBLASLt block-scaled FP4) fed with the row-major scales
re-swizzled per batch - compared with ``rtol = atol = 1e-3``
(eval/nvfp4_gemm/reference.py:11-28,49; eval/nvfp4_gemv/reference.py:11-28,52;
eval/nvfp4_dual_gemm/reference.py:11-45,76; eval/nvfp4_grouped_gemm/reference.py:39-74,204).

Nothing here is on the kernels' path: it is the checker a local run uses in place of the reference checkout.
The reference results are written into fresh tensors, never into ``data`` (the reference writes into ``data[-1]``,
which would overwrite the output under test).
"""
from __future__ import annotations

import torch

from . import check, formats as F

E4M3 = torch.float8_e4m3fn
FP4X2 = torch.float4_e2m1fn_x2


def _blocked(sf_ref: torch.Tensor, l: int) -> torch.Tensor:
    """``to_blocked(sf[:, :, l])``: the row-major scales of one batch in the 128x4-tile layout, zero padded."""
    return F.swizzle_scales(sf_ref[:, :, l].contiguous().view(torch.uint8)[None]).view(E4M3)


def _mm(a, b, sfa, sfb, l, out_dtype):
    return torch._scaled_mm(a[:, :, l].view(FP4X2), b[:, :, l].view(FP4X2).transpose(0, 1), _blocked(sfa, l),
                            _blocked(sfb, l), bias=None, out_dtype=out_dtype)


def ref_gemm(data) -> torch.Tensor:
    a, b, sfa, sfb, _, _, c = data
    out = torch.empty_like(c)
    for l in range(c.shape[2]):
        out[:, :, l] = _mm(a, b, sfa, sfb, l, torch.float16)
    return out


def ref_gemv(data) -> torch.Tensor:
    a, b, sfa, sfb, _, _, c = data
    out = torch.empty_like(c)
    for l in range(c.shape[2]):
        out[:, 0, l] = _mm(a, b, sfa, sfb, l, torch.float16)[:, 0]
    return out


def ref_dual_gemm(data) -> torch.Tensor:
    a, b1, b2, sfa, sfb1, sfb2, _, _, _, c = data
    out = torch.empty_like(c)
    for l in range(c.shape[2]):
        r1 = _mm(a, b1, sfa, sfb1, l, torch.float32)
        r2 = _mm(a, b2, sfa, sfb2, l, torch.float32)
        out[:, :, l] = (torch.nn.functional.silu(r1) * r2).to(torch.float16)
    return out


def ref_grouped_gemm(data) -> list[torch.Tensor]:
    abc, sfs, _, sizes = data
    outs = []
    for (a, b, c), (sfa, sfb), (m, n, k, l) in zip(abc, sfs, sizes):
        out = torch.empty_like(c)
        if m > 0:
            for li in range(l):
                out[:, :, li] = _mm(a, b, sfa.to(c.device), sfb.to(c.device), li, torch.float16)
        outs.append(out)
    return outs


REF_KERNELS = {"nvfp4_gemm": ref_gemm, "nvfp4_gemv": ref_gemv, "nvfp4_dual_gemm": ref_dual_gemm,
               "nvfp4_grouped_gemm": ref_grouped_gemm}


def check_implementation(task: str):
    """``check_implementation(data, output) -> (ok, message)`` of a task, as in the reference's reference.py."""
    return check.make_match_reference(REF_KERNELS[task], rtol=1e-3, atol=1e-3)
