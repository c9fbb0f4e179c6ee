"""GPU quantiser: fp32 / fp16 / bf16 -> packed e2m1 + swizzled e4m3 block scales in one launch (``nvfp4_quantize_f32``).

``quantize_operand(x)`` returns exactly the three tensors of one operand of the kernels' input tuples, bit for bit
what ``formats.quantize_nvfp4`` + ``formats.swizzle_scales`` produce with torch ops.
"""
from __future__ import annotations

import torch

from . import _lib, formats as F


def quantize_operand(x: torch.Tensor, ref_scales: bool = True):
    """x: CUDA fp32, fp16 or bf16 ``[L, rows, K]`` (contiguous) -> (operand ``[rows, K/2, L]`` float4_e2m1fn_x2,
    row-major scales ``[rows, K/16, L]`` float8_e4m3fn, 6-D swizzled view).

    The row-major scales are what the reference's tuples carry for its own checker; the kernels read only the
    swizzled buffer.  ``ref_scales=False`` skips the torch gather that rebuilds them (the second entry is None)."""
    entry = {torch.float32: "nvfp4_quantize_f32", torch.float16: "nvfp4_quantize_f16",
             torch.bfloat16: "nvfp4_quantize_bf16"}.get(x.dtype)
    if not (x.is_cuda and entry and x.dim() == 3 and x.is_contiguous()):
        raise ValueError("quantize_operand: expected a contiguous CUDA float32 / float16 / bfloat16 tensor [L, rows, K]")
    L, rows, K = x.shape
    packed = torch.empty((L, rows, K // 2), dtype=torch.uint8, device=x.device)
    buf = torch.empty(F.sf_buffer_bytes(rows, K, L), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        code = getattr(_lib.load(), entry)(x.data_ptr(), packed.data_ptr(), buf.data_ptr(), rows, K, L,
                                           torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(code, entry)
    sf = F.batch_last(F.unswizzle_scales(buf, rows, K, L)).view(torch.float8_e4m3fn) if ref_scales else None
    return (F.batch_last(packed).view(torch.float4_e2m1fn_x2), sf, F.permuted_view(buf, rows, K, L))
