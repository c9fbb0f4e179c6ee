"""Drop-in for the reference's dual-GEMM entry point (eval/nvfp4_dual_gemm/submission.py:894-957).

``custom_kernel(data)`` takes the 10-tuple of eval/nvfp4_dual_gemm/reference.py:48-73 -
``(a, b1, b2, sfa, sfb1, sfb2, sfa_permuted, sfb1_permuted, sfb2_permuted, c)`` - and writes
``c = fp16(silu(a @ b1^T) * (a @ b2^T))`` (block-scaled products, fp32 accumulation, the gating in fp32, one
rounding) in place on the current stream.

``custom_kernel_nvfp4(data)`` runs the same product but emits the result as an NVFP4 operand (packed e2m1 +
swizzled e4m3 block scales) for the next GEMM, bit for bit what quantising the fp16 output would give; ``c`` of the
tuple is not touched.  The reference has no such entry.
"""
from __future__ import annotations

import torch

from . import _args, _lib


def compile_kernel():
    return _lib.load()


def custom_kernel(data, alpha: float = 1.0):
    a, b1, b2, _, _, _, sfa_p, sfb1_p, sfb2_p, c = data
    tensors = (a, b1, b2, sfa_p, sfb1_p, sfb2_p, c)
    ent = _args.lookup(data, tensors)
    if ent is None:
        m, k2, l = a.shape
        n = b1.shape[0]
        k = 2 * k2
        ent = _args.remember(data, tensors, (
            _args.operand_ptr(a, m, k2, l, "a"), _args.operand_ptr(b1, n, k2, l, "b1"),
            _args.operand_ptr(b2, n, k2, l, "b2"), _args.scales_ptr(sfa_p, m, k, l, "sfa_permuted"),
            _args.scales_ptr(sfb1_p, n, k, l, "sfb1_permuted"), _args.scales_ptr(sfb2_p, n, k, l, "sfb2_permuted"),
            _args.output_ptr(c, m, n, l), m, n, k, l))
    code = _args.launch(_lib.load().nvfp4_dual_gemm, ent, float(alpha))
    if code:
        _lib.check(code, "nvfp4_dual_gemm")
    return c


def custom_kernel_nvfp4(data, alpha: float = 1.0, ref_scales: bool = False):
    """-> (operand ``[M, N/2, L]`` float4_e2m1fn_x2, row-major scales or None, 6-D swizzled scale view): the
    three tensors of an A operand of the GEMM entry points (see ``quantize.quantize_operand``)."""
    from . import formats as F
    a, b1, b2, _, _, _, sfa_p, sfb1_p, sfb2_p, _ = data
    m, k2, l = a.shape
    n, k = b1.shape[0], 2 * k2
    ptrs = (_args.operand_ptr(a, m, k2, l, "a"), _args.operand_ptr(b1, n, k2, l, "b1"),
            _args.operand_ptr(b2, n, k2, l, "b2"), _args.scales_ptr(sfa_p, m, k, l, "sfa_permuted"),
            _args.scales_ptr(sfb1_p, n, k, l, "sfb1_permuted"), _args.scales_ptr(sfb2_p, n, k, l, "sfb2_permuted"))
    packed = torch.empty((l, m, n // 2), dtype=torch.uint8, device=a.device)
    # rows padded to 128 are not written by the kernel: they must read as zero
    alloc = torch.zeros if m % 128 else torch.empty
    buf = alloc(F.sf_buffer_bytes(m, n, l), dtype=torch.uint8, device=a.device)
    with torch.cuda.device(a.device):
        code = _lib.load().nvfp4_dual_gemm_nvfp4(*ptrs, packed.data_ptr(), buf.data_ptr(), m, n, k, l, float(alpha),
                                                 torch.cuda.current_stream(a.device).cuda_stream)
    _lib.check(code, "nvfp4_dual_gemm_nvfp4")
    sf = F.batch_last(F.unswizzle_scales(buf, m, n, l)).view(torch.float8_e4m3fn) if ref_scales else None
    return F.batch_last(packed).view(torch.float4_e2m1fn_x2), sf, F.permuted_view(buf, m, n, l)
