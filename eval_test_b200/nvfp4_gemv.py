"""Drop-in for the reference's GEMV entry point (eval/nvfp4_gemv/submission.py:28-54).

``custom_kernel(data)`` takes the tuple of eval/nvfp4_gemv/reference.py:31-49 -
``(a, b, sfa_ref, sfb_ref, sfa_permuted, sfb_permuted, c)`` with ``b`` the vector padded to 128 rows - writes
``c[m, 0, l]`` in place on the current stream and returns ``c``.  Unlike the reference, which re-swizzles the
row-major scales and runs a 128-column tensor-core GEMM per batch, this streams A once through a hand-written
HBM-bound kernel and reads the pre-swizzled scales directly.
"""
from __future__ import annotations

import torch

from . import _args, _lib


def custom_kernel(data, alpha: float = 1.0):
    a, b, _, _, sfa_p, sfb_p, c = data
    tensors = (a, b, sfa_p, sfb_p, c)
    ent = _args.lookup(data, tensors)
    if ent is None:
        m, k2, l = a.shape
        x_rows = b.shape[0]
        k = 2 * k2
        ent = _args.remember(data, tensors, (
            _args.operand_ptr(a, m, k2, l, "a"), _args.operand_ptr(b, x_rows, k2, l, "b"),
            _args.scales_ptr(sfa_p, m, k, l, "sfa_permuted"), _args.scales_ptr(sfb_p, x_rows, k, l, "sfb_permuted"),
            _args.output_ptr(c, m, 1, l), m, k, l, x_rows))
    code = _args.launch(_lib.load().nvfp4_gemv, ent, float(alpha))
    if code:
        _lib.check(code, "nvfp4_gemv")
    return c
