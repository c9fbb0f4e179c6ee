"""Drop-in for the reference's GEMM entry point (eval/nvfp4_gemm/submission.py:708-761).

``custom_kernel(data)`` takes ``(a, b, sfa_ref, sfb_ref, sfa_permuted, sfb_permuted, c)`` as produced by
eval/nvfp4_gemm/reference.py:31-46, writes ``c[m, n, l] = fp16(alpha * sum_k (a*sfa)(b*sfb))`` in place on the
current stream and returns ``c``.  ``alpha`` is an optional fp32 global scale (the reference has none: 1.0).
``compile_kernel()`` exists because the harness calls it when present (eval/nvfp4_gemm/eval.py:23-40); the
kernels are compiled ahead of time, so it only loads the library.
"""
from __future__ import annotations

import torch

from . import _args, _lib


def compile_kernel():
    return _lib.load()


def custom_kernel(data, alpha: float = 1.0):
    a, b, _, _, sfa_p, sfb_p, c = data
    tensors = (a, b, sfa_p, sfb_p, c)
    ent = _args.lookup(data, tensors)
    if ent is None:
        m, k2, l = a.shape
        n = b.shape[0]
        k = 2 * k2
        ent = _args.remember(data, tensors, (
            _args.operand_ptr(a, m, k2, l, "a"), _args.operand_ptr(b, n, k2, l, "b"),
            _args.scales_ptr(sfa_p, m, k, l, "sfa_permuted"), _args.scales_ptr(sfb_p, n, k, l, "sfb_permuted"),
            _args.output_ptr(c, m, n, l), m, n, k, l))
    code = _args.launch(_lib.load().nvfp4_gemm, ent, float(alpha))
    if code:
        _lib.check(code, "nvfp4_gemm")
    return c
