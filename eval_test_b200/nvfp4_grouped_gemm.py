"""Drop-in for the reference's grouped-GEMM entry point (eval/nvfp4_grouped_gemm/submission.py:1196-1237).

``custom_kernel(data)`` takes the 4-tuple of eval/nvfp4_grouped_gemm/reference.py:137-201 -
``(abc_tensors, sfasfb_tensors, sfasfb_reordered_tensors, problem_sizes)``, one entry per group, L = 1 - runs all
groups in ONE persistent launch over a device-side problem table and returns the list of output tensors
``[m_g, n_g, 1]`` (written in place).  Ragged M (any m_g >= 0, empty groups included) is handled by TMA zero fill
and predicated stores; the reference kernel drops the rows beyond the last multiple of 128
(``tiles_m = M / BLOCK_M``, submission.py:1095).
"""
from __future__ import annotations

import torch

from . import _args, _lib


def compile_kernel():
    return _lib.load()


# Validated descriptor arrays of recent calls.  The harness calls ``custom_kernel`` with the same ``data`` object
# over and over; re-validating 5 tensors per group costs more host time than the kernel runs for.  An entry is
# reused only while everything the descriptors were built from is unchanged: the list object (its id, confirmed
# by a weak reference to the first output tensor, so a recycled id cannot match), every operand, scale and output
# pointer, and the problem sizes.  Nothing is kept alive: the cache holds pointers and weak references only.
import weakref

_CACHE: dict = {}
_CACHE_MAX = 64


def _fingerprint(abc_tensors, sf_reordered, problem_sizes):
    ptrs = tuple(t.data_ptr() for abc in abc_tensors for t in abc)
    sf_ptrs = tuple(t.data_ptr() for pair in sf_reordered for t in pair)
    return ptrs, sf_ptrs, tuple(tuple(int(v) for v in s) for s in problem_sizes)


def _build(abc_tensors, sf_reordered, problem_sizes):
    g = len(abc_tensors)
    groups = (_lib.Group * g)()
    outs = []
    for i, ((a, b, c), (sfa_p, sfb_p), (m, n, k, l)) in enumerate(zip(abc_tensors, sf_reordered, problem_sizes)):
        if l != 1:
            raise ValueError("grouped GEMM: every group must have l == 1")
        k2 = k // 2
        q = groups[i]
        q.M, q.N, q.K = int(m), int(n), int(k)
        if m > 0:
            q.a = _args.operand_ptr(a, m, k2, 1, f"a[{i}]")
            q.sfa_sw = _args.scales_ptr(sfa_p, m, k, 1, f"sfa_reordered[{i}]")
            q.c = _args.output_ptr(c, m, n, 1, f"c[{i}]")
        q.b = _args.operand_ptr(b, n, k2, 1, f"b[{i}]")
        q.sfb_sw = _args.scales_ptr(sfb_p, n, k, 1, f"sfb_reordered[{i}]")
        outs.append(c)
    return groups, outs


def custom_kernel(data, alpha: float = 1.0):
    abc_tensors, _, sf_reordered, problem_sizes = data
    g = len(abc_tensors)
    if g == 0:
        return []
    device = abc_tensors[0][2].device
    fp = _fingerprint(abc_tensors, sf_reordered, problem_sizes)
    key = id(abc_tensors)
    ent = _CACHE.get(key)
    if ent is not None and ent[0]() is abc_tensors[0][2] and ent[1] == fp:
        groups = ent[2]
    else:
        groups, _ = _build(abc_tensors, sf_reordered, problem_sizes)
        _CACHE.pop(key, None)
        if len(_CACHE) >= _CACHE_MAX:
            _CACHE.pop(next(iter(_CACHE)))
        _CACHE[key] = (weakref.ref(abc_tensors[0][2]), fp, groups)
    with torch.cuda.device(device):
        code = _lib.load().nvfp4_grouped_gemm(groups, g, float(alpha), _args.stream_ptr(device))
    _lib.check(code, "nvfp4_grouped_gemm")
    return [c for (_, _, c) in abc_tensors]
