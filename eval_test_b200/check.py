"""Output checkers.

``verbose_allclose`` / ``compare_nested`` / ``make_match_reference`` follow the reference's acceptance test
(eval/common/utils.py:27-60, 80-127: ``|out-ref| <= atol + rtol*|ref|`` element-wise, NaN and +-inf positions
must coincide, nested list/tuple/dict outputs compared recursively, used with rtol = atol = 1e-3,
eval/nvfp4_gemm/reference.py:49).  ``max_delta_ok`` is the looser whole-tensor bound
``max|out-ref| <= 1e-2 * max|ref|`` used for N(0,1)-quantised inputs.
"""
from __future__ import annotations

import torch


@torch.no_grad()
def verbose_allclose(received: torch.Tensor, expected: torch.Tensor, rtol=1e-5, atol=1e-8, max_print=5) -> list[str]:
    if received.shape != expected.shape:
        return ["SIZE MISMATCH"]
    r, e = received.float(), expected.float()
    bad = (r - e).abs() > atol + rtol * e.abs()
    bad |= torch.isnan(r) ^ torch.isnan(e)
    bad |= torch.isposinf(r) ^ torch.isposinf(e)
    bad |= torch.isneginf(r) ^ torch.isneginf(e)
    n = int(bad.count_nonzero())
    if n == 0:
        return []
    out = [f"Number of mismatched elements: {n}"]
    for idx in torch.nonzero(bad)[:max_print]:
        i = tuple(idx.tolist())
        out.append(f"ERROR AT {i}: {received[i]} {expected[i]}")
    if n > max_print:
        out.append(f"... and {n - max_print} more mismatched elements.")
    return out


def compare_nested(received, expected, rtol=1e-5, atol=1e-8, path: str = "") -> list[str]:
    pre = f"{path}: " if path else ""
    if isinstance(received, torch.Tensor) and isinstance(expected, torch.Tensor):
        return [pre + r for r in verbose_allclose(received, expected, rtol=rtol, atol=atol)]
    if isinstance(received, (list, tuple)) and isinstance(expected, (list, tuple)):
        if len(received) != len(expected):
            return [pre + "LENGTH MISMATCH"]
        for i, (r, e) in enumerate(zip(received, expected)):
            reasons = compare_nested(r, e, rtol, atol, f"{path}[{i}]" if path else f"[{i}]")
            if reasons:
                return reasons
        return []
    if isinstance(received, dict) and isinstance(expected, dict):
        if set(received) != set(expected):
            return [pre + "KEY MISMATCH"]
        for k in sorted(received):
            reasons = compare_nested(received[k], expected[k], rtol, atol, f"{path}.{k}" if path else str(k))
            if reasons:
                return reasons
        return []
    return [pre + "TYPE MISMATCH"]


def match_reference(data, output, reference, rtol=1e-5, atol=1e-8) -> tuple[bool, str]:
    reasons = compare_nested(output, reference(data), rtol=rtol, atol=atol)
    if reasons:
        return False, "mismatch found! custom implementation doesn't match reference: " + " ".join(reasons)
    return True, ""


def make_match_reference(reference, **kwargs):
    def wrapped(data, output):
        return match_reference(data, output, reference=reference, **kwargs)
    return wrapped


@torch.no_grad()
def max_delta_ok(received: torch.Tensor, expected: torch.Tensor, frac: float = 1e-2) -> tuple[bool, float, float]:
    """``max|out-ref| <= frac * max|ref|`` over the finite reference values; returns (ok, max delta, max |ref|).
    Where the reference overflowed fp16 (an infinity) or is NaN, the output must hold the same special value, as in
    the element-wise check (the harness compares NaN / infinity positions, eval/common/utils.py:38-48)."""
    if received.shape != expected.shape:
        return False, float("inf"), 0.0
    if received.numel() == 0:
        return True, 0.0, 0.0
    r, e = received.float(), expected.float()
    if bool((torch.isnan(r) ^ torch.isnan(e)).any()):
        return False, float("nan"), float(e.abs().max())
    special = ~torch.isfinite(e)
    if bool((special & ~torch.isnan(e) & (r != e)).any()) or bool((~torch.isfinite(r) & ~special).any()):
        return False, float("inf"), float(e[~special].abs().max()) if bool((~special).any()) else 0.0
    if not bool((~special).any()):
        return True, 0.0, 0.0
    d, m = float((r - e)[~special].abs().max()), float(e[~special].abs().max())
    return d <= frac * m, d, m
