"""Helpers shared by the tests: turn the harness's input tuples into the plain arrays the CPU oracle takes."""
from __future__ import annotations

import torch

from eval_test_b200.hostviews import operand_np, out_np, scales_np  # noqa: F401  (re-exported for the tests)


def to_device(data, device="cuda"):
    """Move a (nested) input tuple; the permuted views are dense, so ``.to`` keeps their strides."""
    if isinstance(data, torch.Tensor):
        out = data.to(device)
        assert out.numel() == 0 or out.stride() == data.stride(), (out.stride(), data.stride())
        return out
    if isinstance(data, (list, tuple)):
        return type(data)(to_device(x, device) for x in data)
    return data


def gemm_oracle_args(data):
    a, b, _, _, sfa_p, sfb_p, _ = data
    return operand_np(a), operand_np(b), scales_np(sfa_p), scales_np(sfb_p)


def dual_oracle_args(data):
    a, b1, b2, _, _, _, sfa_p, sfb1_p, sfb2_p, _ = data
    return (operand_np(a), operand_np(b1), operand_np(b2), scales_np(sfa_p), scales_np(sfb1_p), scales_np(sfb2_p))


def grouped_oracle_args(data):
    abc, _, sfs_p, _ = data
    return [(operand_np(a)[0], operand_np(b)[0], scales_np(sa), scales_np(sb))
            for (a, b, _), (sa, sb) in zip(abc, sfs_p)]
