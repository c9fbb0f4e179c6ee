"""Helpers shared by the tests: turn the harness's input tuples into the plain arrays the CPU oracle takes."""
from __future__ import annotations

import numpy as np
import torch


def operand_np(t: torch.Tensor) -> np.ndarray:
    """``[rows, K/2, L]`` packed operand -> ``[L, rows, K/2]`` uint8."""
    return t.view(torch.uint8).permute(2, 0, 1).contiguous().cpu().numpy()


def scales_np(p: torch.Tensor) -> np.ndarray:
    """6-D swizzled view ``[32,4,R,4,Kb,L]`` -> flat buffer bytes in memory order."""
    return p.view(torch.uint8).permute(5, 2, 4, 0, 1, 3).contiguous().cpu().numpy().reshape(-1)


def out_np(c: torch.Tensor) -> np.ndarray:
    """``[M, N, L]`` output -> ``[L, M, N]`` float16."""
    return c.permute(2, 0, 1).contiguous().cpu().numpy()


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
