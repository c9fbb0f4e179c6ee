"""Plain host arrays of the harness's tensors, in memory order: what a CPU routine, a file or a copy loop takes.
(The harness's tensors are batch-last *views*: ``[rows, K/2, L]`` over ``[L][rows][K/2]`` bytes, and 6-D swizzled
scale views over flat atom buffers; eval/nvfp4_gemm/reference.py:35-46, eval/common/scale_helpers.py:41-68.)"""
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
