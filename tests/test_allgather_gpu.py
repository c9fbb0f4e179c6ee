"""Fused all-gather epilogue of the N-sharded GEMM / dual GEMM.

On one GPU the "ranks" are launches that write into several full-size buffers of the same device: that exercises
everything the kernel does (column offsets, row pitch of the full C, one store per rank).  With two or more GPUs the
same entry point is driven through symmetric memory by torchrun (tests/allgather_worker.py)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _buffers(m, n, l, world):
    bufs = [torch.full((l, m, n), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
    return bufs, [b.data_ptr() for b in bufs]


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("m,n,k,l", [(256, 1024, 512, 1), (200, 512, 768, 2), (1024, 4096, 256, 1)])
def test_gemm_allgather_equals_unsharded(world, m, n, k, l):
    from eval_test_b200 import _lib, inputs, nvfp4_gemm, shard
    if (n // world) % 128:
        pytest.skip("N/world must be a multiple of 128")
    full = inputs.gemm_quantized(m, n, k, l, seed=3, device="cuda")
    want = nvfp4_gemm.custom_kernel(full, alpha=0.5).clone()
    bufs, ptrs = _buffers(m, n, l, world)
    for r in range(world):
        out = shard.GatheredOutput(m, n, l, "cuda", ptrs=ptrs, buf=bufs[r])
        shard.gemm_allgather(shard.shard_gemm(full, r, world), out, r, alpha=0.5)
    torch.cuda.synchronize()
    assert _lib.device_status(torch.cuda.current_device()) == 0
    for b in bufs:
        assert torch.equal(b.permute(1, 2, 0).view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("world", [2, 7])
def test_dual_gemm_allgather_equals_unsharded(world):
    from eval_test_b200 import inputs, nvfp4_dual_gemm, shard
    m, n, k, l = 384, 128 * world * 2, 512, 1
    full = inputs.dual_gemm_quantized(m, n, k, l, seed=4, device="cuda")
    want = nvfp4_dual_gemm.custom_kernel(full).clone()
    bufs, ptrs = _buffers(m, n, l, world)
    for r in range(world):
        out = shard.GatheredOutput(m, n, l, "cuda", ptrs=ptrs, buf=bufs[r])
        shard.dual_gemm_allgather(shard.shard_dual_gemm(full, r, world), out, r)
    torch.cuda.synchronize()
    for b in bufs:
        assert torch.equal(b.permute(1, 2, 0).view(torch.int16), want.view(torch.int16))


def test_bad_arguments_are_rejected():
    import ctypes
    from eval_test_b200 import _lib
    lib = _lib.load()
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    arr = (ctypes.c_void_p * 2)(p, p + 4096)
    assert lib.nvfp4_gemm_allgather(p, p, p, p, arr, 9, 0, 128, 128, 256, 1, 1.0, None) == -2    # world > 8
    assert lib.nvfp4_gemm_allgather(p, p, p, p, arr, 2, 2, 128, 128, 256, 1, 1.0, None) == -2    # rank >= world
    bad = (ctypes.c_void_p * 2)(p, p + 16)
    assert lib.nvfp4_gemm_allgather(p, p, p, p, bad, 2, 0, 128, 128, 256, 1, 1.0, None) == -5    # 32-byte alignment
    assert lib.nvfp4_gemm_allgather(p, p, p, p, None, 2, 0, 128, 128, 256, 1, 1.0, None) == -1


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_through_symmetric_memory():
    """Two processes, one GPU each: every rank's copy of C must equal the unsharded product, bit for bit."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(os.path.dirname(__file__), "allgather_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert out.stdout.count("allgather ok") == 2
