"""Sharded execution on the GPU: the shards of a problem, run one after the other on one device, must reproduce
the unsharded kernel output bit for bit whenever shard and whole take the same kernel family (nothing is split
along K across ranks, so every output element is accumulated in the same order).  A skinny shard with a long K
may be sent to the cluster split-K kernel while the whole problem is not; its fp32 partial sums are then added in
another order and the fp16 results may differ in the last bit: that case is held to the harness's tolerance."""
import numpy as np
import pytest
import torch

from _util import out_np, to_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4])
def test_gemm_column_shards_are_bit_identical(world):
    from eval_test_b200 import inputs, nvfp4_gemm, shard
    full = inputs.gemm_quantized(256, 2048, 1024, 2, seed=31, device="cuda")
    want = out_np(nvfp4_gemm.custom_kernel(full, alpha=0.5))
    parts = [out_np(nvfp4_gemm.custom_kernel(shard.shard_gemm(full, r, world), alpha=0.5)) for r in range(world)]
    torch.cuda.synchronize()
    assert np.array_equal(np.concatenate(parts, axis=2).view(np.uint16), want.view(np.uint16))


def test_gemm_shards_on_another_kernel_family_stay_within_tolerance():
    """M = 128, N = 16384, K = 8192 runs on the persistent kernel (128 tiles); its four column shards have 32 tiles
    each and take the cluster split-K kernel."""
    from eval_test_b200 import check, inputs, nvfp4_gemm, shard
    full = inputs.gemm_quantized(128, 16384, 8192, 1, seed=35, device="cuda")
    want = nvfp4_gemm.custom_kernel(full).clone()
    parts = [nvfp4_gemm.custom_kernel(shard.shard_gemm(full, r, 4)).clone() for r in range(4)]
    torch.cuda.synchronize()
    got = torch.cat(parts, dim=1)
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []


def test_dual_gemm_column_shards_are_bit_identical():
    from eval_test_b200 import inputs, nvfp4_dual_gemm, shard
    full = inputs.dual_gemm_quantized(256, 1024, 512, 1, seed=32, device="cuda")
    want = out_np(nvfp4_dual_gemm.custom_kernel(full))
    parts = [out_np(nvfp4_dual_gemm.custom_kernel(shard.shard_dual_gemm(full, r, 4))) for r in range(4)]
    torch.cuda.synchronize()
    assert np.array_equal(np.concatenate(parts, axis=2).view(np.uint16), want.view(np.uint16))


def test_gemv_row_shards_are_bit_identical():
    from eval_test_b200 import inputs, nvfp4_gemv, shard
    full = inputs.gemv_quantized(1024, 2048, 2, seed=33, device="cuda")
    want = out_np(nvfp4_gemv.custom_kernel(full))
    parts = [out_np(nvfp4_gemv.custom_kernel(shard.shard_gemv(full, r, 4))) for r in range(4)]
    torch.cuda.synchronize()
    assert np.array_equal(np.concatenate(parts, axis=1).view(np.uint16), want.view(np.uint16))


def test_grouped_shards_cover_every_group_once():
    from eval_test_b200 import inputs, nvfp4_grouped_gemm, shard
    ms = [100, 0, 300, 40, 128, 0, 77, 130]
    full = inputs.grouped_gemm_quantized(ms, [256] * 8, [512] * 8, 8, seed=34, device="cuda")
    want = [out_np(c)[0].copy() for c in nvfp4_grouped_gemm.custom_kernel(full)]
    torch.cuda.synchronize()
    for (_, _, c) in full[0]:
        c.zero_()
    seen = []
    for r in range(3):
        loc, mine = shard.shard_grouped_gemm(full, r, 3)
        outs = nvfp4_grouped_gemm.custom_kernel(loc)
        torch.cuda.synchronize()
        for i, c in zip(mine, outs):
            assert np.array_equal(out_np(c)[0].view(np.uint16), want[i].view(np.uint16))
        seen += mine
    assert sorted(seen) == list(range(8))


def test_shutdown_frees_and_the_library_keeps_working():
    from eval_test_b200 import _lib, inputs, nvfp4_grouped_gemm
    data = to_device(inputs.grouped_gemm_reference_style([96, 128], [128, 256], [256, 512], 2, seed=1, device="cpu"))
    first = [out_np(c)[0].copy() for c in nvfp4_grouped_gemm.custom_kernel(data)]
    torch.cuda.synchronize()
    assert _lib.load().nvfp4_shutdown() == 0
    again = [out_np(c)[0] for c in nvfp4_grouped_gemm.custom_kernel(data)]
    torch.cuda.synchronize()
    assert all(np.array_equal(a.view(np.uint16), b.view(np.uint16)) for a, b in zip(first, again))
    assert _lib.device_status(torch.cuda.current_device()) == 0
