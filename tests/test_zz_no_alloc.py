"""nvfp4_grouped_gemm_noalloc - the grouped GEMM for callers that cannot let the library allocate (their own
allocator owns all of HBM, or they cannot take the device-wide synchronisation an allocation implies) - must give
exactly what nvfp4_grouped_gemm gives.  Both run the same kernel; only the home of the problem table differs (a
fixed array inside the library instead of memory allocated on first use), so the comparison is bit for bit.

Two calls in a row with different problems check that the shared table is rewritten correctly: the second call
has fewer groups than the first, so stale entries of the first call sit behind the ones it reads.
This file is collected last on purpose (its name sorts after the others).
"""
import numpy as np
import pytest
import torch

from _util import grouped_oracle_args, out_np, to_device

pytestmark = pytest.mark.gpu


def _groups(data):
    from eval_test_b200 import _lib
    abc, _, sfs_p, sizes = data
    arr = (_lib.Group * len(abc))()
    for q, (a, b, c), (sa, sb), (m, n, k, _) in zip(arr, abc, sfs_p, sizes):
        q.M, q.N, q.K = m, n, k
        q.b, q.sfb_sw = b.data_ptr(), sb.data_ptr()
        if m > 0:
            q.a, q.sfa_sw, q.c = a.data_ptr(), sa.data_ptr(), c.data_ptr()
    return arr


def _run(entry, data):
    """Call one entry point through the C ABI on fresh, poisoned outputs; return the outputs."""
    from eval_test_b200 import _lib
    abc = data[0]
    for (_, _, c) in abc:
        c.fill_(float("nan"))
    arr = _groups(data)
    stream = torch.cuda.current_stream().cuda_stream
    rc = entry(arr, len(abc), 1.0, stream)
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    return [c.clone() for (_, _, c) in abc]


def test_noalloc_entry_matches_regular_entry_twice():
    from eval_test_b200 import _lib, inputs
    lib = _lib.load()
    first = to_device(inputs.grouped_gemm_quantized([100, 0, 300, 40, 128], [256, 256, 512, 128, 384],
                                                    [512, 256, 768, 256, 512], 5, seed=21, device="cpu"))
    second = to_device(inputs.grouped_gemm_reference_style([72, 256], [384, 128], [256, 512], 2, seed=22,
                                                           device="cpu"))
    for data in (first, second):
        got = _run(lib.nvfp4_grouped_gemm_noalloc, data)
        want = _run(lib.nvfp4_grouped_gemm, data)
        for g, w in zip(got, want):
            assert g.shape == w.shape
            assert not torch.isnan(g).any()
            assert torch.equal(g.view(torch.int16), w.view(torch.int16))
    assert _lib.device_status(torch.cuda.current_device()) == 0


def test_noalloc_entry_wide_tiles_against_the_oracle(oracle):
    """Every N a multiple of 256, so both entry points take the 256-column tile instantiation; dyadic inputs, so
    the fixed-table entry point must reproduce the CPU oracle (and the regular entry point) bit for bit; again on
    two calls in a row, the second with fewer groups."""
    from eval_test_b200 import _lib, inputs
    lib = _lib.load()
    first = to_device(inputs.grouped_gemm_reference_style([200, 0, 96, 384], [256, 512, 768, 256], [512, 256, 256, 768],
                                                          4, seed=23, device="cpu"))
    second = to_device(inputs.grouped_gemm_reference_style([130, 64], [512, 256], [256, 1024], 2, seed=24,
                                                           device="cpu"))
    for data in (first, second):
        want = oracle.c_grouped_gemm(grouped_oracle_args(data))
        for entry in (lib.nvfp4_grouped_gemm_noalloc, lib.nvfp4_grouped_gemm):
            got = _run(entry, data)
            for g, w in zip(got, want):
                assert np.array_equal(out_np(g)[0].view(np.uint16), w.view(np.uint16))
    assert _lib.device_status(torch.cuda.current_device()) == 0


def test_noalloc_entry_rejects_more_groups_than_its_table_holds():
    from eval_test_b200 import _lib
    lib = _lib.load()
    p = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda").data_ptr()
    n = 257
    arr = (_lib.Group * n)()
    for q in arr:
        q.a = q.b = q.sfa_sw = q.sfb_sw = q.c = p
        q.M, q.N, q.K = 128, 128, 256
    rc = lib.nvfp4_grouped_gemm_noalloc(arr, n, 1.0, None)
    assert rc == -9 and "groups" in _lib.strerror(rc)
