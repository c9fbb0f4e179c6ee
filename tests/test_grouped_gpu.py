"""GPU parity of nvfp4_grouped_gemm (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from _util import grouped_oracle_args, out_np, to_device

pytestmark = pytest.mark.gpu

# the harness's grouped correctness list: (m list, n list, k list)
GROUPED_TESTS = [
    ([96, 128], [128, 256], [256, 512]),
    ([256, 72], [512, 384], [256, 256]),
    ([128, 128], [128, 256], [512, 256]),
    ([80, 128, 256], [384, 256, 128], [256, 512, 256]),
    ([64, 72, 96], [128, 384, 512], [512, 512, 256]),
    ([64, 256, 128], [768, 128, 256], [512, 256, 512]),
    ([128, 128, 64], [256, 512, 512], [768, 256, 768]),
    ([128, 128, 128, 128], [128, 128, 128, 128], [512, 256, 512, 256]),
    ([40, 56, 384, 512], [512, 384, 256, 128], [256, 256, 256, 256]),
    ([512, 384, 256, 128], [256, 256, 256, 256], [512, 768, 512, 768]),
]


def _run(data, alpha=1.0):
    from eval_test_b200 import _lib, nvfp4_grouped_gemm
    outs = nvfp4_grouped_gemm.custom_kernel(data, alpha=alpha)
    torch.cuda.synchronize()
    st = _lib.device_status(torch.cuda.current_device())
    assert st == 0, _lib.strerror(st)
    assert len(outs) == len(data[0])
    return [out_np(c)[0] for c in outs]


@pytest.mark.parametrize("m,n,k", GROUPED_TESTS)
def test_grouped_reference_style_bit_exact(oracle, m, n, k):
    """Dyadic inputs, ragged M, random garbage in the padding rows of the scale buffers: bit-exact."""
    from eval_test_b200 import inputs
    data = to_device(inputs.grouped_gemm_reference_style(m, n, k, len(m), seed=1111, device="cpu"))
    got, want = _run(data), oracle.c_grouped_gemm(grouped_oracle_args(data))
    for g, w in zip(got, want):
        assert g.shape == w.shape and np.array_equal(g.view(np.uint16), w.view(np.uint16))


def test_grouped_with_empty_groups(oracle):
    """Groups with M = 0 are skipped; their neighbours are unaffected; untouched outputs keep their contents."""
    from eval_test_b200 import check, inputs
    m, n, k = [0, 100, 0, 0, 300, 1, 0], [256] * 7, [512, 256, 256, 512, 768, 256, 256]
    data = to_device(inputs.grouped_gemm_quantized(m, n, k, len(m), seed=2, device="cpu"))
    got, want = _run(data, alpha=0.5), oracle.c_grouped_gemm(grouped_oracle_args(data), alpha=0.5)
    for g, w in zip(got, want):
        assert g.shape == w.shape
        if w.size:
            assert check.verbose_allclose(torch.from_numpy(g), torch.from_numpy(w), rtol=1e-3, atol=1e-3) == []


def test_grouped_all_empty_is_a_no_op():
    from eval_test_b200 import inputs
    data = to_device(inputs.grouped_gemm_quantized([0, 0], [128, 256], [256, 256], 2, seed=2, device="cpu"))
    assert [g.shape for g in _run(data)] == [(0, 128), (0, 256)]


def test_grouped_poisson_sizes_wide_tiles(oracle):
    """A scaled-down version of the MoE configuration (M ~ Poisson(128), N a multiple of 256): sampled groups
    are compared with the oracle within the harness's tolerance."""
    from eval_test_b200 import check, inputs
    g = 12
    m = inputs.poisson_group_sizes(g, 128.0, 0, 1024, seed=0)
    m[3] = 0
    data = to_device(inputs.grouped_gemm_quantized(m, [512] * g, [1024] * g, g, seed=0, device="cpu"))
    got, want = _run(data), oracle.c_grouped_gemm(grouped_oracle_args(data))
    for gg, w in zip(got, want):
        assert gg.shape == w.shape
        if w.size:
            assert check.verbose_allclose(torch.from_numpy(gg), torch.from_numpy(w), rtol=1e-3, atol=1e-3) == []


def test_grouped_repeated_calls_and_streams(oracle):
    """More back-to-back calls than the library has problem-table slots, on two streams: every call's table
    must stay intact until its launch has read it."""
    from eval_test_b200 import inputs, nvfp4_grouped_gemm
    sets = [to_device(inputs.grouped_gemm_reference_style([96 + 8 * i, 128], [128, 256], [256, 512], 2, seed=i,
                                                          device="cpu")) for i in range(12)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for rep in range(3):
        for i, d in enumerate(sets):
            with torch.cuda.stream(streams[i % 2]):
                nvfp4_grouped_gemm.custom_kernel(d)
    torch.cuda.synchronize()
    for d in sets:
        want = oracle.c_grouped_gemm(grouped_oracle_args(d))
        for (_, _, c), w in zip(d[0], want):
            assert np.array_equal(out_np(c)[0].view(np.uint16), w.view(np.uint16))


def test_grouped_bad_arguments():
    import ctypes
    from eval_test_b200 import _lib
    lib = _lib.load()
    p = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda").data_ptr()
    grp = (_lib.Group * 1)()
    grp[0].a = grp[0].b = grp[0].sfa_sw = grp[0].sfb_sw = grp[0].c = p
    grp[0].M, grp[0].N, grp[0].K = 128, 128, 100
    assert lib.nvfp4_grouped_gemm(grp, 1, 1.0, None) == -3
    grp[0].K, grp[0].N = 256, 100
    assert lib.nvfp4_grouped_gemm(grp, 1, 1.0, None) == -4
    grp[0].N, grp[0].c = 128, None
    assert lib.nvfp4_grouped_gemm(grp, 1, 1.0, None) == -1
    assert lib.nvfp4_grouped_gemm(grp, 0, 1.0, None) == -2
    assert lib.nvfp4_grouped_gemm(None, 1, 1.0, None) == -1
