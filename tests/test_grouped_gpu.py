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


@pytest.mark.parametrize("forced_empty", [(), (3, 17, 18, 40, 63)])
def test_grouped_moe_configuration_full_size(oracle, forced_empty):
    """The MoE expert-layer configuration at full size: 64 groups, N = 4096, K = 7168, M_g ~ Poisson(128) clipped
    to [0, 1024] from numpy's default_rng(0); the second variant forces five groups to M = 0 (a seeded draw never
    gives an empty group).  Every group against the reference's arithmetic (torch._scaled_mm per group,
    eval/nvfp4_grouped_gemm/reference.py:48-74), sampled groups against the CPU oracle, under rtol = atol = 1e-3 and
    max|d| <= 1e-2 max|ref|; outputs of empty groups stay empty and nothing else is touched."""
    from _util import operand_np, scales_np
    from eval_test_b200 import check, inputs, reference_check
    g = 64
    m = inputs.poisson_group_sizes(g, 128.0, 0, 1024, seed=0)
    for i in forced_empty:
        m[i] = 0
    data = inputs.grouped_gemm_quantized(m, [4096] * g, [7168] * g, g, seed=0, device="cuda")
    got = _run(data)
    want = reference_check.ref_grouped_gemm(data)
    abc, _, sfs_p, _ = data
    for i, (mine, ref) in enumerate(zip(got, want)):
        assert mine.shape == (m[i], 4096)
        if m[i]:
            mine_t, ref_t = torch.from_numpy(mine), ref[:, :, 0].cpu()
            assert check.verbose_allclose(mine_t, ref_t, rtol=1e-3, atol=1e-3) == [], i
            assert check.max_delta_ok(mine_t, ref_t)[0], i
    for i in (0, 19, 41, 62):
        (a, b, _), (sa, sb) = abc[i], sfs_p[i]
        ref = oracle.c_gemm(operand_np(a), operand_np(b), scales_np(sa), scales_np(sb))[0]
        assert check.verbose_allclose(torch.from_numpy(got[i]), torch.from_numpy(ref), rtol=1e-3, atol=1e-3) == [], i


def test_grouped_same_call_again_and_from_a_second_stream(oracle):
    """The library reuses a problem table when a call repeats an earlier one (same pointers and sizes).  The
    repeat may come on another stream while the first call's table upload is still queued, so the reuse must be
    ordered after the upload; outputs are poisoned between the calls and compared with the oracle bit for bit."""
    from eval_test_b200 import inputs, nvfp4_grouped_gemm
    data = to_device(inputs.grouped_gemm_reference_style([200, 96, 0, 384], [256, 512, 256, 256], [512, 256, 256, 768],
                                                         4, seed=31, device="cpu"))
    want = oracle.c_grouped_gemm(grouped_oracle_args(data))
    side = torch.cuda.Stream()

    def poison():
        for (_, _, c) in data[0]:
            c.fill_(float("nan"))

    def verify():
        torch.cuda.synchronize()
        for (_, _, c), w in zip(data[0], want):
            assert np.array_equal(out_np(c)[0].view(np.uint16), w.view(np.uint16))

    poison()
    torch.cuda.synchronize()
    # a long copy keeps the first stream busy, so its table upload and launch are still queued when the
    # second stream asks for the same table
    busy = torch.empty(1 << 28, dtype=torch.uint8, device="cuda")
    for _ in range(8):
        busy.fill_(1)
    nvfp4_grouped_gemm.custom_kernel(data)
    with torch.cuda.stream(side):
        nvfp4_grouped_gemm.custom_kernel(data)
    verify()
    for stream in (torch.cuda.current_stream(), side, torch.cuda.current_stream()):
        poison()
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            nvfp4_grouped_gemm.custom_kernel(data)
        verify()


def test_grouped_repeated_calls_and_streams(oracle):
    """More distinct problems back to back than the library has problem-table slots (40 for 32), on two streams:
    every call's table must stay intact until its launch has read it."""
    from eval_test_b200 import inputs, nvfp4_grouped_gemm
    sets = [to_device(inputs.grouped_gemm_reference_style([96 + 8 * i, 128], [128, 256], [256, 512], 2, seed=i,
                                                          device="cpu")) for i in range(40)]
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


_PAIR_CHILD = r'''
import sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from _util import grouped_oracle_args, out_np, to_device
from eval_test_b200 import _lib, check, inputs, nvfp4_grouped_gemm
from oracle import nvfp4_oracle as O
cases = [([96, 128], [256, 256], [256, 512]),                    # one pair tile each, second CTA without rows / full
         ([300, 0, 130, 512, 1], [256, 512, 256, 768, 256], [512, 256, 256, 256, 768]),   # ragged, empty, several row tiles
         ([256, 257], [512, 256], [1024, 256])]
for m, n, k in cases:
    d = to_device(inputs.grouped_gemm_reference_style(m, n, k, len(m), seed=41, device="cpu"))
    outs = nvfp4_grouped_gemm.custom_kernel(d)
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0
    for got, want in zip(outs, O.c_grouped_gemm(grouped_oracle_args(d))):
        assert np.array_equal(out_np(got)[0].view(np.uint16), want.view(np.uint16)), (m, n, k)
    outs = nvfp4_grouped_gemm.custom_kernel(d)                   # the same call again: reused table
    torch.cuda.synchronize()
    for got, want in zip(outs, O.c_grouped_gemm(grouped_oracle_args(d))):
        assert np.array_equal(out_np(got)[0].view(np.uint16), want.view(np.uint16)), (m, n, k)
d = to_device(inputs.grouped_gemm_quantized([140, 100, 0, 260], [512] * 4, [768] * 4, 4, seed=42, device="cpu"))
outs = nvfp4_grouped_gemm.custom_kernel(d, alpha=0.5)
torch.cuda.synchronize()
for got, want in zip(outs, O.c_grouped_gemm(grouped_oracle_args(d), alpha=0.5)):
    if want.size:
        assert check.verbose_allclose(torch.from_numpy(out_np(got)[0]), torch.from_numpy(want), rtol=1e-3, atol=1e-3) == []
print("grouped pair ok")
'''


def test_grouped_on_cta_pairs_in_a_child_process():
    """The CTA-pair kernel under the grouped scheduler (opt-in: NVFP4_GEMM_PAIR=1, read once per process): groups of
    one pair tile whose second CTA owns no rows, ragged and empty groups, several row tiles, a repeated call; dyadic
    inputs bit-exact, quantised inputs within the harness's tolerance."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = str(Path(__file__).resolve().parent.parent)
    env = dict(os.environ, NVFP4_GEMM_PAIR="1")
    res = subprocess.run([sys.executable, "-c", _PAIR_CHILD, root], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "grouped pair ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


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
