"""GPU parity of nvfp4_gemm / nvfp4_dual_gemm (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from _util import dual_oracle_args, gemm_oracle_args, out_np, to_device

pytestmark = pytest.mark.gpu

# the harness's correctness lists (m, n, k, l): every line of eval/nvfp4_gemm/tests.txt and every distinct line of
# eval/nvfp4_dual_gemm/tests.txt
GEMM_TESTS = [(128, 256, 256, 1), (128, 1536, 7168, 1), (128, 3072, 1536, 1), (256, 7168, 256, 1),
              (256, 7168, 2048, 1), (2304, 4608, 7168, 1), (384, 7168, 2304, 1), (512, 512, 7168, 1),
              (512, 4096, 512, 1), (512, 1536, 7168, 1)]
DUAL_TESTS = [(1536, 512, 7168, 1), (256, 512, 256, 1), (3072, 1024, 1536, 1), (7168, 1024, 256, 1),
              (7168, 2304, 2048, 1), (4608, 384, 7168, 1), (7168, 384, 2304, 1), (512, 768, 7168, 1),
              (4096, 768, 512, 1)]


def _status_ok():
    from eval_test_b200 import _lib
    torch.cuda.synchronize()
    st = _lib.device_status(torch.cuda.current_device())
    assert st == 0, _lib.strerror(st)


def _gemm(data, alpha=1.0):
    from eval_test_b200 import nvfp4_gemm
    out = nvfp4_gemm.custom_kernel(data, alpha=alpha)
    _status_ok()
    assert out is data[-1]
    return out_np(out)


def _dual(data, alpha=1.0):
    from eval_test_b200 import nvfp4_dual_gemm
    out = nvfp4_dual_gemm.custom_kernel(data, alpha=alpha)
    _status_ok()
    return out_np(out)


def test_one_tile_one_k_iteration(oracle):
    """Smallest case the kernel takes: pins nibble order, swizzles, descriptors and the scale layout."""
    from eval_test_b200 import inputs
    data = to_device(inputs.gemm_reference_style(128, 128, 256, 1, seed=1, device="cpu"))
    got, want = _gemm(data), oracle.c_gemm(*gemm_oracle_args(data))
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("m,n,k,l", GEMM_TESTS)
def test_gemm_reference_style_bit_exact(oracle, m, n, k, l):
    """Dyadic inputs: fp32 accumulation is exact in any order, so the result must equal the oracle's bits."""
    from eval_test_b200 import inputs
    data = to_device(inputs.gemm_reference_style(m, n, k, l, seed=1111, device="cpu"))
    got, want = _gemm(data), oracle.c_gemm(*gemm_oracle_args(data))
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("m,n,k,l", [(2176, 2560, 1024, 1), (2048, 2304, 512, 2), (4096, 2048, 256, 1)])
def test_gemm_cta_pairs_by_default_bit_exact(oracle, m, n, k, l):
    """Shapes with at least one 256 x 256 tile per pair of SMs take the CTA-pair kernel by default: a ragged last row
    tile (M = 8.5 x 256: its second CTA owns no rows), batches, a single K step per tile."""
    from eval_test_b200 import inputs
    data = to_device(inputs.gemm_reference_style(m, n, k, l, seed=61, device="cpu"))
    got, want = _gemm(data), oracle.c_gemm(*gemm_oracle_args(data))
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("m,n,k,l", [(2304, 1280, 512, 1), (2176, 640, 256, 2)])
def test_dual_gemm_cta_pairs_by_default(oracle, m, n, k, l):
    from eval_test_b200 import check, inputs
    data = to_device(inputs.dual_gemm_reference_style(m, n, k, l, seed=62, device="cpu"))
    got = torch.from_numpy(_dual(data))
    want = torch.from_numpy(oracle.c_dual_gemm(*dual_oracle_args(data)))
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []


def test_gemm_wide_single_cta_tiles_bit_exact(oracle):
    """M = 640 is not a multiple of 256, so the CTA-pair kernel is not chosen; 5 x 32 tiles of 128 x 256 fill the
    machine, so the single-CTA kernel runs with its 256-column tiles."""
    from eval_test_b200 import inputs
    data = to_device(inputs.gemm_reference_style(640, 8192, 512, 1, seed=12, device="cpu"))
    got, want = _gemm(data), oracle.c_gemm(*gemm_oracle_args(data))
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("m,n,k,l,alpha", [(128, 256, 512, 1, 1.0), (200, 384, 768, 2, 0.5), (1000, 1280, 1024, 1, 0.5)])
def test_gemm_quantized_within_tolerance(oracle, m, n, k, l, alpha):
    """N(0,1) data through the quantiser (the first case is the CPU-runnable configuration), ragged M,
    batches, alpha: rtol = atol = 1e-3 element-wise and max|d| <= 1e-2 max|ref|."""
    from eval_test_b200 import check, inputs
    data = to_device(inputs.gemm_quantized(m, n, k, l, seed=0, device="cpu"))
    got = torch.from_numpy(_gemm(data, alpha))
    want = torch.from_numpy(oracle.c_gemm(*gemm_oracle_args(data), alpha))
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []
    assert check.max_delta_ok(got, want)[0]


@pytest.mark.parametrize("m,n,k,l", DUAL_TESTS)
def test_dual_gemm_reference_style(oracle, m, n, k, l):
    """U[0,1) e4m3 scales (subnormals and zeros included): inexact in fp32, so the harness's tolerance."""
    from eval_test_b200 import check, inputs
    data = to_device(inputs.dual_gemm_reference_style(m, n, k, l, seed=1111, device="cpu"))
    got = torch.from_numpy(_dual(data))
    want = torch.from_numpy(oracle.c_dual_gemm(*dual_oracle_args(data)))
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []


def test_dual_gemm_quantized(oracle):
    from eval_test_b200 import check, inputs
    data = to_device(inputs.dual_gemm_quantized(384, 512, 1024, 2, seed=0, device="cpu"))
    got = torch.from_numpy(_dual(data))
    want = torch.from_numpy(oracle.c_dual_gemm(*dual_oracle_args(data)))
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []
    assert check.max_delta_ok(got, want)[0]


def test_large_gemm_rows_against_oracle(oracle):
    """8192^3 with alpha = 0.5 (the large benchmark configuration): a 128-row band of the output is checked
    against the oracle, the whole output through linearity in alpha."""
    from eval_test_b200 import check, inputs, nvfp4_gemm
    m = n = k = 8192
    data = inputs.gemm_quantized(m, n, k, 1, seed=0, device="cuda")
    a, b, _, _, sfa_p, sfb_p, c = data
    c_half = nvfp4_gemm.custom_kernel(data, alpha=0.5).clone()
    c_one = nvfp4_gemm.custom_kernel(data, alpha=1.0).clone()
    _status_ok()
    ok = (c_half.float().abs() > 1e-3) & (c_one.float().abs() < 3e4)
    assert ok.float().mean() > 0.9
    assert torch.equal((2 * c_half.float())[ok], c_one.float()[ok])
    band = slice(128 * 17, 128 * 18)
    from _util import operand_np, scales_np
    sfa = scales_np(sfa_p).reshape(m // 128, -1)[17].reshape(-1)
    want = torch.from_numpy(oracle.c_gemm(operand_np(a)[:, band], operand_np(b), sfa, scales_np(sfb_p), 0.5))
    got = torch.from_numpy(out_np(c_half)[:, band])
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []
    assert check.max_delta_ok(got, want)[0]


def test_large_gemm_whole_output_against_scaled_mm():
    """8192^3, N(0,1)-quantised operands: every element against the reference's arithmetic
    (torch._scaled_mm, eval/nvfp4_gemm/reference.py:16-27) under the harness's rtol = atol = 1e-3."""
    from eval_test_b200 import check, inputs, nvfp4_gemm, reference_check
    data = inputs.gemm_quantized(8192, 8192, 8192, 1, seed=0, device="cuda")
    got = nvfp4_gemm.custom_kernel(data).clone()
    _status_ok()
    want = reference_check.ref_gemm(data)
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []
    assert check.max_delta_ok(got, want)[0]


def test_large_dual_gemm_rows_against_oracle_and_whole_output_against_scaled_mm(oracle):
    """The SwiGLU up-projection configuration, M = 4096, N = 14336, K = 4096, N(0,1)-quantised operands: two
    128-row bands of the output against the CPU oracle, every element against the reference's arithmetic (two fp32
    torch._scaled_mm products, silu(r1) * r2 in fp32, one rounding: eval/nvfp4_dual_gemm/reference.py:24-44), both
    under the harness's rtol = atol = 1e-3 and under max|d| <= 1e-2 max|ref|."""
    from _util import operand_np, scales_np
    from eval_test_b200 import check, inputs, nvfp4_dual_gemm, reference_check
    m, n, k = 4096, 14336, 4096
    data = inputs.dual_gemm_quantized(m, n, k, 1, seed=0, device="cuda")
    a, b1, b2, _, _, _, sfa_p, sfb1_p, sfb2_p, c = data
    got = nvfp4_dual_gemm.custom_kernel(data).clone()
    _status_ok()
    want = reference_check.ref_dual_gemm(data)
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []
    assert check.max_delta_ok(got, want)[0]
    sfa_blocks = scales_np(sfa_p).reshape(m // 128, -1)
    for blk in (0, 23):
        band = slice(128 * blk, 128 * (blk + 1))
        ref = torch.from_numpy(oracle.c_dual_gemm(operand_np(a)[:, band], operand_np(b1), operand_np(b2),
                                                  sfa_blocks[blk].reshape(-1), scales_np(sfb1_p), scales_np(sfb2_p)))
        mine = torch.from_numpy(out_np(got)[:, band])
        assert check.verbose_allclose(mine, ref, rtol=1e-3, atol=1e-3) == []
        assert check.max_delta_ok(mine, ref)[0]


def test_gemm_bad_arguments():
    from eval_test_b200 import _lib
    lib = _lib.load()
    p = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda").data_ptr()
    assert lib.nvfp4_gemm(p, p, p, p, p, 128, 128, 128, 1, 1.0, None) == -3    # K % 256
    assert lib.nvfp4_gemm(p, p, p, p, p, 128, 64, 256, 1, 1.0, None) == -4     # N % 128
    assert lib.nvfp4_gemm(p, p, p, p, None, 128, 128, 256, 1, 1.0, None) == -1
    assert lib.nvfp4_dual_gemm(p, p, p, p, p, p, p, 0, 128, 256, 1, 1.0, None) == -2


_PAIR_CHILD = r'''
import sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from _util import dual_oracle_args, gemm_oracle_args, out_np, to_device
from eval_test_b200 import _lib, inputs, nvfp4_dual_gemm, nvfp4_gemm
from oracle import nvfp4_oracle as O
for (m, n, k, l) in [(256, 256, 256, 1), (384, 256, 512, 1), (512, 512, 512, 2), (1024, 768, 2048, 1)]:
    d = to_device(inputs.gemm_reference_style(m, n, k, l, seed=5, device="cpu"))
    nvfp4_gemm.custom_kernel(d)
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0
    assert np.array_equal(out_np(d[-1]).view(np.uint16), O.c_gemm(*gemm_oracle_args(d)).view(np.uint16)), (m, n, k, l)
for (m, n, k, l) in [(256, 128, 256, 1), (384, 256, 512, 2)]:
    d = to_device(inputs.dual_gemm_reference_style(m, n, k, l, seed=5, device="cpu"))
    nvfp4_dual_gemm.custom_kernel(d)
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0
    got, want = out_np(d[-1]).astype(np.float32), O.c_dual_gemm(*dual_oracle_args(d)).astype(np.float32)
    assert np.all(np.abs(got - want) <= 1e-3 + 1e-3 * np.abs(want)), (m, n, k, l)
print("pair ok")
'''


def test_cta_pair_kernels_in_a_child_process():
    """The cta_group::2 variants forced onto small shapes (NVFP4_GEMM_PAIR=1, read once per process; by default
    they are taken only when there are enough 256-row tiles to fill the machine): one pair tile, ragged
    M (the second CTA of the last row tile owns no rows), batches, several tiles per pair; GEMM bit-exact, dual
    GEMM within the harness's tolerance."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = str(Path(__file__).resolve().parent.parent)
    env = dict(os.environ, NVFP4_GEMM_PAIR="1")
    res = subprocess.run([sys.executable, "-c", _PAIR_CHILD, root], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "pair ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


_STREAMK_CHILD = r'''
import sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from _util import dual_oracle_args, gemm_oracle_args, out_np, to_device
from eval_test_b200 import _lib, check, inputs, nvfp4_dual_gemm, nvfp4_gemm
from oracle import nvfp4_oracle as O
# pair tiles on 74 pairs: 128 tiles of 8 K steps (shares of 13.8 steps: every tile whole or cut in two), 40 tiles of
# 16 steps (shares of 8.6: every tile cut into two or three pieces; ragged M: the last row tile's second CTA owns no
# rows), 48 tiles of 16 steps in two batches
for (m, n, k, l) in [(2048, 4096, 2048, 1), (1100, 2048, 4096, 1), (768, 2048, 4096, 2)]:
    d = to_device(inputs.gemm_reference_style(m, n, k, l, seed=51, device="cpu"))
    nvfp4_gemm.custom_kernel(d)
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0
    assert np.array_equal(out_np(d[-1]).view(np.uint16), O.c_gemm(*gemm_oracle_args(d)).view(np.uint16)), (m, n, k, l)
    nvfp4_gemm.custom_kernel(d)            # again: the flags of the first launch must not satisfy the second
    torch.cuda.synchronize()
    assert np.array_equal(out_np(d[-1]).view(np.uint16), O.c_gemm(*gemm_oracle_args(d)).view(np.uint16)), (m, n, k, l)
d = to_device(inputs.gemm_quantized(1024, 2304, 2048, 1, seed=52, device="cpu"))
nvfp4_gemm.custom_kernel(d, alpha=0.5)
torch.cuda.synchronize()
got, want = torch.from_numpy(out_np(d[-1])), torch.from_numpy(O.c_gemm(*gemm_oracle_args(d), 0.5))
assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []
for (m, n, k, l) in [(1024, 1792, 1024, 1), (768, 1920, 4096, 1)]:
    d = to_device(inputs.dual_gemm_reference_style(m, n, k, l, seed=53, device="cpu"))
    nvfp4_dual_gemm.custom_kernel(d)
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0
    got, want = out_np(d[-1]).astype(np.float32), O.c_dual_gemm(*dual_oracle_args(d)).astype(np.float32)
    assert np.all(np.abs(got - want) <= 1e-3 + 1e-3 * np.abs(want)), (m, n, k, l)
print("streamk ok")
'''


def test_stream_k_on_cta_pairs_in_a_child_process():
    """The stream-K schedule of the CTA-pair kernel (opt-in: NVFP4_GEMM_STREAMK=1, with NVFP4_GEMM_PAIR=1, read once
    per process) on shapes whose tiles do not fill the last round of pairs: tiles cut into two and into several
    pieces, ragged M, batches, the same call twice (a new epoch of the flags); dyadic inputs must match the oracle bit
    for bit whatever the order in which the partial sums are added; quantised and dual-GEMM inputs within the
    harness's tolerance."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = str(Path(__file__).resolve().parent.parent)
    env = dict(os.environ, NVFP4_GEMM_PAIR="1", NVFP4_GEMM_STREAMK="1")
    res = subprocess.run([sys.executable, "-c", _STREAMK_CHILD, root], env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0 and "streamk ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


def test_column_shard_of_the_large_gemm_against_scaled_mm():
    """M = 8192, N = 1024, K = 8192 (one eighth of the large GEMM's columns, what a rank of an 8-GPU run computes:
    128 pair tiles for 74 pairs of SMs, a partly filled second round): every element against torch._scaled_mm."""
    from eval_test_b200 import check, inputs, nvfp4_gemm, reference_check
    data = inputs.gemm_quantized(8192, 1024, 8192, 1, seed=3, device="cuda")
    got = nvfp4_gemm.custom_kernel(data, alpha=1.0).clone()
    _status_ok()
    want = reference_check.ref_gemm(data)
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []
    assert check.max_delta_ok(got, want)[0]


_SPLITK_CHILD = r'''
import sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from _util import gemm_oracle_args, out_np, to_device
from eval_test_b200 import _lib, check, inputs, nvfp4_gemm
from oracle import nvfp4_oracle as O
for (m, n, k, l) in [(128, 1536, 7168, 1), (200, 512, 1792, 2), (128, 128, 4096, 1), (384, 256, 2560, 1)]:
    d = to_device(inputs.gemm_reference_style(m, n, k, l, seed=77, device="cpu"))
    nvfp4_gemm.custom_kernel(d)
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0
    assert np.array_equal(out_np(d[-1]).view(np.uint16), O.c_gemm(*gemm_oracle_args(d)).view(np.uint16)), (m, n, k, l)
d = to_device(inputs.gemm_quantized(128, 1024, 4096, 1, seed=9, device="cpu"))
nvfp4_gemm.custom_kernel(d, alpha=0.5)
torch.cuda.synchronize()
got, want = torch.from_numpy(out_np(d[-1])), torch.from_numpy(O.c_gemm(*gemm_oracle_args(d), 0.5))
assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []
print("splitk ok")
'''


@pytest.mark.parametrize("cluster", [2, 4, 8])
def test_gemm_cluster_split_k_in_a_child_process(cluster):
    """The cluster split-K kernel with every cluster size (forced through NVFP4_GEMM_SPLITK, read once per
    process): dyadic inputs must match the oracle bit for bit (the partial sums and their fixed-order reduction
    are exact), including an uneven split of the K steps (7 or 10 steps), ragged M and batches; a quantised case
    within the harness's tolerance."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = str(Path(__file__).resolve().parent.parent)
    env = dict(os.environ, NVFP4_GEMM_SPLITK=str(cluster))
    res = subprocess.run([sys.executable, "-c", _SPLITK_CHILD, root], env=env, capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0 and "splitk ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


_DUAL_SPLITK_CHILD = r'''
import sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from _util import dual_oracle_args, out_np, to_device
from eval_test_b200 import _lib, check, inputs, nvfp4_dual_gemm
from oracle import nvfp4_oracle as O
cases = [("ref", 128, 512, 7168, 1), ("ref", 200, 256, 2560, 2), ("quant", 256, 384, 4096, 1), ("quant", 100, 128, 1792, 1)]
for kind, m, n, k, l in cases:
    gen = inputs.dual_gemm_reference_style if kind == "ref" else inputs.dual_gemm_quantized
    d = to_device(gen(m, n, k, l, seed=5, device="cpu"))
    nvfp4_dual_gemm.custom_kernel(d)
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0
    got, want = torch.from_numpy(out_np(d[-1])), torch.from_numpy(O.c_dual_gemm(*dual_oracle_args(d)))
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == [], (kind, m, n, k, l)
    assert check.max_delta_ok(got, want)[0], (kind, m, n, k, l)
print("dual splitk ok")
'''


@pytest.mark.parametrize("cluster", [2, 4])
def test_dual_gemm_cluster_split_k_in_a_child_process(cluster):
    """The dual GEMM on the cluster split-K kernel (both products reduced across the cluster before silu(x) * y),
    cluster sizes 2 and 4 forced through NVFP4_GEMM_SPLITK: reference-style and N(0,1)-quantised inputs, ragged M, an
    uneven split of the K steps (7 or 10 steps) and batches, against the oracle under the harness's tolerance."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = str(Path(__file__).resolve().parent.parent)
    env = dict(os.environ, NVFP4_GEMM_SPLITK=str(cluster))
    res = subprocess.run([sys.executable, "-c", _DUAL_SPLITK_CHILD, root], env=env, capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0 and "dual splitk ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


def test_dual_gemm_few_tiles_take_split_k_by_default(oracle):
    """M = 256, N = 4096, K = 7168 (a benchmark shape of the reference's dual-GEMM list): 64 tiles for 148 SMs, split
    across clusters of 2 by the default heuristic."""
    from eval_test_b200 import check, inputs
    data = to_device(inputs.dual_gemm_reference_style(256, 4096, 7168, 1, seed=1111, device="cpu"))
    got = torch.from_numpy(_dual(data))
    want = torch.from_numpy(oracle.c_dual_gemm(*dual_oracle_args(data)))
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []
    assert check.max_delta_ok(got, want)[0]


def test_gemm_long_k_takes_split_k_by_default(oracle):
    """M = 128, N = 7168, K = 16384 (the reference's first benchmark shape) is split across clusters of 2 by the
    default heuristic."""
    from eval_test_b200 import inputs
    data = to_device(inputs.gemm_reference_style(128, 7168, 16384, 1, seed=1111, device="cpu"))
    got, want = _gemm(data), oracle.c_gemm(*gemm_oracle_args(data))
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
