"""GPU parity of nvfp4_gemv (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from _util import operand_np, out_np, scales_np, to_device

pytestmark = pytest.mark.gpu

# shapes of the harness's GEMV correctness list (m, k, l)
REFERENCE_TESTS = [(128, 256, 1), (128, 1536, 1), (128, 3072, 1), (256, 7168, 1), (2432, 4608, 2),
                   (384, 7168, 2), (512, 512, 2), (512, 4096, 2), (512, 1536, 2)]


@pytest.fixture(params=["tensor", "alu"])
def path(request, monkeypatch):
    """Both GEMV kernels, each forced: the tensor-core stream and the decode-on-CUDA-cores kernel (the entry point
    picks one by the number of 128-row tiles when nothing is forced)."""
    monkeypatch.setenv("NVFP4_GEMV_PATH", request.param)
    return request.param


def _run(data, alpha=1.0):
    from eval_test_b200 import _lib, nvfp4_gemv
    out = nvfp4_gemv.custom_kernel(data, alpha=alpha) if alpha != 1.0 else nvfp4_gemv.custom_kernel(data)
    torch.cuda.synchronize()
    assert _lib.device_status(torch.cuda.current_device()) == 0
    assert out is data[-1]
    return out_np(out)[:, :, 0]


def _oracle(oracle, data, alpha=1.0):
    a, b, _, _, sfa_p, sfb_p, _ = data
    return oracle.c_gemv(operand_np(a), operand_np(b), scales_np(sfa_p), scales_np(sfb_p), alpha)


@pytest.mark.parametrize("m,k,l", REFERENCE_TESTS)
def test_reference_style_bit_exact(oracle, path, m, k, l):
    from eval_test_b200 import inputs
    data = to_device(inputs.gemv_reference_style(m, k, l, seed=1111, device="cpu"))
    got, want = _run(data), _oracle(oracle, data)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("m,k,l", [(128, 256, 1), (384, 2048 + 64, 3), (200, 1024, 2), (4096, 7168, 2), (128, 64, 1),
                                   (130, 192, 2), (1, 4096, 1)])
def test_quantized_within_tolerance(oracle, path, m, k, l):
    """N(0,1) data: fp32 summation order differs from the oracle, so compare with the harness's
    rtol = atol = 1e-3 rule and the 1e-2 * max|ref| bound."""
    from eval_test_b200 import check, inputs
    data = to_device(inputs.gemv_quantized(m, k, l, seed=3, device="cpu"))
    got, want = torch.from_numpy(_run(data, alpha=0.5)), torch.from_numpy(_oracle(oracle, data, alpha=0.5))
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []
    assert check.max_delta_ok(got, want)[0]


def test_all_bit_patterns(oracle, path):
    """Every byte value (all 16 x 16 nibble pairs, negative zeros included) in A and in x."""
    from eval_test_b200 import inputs
    data = list(inputs.gemm_reference_style(256, 128, 1024, 2, seed=5, device="cpu"))
    data[-1] = torch.empty((2, 256, 1), dtype=torch.float16).permute(1, 2, 0)  # [m, 1, l] output
    data = to_device(tuple(data))
    got, want = _run(data), _oracle(oracle, data)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_cluster_size_does_not_change_a_bit(monkeypatch):
    """The tensor-core kernel splits K over the CTAs of a cluster; the partial sums are formed and added per fixed
    K segment, so every cluster size must give the same bits (and so must a different M or L around the same rows)."""
    from eval_test_b200 import inputs, nvfp4_gemv, shard
    monkeypatch.setenv("NVFP4_GEMV_PATH", "tensor")
    data = inputs.gemv_quantized(1024, 4096 + 192, 2, seed=21, device="cuda")
    outs = []
    for s in (1, 2):
        monkeypatch.setenv("NVFP4_GEMV_SPLIT", str(s))
        data[-1].zero_()
        outs.append(_run(data).copy())
    for o in outs[1:]:
        assert np.array_equal(o.view(np.uint16), outs[0].view(np.uint16))
    monkeypatch.delenv("NVFP4_GEMV_SPLIT")
    part = _run(shard.shard_gemv(data, 1, 4))
    assert np.array_equal(part.view(np.uint16), outs[0][:, 256:512].view(np.uint16))


def test_default_dispatch_and_tensor_map_layouts(oracle, monkeypatch):
    """Nothing forced: small problems go to the decode kernel, large ones to the tensor-core stream; the stream's
    two ways of fetching A (one 5-D box per stage, one 128-row box per 256 elements) give the same bits; M that is
    not a multiple of 8 and K beyond 65536 are served."""
    from eval_test_b200 import inputs
    monkeypatch.delenv("NVFP4_GEMV_PATH", raising=False)
    for m, k, l in [(256, 1024, 1), (128 * 40, 1024, 1), (1000, 2048, 5), (1001, 1024 + 64, 5), (128, 65536 + 512, 1)]:
        data = to_device(inputs.gemv_reference_style(m, k, l, seed=7, device="cpu"))
        want = _oracle(oracle, data)
        got = _run(data).copy()
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), (m, k, l)
        monkeypatch.setenv("NVFP4_GEMV_ABOX", "3d")
        data[-1].zero_()
        assert np.array_equal(_run(data).view(np.uint16), want.view(np.uint16)), (m, k, l, "3d")
        monkeypatch.delenv("NVFP4_GEMV_ABOX")


def test_linearity_full_size():
    """Size-independent property at the full benchmark shape: doubling alpha doubles every output exactly
    (power-of-two scaling commutes with the fp16 rounding while no value is subnormal or overflows)."""
    from eval_test_b200 import inputs, nvfp4_gemv
    data = inputs.gemv_quantized(16384, 16384, 4, seed=0, device="cuda")
    c1 = nvfp4_gemv.custom_kernel(data, alpha=1.0).clone()
    c2 = nvfp4_gemv.custom_kernel(data, alpha=2.0).clone()
    torch.cuda.synchronize()
    ok = (c1.float().abs() > 1e-3) & (c1.float().abs() < 3e4)
    assert ok.float().mean() > 0.9
    assert torch.equal((2 * c1.float())[ok], c2.float()[ok])


def test_full_size_rows_against_oracle(oracle):
    """Full benchmark shape; a sample of rows is checked against the oracle (the whole matrix would take the
    CPU too long inside the test budget)."""
    from eval_test_b200 import check, inputs, nvfp4_gemv
    m = k = 16384
    data = inputs.gemv_quantized(m, k, 4, seed=0, device="cuda")
    a, b, _, _, sfa_p, sfb_p, c = data
    nvfp4_gemv.custom_kernel(data)
    torch.cuda.synchronize()
    rows = slice(128 * 37, 128 * 39)  # two whole 128-row blocks
    a_np = operand_np(a)[:, rows]
    sf = scales_np(sfa_p).reshape(4, m // 128, -1)[:, 37:39].reshape(-1)
    want = torch.from_numpy(oracle.c_gemv(a_np, operand_np(b), sf, scales_np(sfb_p)))
    got = torch.from_numpy(out_np(c)[:, rows, 0])
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []


def test_bad_arguments_are_rejected():
    from eval_test_b200 import _lib
    lib = _lib.load()
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    assert lib.nvfp4_gemv(p, p, p, p, p, 128, 100, 1, 128, 1.0, None) == -3   # K % 64
    assert lib.nvfp4_gemv(p, p, p, p, p, 0, 256, 1, 128, 1.0, None) == -2     # M <= 0
    assert lib.nvfp4_gemv(None, p, p, p, p, 128, 256, 1, 128, 1.0, None) == -1
    assert lib.nvfp4_gemv(p + 4, p, p, p, p, 128, 256, 1, 128, 1.0, None) == -5
    assert "K" in _lib.strerror(-3)


def test_wait_selftest_expires_and_reports():
    """A wait that nothing satisfies returns an error status instead of hanging; the context stays usable."""
    import ctypes
    from eval_test_b200 import _lib
    lib = _lib.load()
    _lib.device_status(torch.cuda.current_device())
    ms = ctypes.c_double(0)
    assert lib.nvfp4_wait_selftest(50, ctypes.byref(ms), None) == 0
    assert 40 <= ms.value < 500
    assert _lib.device_status(torch.cuda.current_device()) == 105
    assert _lib.device_status(torch.cuda.current_device()) == 0
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


def test_two_streams_at_once(monkeypatch):
    """Launches of the tensor-core kernel that overlap on two streams (each grid hands out its own tiles through
    cluster launch control; nothing is shared between launches) give the bits of the same launches run alone."""
    from eval_test_b200 import _lib, inputs, nvfp4_gemv
    monkeypatch.setenv("NVFP4_GEMV_PATH", "tensor")
    d1 = inputs.gemv_quantized(128 * 60, 4096, 1, seed=41, device="cuda")     # 60 tiles: leaves SMs for the other launch
    d2 = inputs.gemv_quantized(128 * 50, 2048, 2, seed=42, device="cuda")
    want1 = nvfp4_gemv.custom_kernel(d1).clone()
    want2 = nvfp4_gemv.custom_kernel(d2).clone()
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    for _ in range(20):
        d1[-1].zero_(); d2[-1].zero_()
        torch.cuda.synchronize()
        with torch.cuda.stream(s1):
            for _ in range(3):
                nvfp4_gemv.custom_kernel(d1)
        with torch.cuda.stream(s2):
            for _ in range(3):
                nvfp4_gemv.custom_kernel(d2)
        torch.cuda.synchronize()
        assert torch.equal(d1[-1].view(torch.int16), want1.view(torch.int16))
        assert torch.equal(d2[-1].view(torch.int16), want2.view(torch.int16))
    assert _lib.device_status(torch.cuda.current_device()) == 0
