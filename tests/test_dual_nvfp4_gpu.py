"""The dual GEMM that emits NVFP4: bit for bit the quantiser applied to the fp16 output of the plain dual GEMM,
and accepted as the A operand of the next GEMM."""
import numpy as np
import pytest
import torch

from _util import gemm_oracle_args, out_np

pytestmark = pytest.mark.gpu


def _two_step(data):
    from eval_test_b200 import nvfp4_dual_gemm, quantize
    c = nvfp4_dual_gemm.custom_kernel(data)
    return quantize.quantize_operand(c.permute(2, 0, 1).contiguous().float())


@pytest.mark.parametrize("m,n,k,l", [(256, 256, 512, 1), (200, 384, 768, 2), (512, 128, 256, 1), (1, 128, 256, 3),
                                     (384, 1024, 1024, 1)])
@pytest.mark.parametrize("family", ["reference", "quantized"])
def test_equals_quantised_fp16_output(m, n, k, l, family):
    from eval_test_b200 import _lib, inputs, nvfp4_dual_gemm
    gen = inputs.dual_gemm_reference_style if family == "reference" else inputs.dual_gemm_quantized
    data = gen(m, n, k, l, seed=5, device="cuda")
    op, sf, sf_p = nvfp4_dual_gemm.custom_kernel_nvfp4(data, alpha=0.75, ref_scales=True)
    torch.cuda.synchronize()
    assert _lib.device_status(torch.cuda.current_device()) == 0
    from eval_test_b200 import nvfp4_dual_gemm as d2, quantize
    c = d2.custom_kernel(data, alpha=0.75)
    op2, sf2, sf_p2 = quantize.quantize_operand(c.permute(2, 0, 1).contiguous().float())
    torch.cuda.synchronize()
    assert op.shape == op2.shape and op.stride() == op2.stride()
    assert torch.equal(op.view(torch.uint8), op2.view(torch.uint8))
    assert torch.equal(sf.view(torch.uint8), sf2.view(torch.uint8))
    assert sf_p.shape == sf_p2.shape and sf_p.stride() == sf_p2.stride()
    assert torch.equal(sf_p.view(torch.uint8), sf_p2.view(torch.uint8))     # padding rows included


def test_feeds_the_next_gemm(oracle):
    """up-projection with gating -> NVFP4 -> down-projection, against the oracle on the same operand bytes."""
    from eval_test_b200 import inputs, nvfp4_dual_gemm, nvfp4_gemm, quantize
    m, hidden, inter = 256, 256, 512
    up = inputs.dual_gemm_quantized(m, inter, hidden, 1, seed=11, device="cuda")
    h, _, h_sf_p = nvfp4_dual_gemm.custom_kernel_nvfp4(up)
    g = torch.Generator(device="cuda").manual_seed(12)
    w, w_sf, w_sf_p = quantize.quantize_operand(torch.randn((1, hidden, inter), generator=g, device="cuda"))
    c = torch.empty((1, m, hidden), dtype=torch.float16, device="cuda").permute(1, 2, 0)
    data = (h, w, None, w_sf, h_sf_p, w_sf_p, c)
    nvfp4_gemm.custom_kernel(data)
    torch.cuda.synchronize()
    got = torch.from_numpy(out_np(c))
    want = torch.from_numpy(oracle.c_gemm(*gemm_oracle_args(data)))
    from eval_test_b200 import check
    assert check.verbose_allclose(got, want, rtol=1e-3, atol=1e-3) == []


def test_bad_arguments_are_rejected():
    from eval_test_b200 import _lib
    lib = _lib.load()
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    assert lib.nvfp4_dual_gemm_nvfp4(p, p, p, p, p, p, p, p, 128, 100, 256, 1, 1.0, None) == -4    # N % 128
    assert lib.nvfp4_dual_gemm_nvfp4(p, p, p, p, p, p, p + 16, p, 128, 128, 256, 1, 1.0, None) == -5  # 32-byte output
    assert lib.nvfp4_dual_gemm_nvfp4(p, p, p, p, p, p, p, None, 128, 128, 256, 1, 1.0, None) == -1
