"""GPU quantiser against the torch-op quantiser: bit for bit."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("L,rows,K", [(1, 128, 256), (2, 200, 320), (1, 1, 16), (3, 384, 4096)])
def test_quantize_kernel_matches_torch_quantizer(L, rows, K):
    from eval_test_b200 import formats as F, quantize
    g = torch.Generator(device="cuda").manual_seed(L * 1000 + rows)
    x = torch.randn((L, rows, K), generator=g, device="cuda")
    x[0, 0, :16] = 0                      # an all-zero block
    x[0, -1, -16:] *= 1e4                 # a block whose scale saturates at 448
    if K >= 32:
        x[0, 0, 16:32] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5,
                                       -3.5, -5.0, -6.0], device="cuda")   # ties on the e2m1 grid at scale 1
    op, sf, sf_p = quantize.quantize_operand(x)
    want_packed, want_sf = F.quantize_nvfp4(x)
    assert torch.equal(op.view(torch.uint8).permute(2, 0, 1), want_packed)
    assert torch.equal(sf.view(torch.uint8).permute(2, 0, 1), want_sf)
    assert torch.equal(sf_p.view(torch.uint8).permute(5, 2, 4, 0, 1, 3).reshape(-1), F.swizzle_scales(want_sf))
    # and the CPU path gives the same bits, so seeded CPU fixtures and GPU-quantised data agree
    cpu_packed, cpu_sf = F.quantize_nvfp4(x.cpu())
    assert torch.equal(cpu_packed, want_packed.cpu()) and torch.equal(cpu_sf, want_sf.cpu())


def test_quantized_operands_feed_the_gemm(oracle):
    import numpy as np
    from _util import gemm_oracle_args, out_np
    from eval_test_b200 import check, nvfp4_gemm, quantize
    g = torch.Generator(device="cuda").manual_seed(1)
    a, sfa, sfa_p = quantize.quantize_operand(torch.randn((1, 256, 512), generator=g, device="cuda"))
    b, sfb, sfb_p = quantize.quantize_operand(torch.randn((1, 384, 512), generator=g, device="cuda"))
    c = torch.empty((1, 256, 384), dtype=torch.float16, device="cuda").permute(1, 2, 0)
    data = (a, b, sfa, sfb, sfa_p, sfb_p, c)
    nvfp4_gemm.custom_kernel(data)
    torch.cuda.synchronize()
    want = torch.from_numpy(oracle.c_gemm(*gemm_oracle_args(data)))
    assert check.verbose_allclose(torch.from_numpy(out_np(c)), want, rtol=1e-3, atol=1e-3) == []


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L,rows,K", [(1, 128, 256), (2, 200, 320), (1, 3, 16), (1, 512, 2048)])
def test_half_precision_inputs_quantise_like_their_fp32_value(dtype, L, rows, K):
    """fp16 / bf16 activations: widening to fp32 is exact, so the result must equal quantising x.float()."""
    from eval_test_b200 import quantize
    g = torch.Generator(device="cuda").manual_seed(7 * rows + K)
    x = (torch.randn((L, rows, K), generator=g, device="cuda") * 3).to(dtype)
    x[0, 0, :16] = 0
    x[0, -1, -16:] = 6e4 if dtype == torch.float16 else 3e38    # scale saturates
    op, sf, sf_p = quantize.quantize_operand(x)
    op32, sf32, sf_p32 = quantize.quantize_operand(x.float())
    assert torch.equal(op.view(torch.uint8), op32.view(torch.uint8))
    assert torch.equal(sf.view(torch.uint8), sf32.view(torch.uint8))
    assert torch.equal(sf_p.view(torch.uint8), sf_p32.view(torch.uint8))
