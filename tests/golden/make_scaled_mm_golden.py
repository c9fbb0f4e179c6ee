"""Generates ``scaled_mm_golden.npz`` on a B200: outputs of ``torch._scaled_mm`` (cuBLASLt NVFP4), the library
call that defines the reference's results, on small seeded inputs.

    python tests/golden/make_scaled_mm_golden.py [out.npz]

The reference's ``ref_kernel`` functions are this call and nothing else
(eval/nvfp4_gemm/reference.py:16-27, eval/nvfp4_gemv/reference.py:16-27,
eval/nvfp4_dual_gemm/reference.py:19-44, eval/nvfp4_grouped_gemm/reference.py:57-72):

    torch._scaled_mm(a[:, :, l], b[:, :, l].transpose(0, 1), to_blocked(sfa[:, :, l]), to_blocked(sfb[:, :, l]),
                     bias=None, out_dtype=torch.float16)            # float32 twice + silu(r1) * r2 for the dual GEMM

The reference checkout cannot travel to the GPU machine, so the call is restated here; ``to_blocked`` of a
row-major scale matrix is ``formats.swizzle_scales`` (pinned against the reference's own function by
``layout_golden.npz``).  Inputs come from the CPU generators (same tensors on every machine) and are stored next
to the outputs, so the fixture is self-contained.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from _util import operand_np, scales_np, to_device  # noqa: E402
from eval_test_b200 import formats as F, inputs  # noqa: E402

E4M3 = torch.float8_e4m3fn


def scaled_mm(a, b, sfa_ref, sfb_ref, l, out_dtype):
    """One batch, exactly as the reference calls it (scales re-swizzled from the row-major tensors, zero padded)."""
    sa = F.swizzle_scales(sfa_ref[:, :, l].view(torch.uint8)[None].contiguous()).view(E4M3)
    sb = F.swizzle_scales(sfb_ref[:, :, l].view(torch.uint8)[None].contiguous()).view(E4M3)
    return torch._scaled_mm(a[:, :, l], b[:, :, l].transpose(0, 1), sa, sb, bias=None, out_dtype=out_dtype)


def main(out_path):
    out = {}

    def put_operands(tag, names, tensors):
        for n, t in zip(names, tensors):
            out[f"{tag}_{n}"] = operand_np(t)

    for i, (m, n, k, l, seed) in enumerate([(128, 256, 256, 1, 11), (256, 128, 512, 2, 12)]):
        data = to_device(inputs.gemm_reference_style(m, n, k, l, seed, device="cpu"))
        a, b, sfa, sfb, sfa_p, sfb_p, _ = data
        c = torch.stack([scaled_mm(a, b, sfa, sfb, li, torch.float16) for li in range(l)])
        put_operands(f"gemm{i}", ["a", "b"], [a, b])
        out[f"gemm{i}_sfa"], out[f"gemm{i}_sfb"] = scales_np(sfa_p), scales_np(sfb_p)
        out[f"gemm{i}_c"] = c.cpu().numpy()

    data = to_device(inputs.gemm_quantized(128, 128, 512, 1, 13, device="cpu"))
    a, b, sfa, sfb, sfa_p, sfb_p, _ = data
    put_operands("gemmq", ["a", "b"], [a, b])
    out["gemmq_sfa"], out["gemmq_sfb"] = scales_np(sfa_p), scales_np(sfb_p)
    out["gemmq_c"] = scaled_mm(a, b, sfa, sfb, 0, torch.float16)[None].cpu().numpy()

    data = to_device(inputs.gemv_reference_style(128, 512, 2, 14, device="cpu"))
    a, b, sfa, sfb, sfa_p, sfb_p, _ = data
    c = torch.stack([scaled_mm(a, b, sfa, sfb, li, torch.float16)[:, 0] for li in range(2)])
    put_operands("gemv", ["a", "x"], [a, b])
    out["gemv_sfa"], out["gemv_sfx"] = scales_np(sfa_p), scales_np(sfb_p)
    out["gemv_c"] = c.cpu().numpy()

    data = to_device(inputs.dual_gemm_reference_style(128, 128, 256, 1, 15, device="cpu"))
    a, b1, b2, sfa, sfb1, sfb2, sfa_p, sfb1_p, sfb2_p, _ = data
    r1 = scaled_mm(a, b1, sfa, sfb1, 0, torch.float32)
    r2 = scaled_mm(a, b2, sfa, sfb2, 0, torch.float32)
    put_operands("dual", ["a", "b1", "b2"], [a, b1, b2])
    out["dual_sfa"], out["dual_sfb1"], out["dual_sfb2"] = scales_np(sfa_p), scales_np(sfb1_p), scales_np(sfb2_p)
    out["dual_c"] = (torch.nn.functional.silu(r1) * r2).to(torch.float16)[None].cpu().numpy()

    data = to_device(inputs.grouped_gemm_reference_style([96, 128], [128, 256], [256, 512], 2, 16, device="cpu"))
    abc, sfs, sfs_p, _ = data
    for g, ((a, b, _), (sfa, sfb), (sfa_p, sfb_p)) in enumerate(zip(abc, sfs, sfs_p)):
        put_operands(f"grp{g}", ["a", "b"], [a, b])
        out[f"grp{g}_sfa"], out[f"grp{g}_sfb"] = scales_np(sfa_p), scales_np(sfb_p)
        out[f"grp{g}_c"] = scaled_mm(a, b, sfa, sfb, 0, torch.float16)[None].cpu().numpy()

    out["torch_version"] = np.array(torch.__version__)
    out["device"] = np.array(torch.cuda.get_device_name(0))
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, "with", len(out), "arrays on", torch.cuda.get_device_name(0))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else str(Path(__file__).parent / "scaled_mm_golden.npz"))
