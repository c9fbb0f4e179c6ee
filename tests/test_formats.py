"""Host-side formats, layouts, generators, spec parser and checkers (CPU only)."""
from pathlib import Path

import numpy as np
import pytest
import torch

from eval_test_b200 import check, formats as F, inputs, spec

GOLD = np.load(Path(__file__).parent / "golden" / "layout_golden.npz")


@pytest.mark.parametrize("i", range(4))
def test_swizzle_matches_reference_to_blocked(i):
    sf = torch.from_numpy(GOLD[f"tb{i}_in"])
    assert np.array_equal(F.swizzle_scales(sf[None]).numpy(), GOLD[f"tb{i}_out"])


@pytest.mark.parametrize("i", range(3))
def test_swizzle_padded_matches_reference(i):
    """Ragged row counts: rows are zero-padded to 128 (the grouped task's to_blocked)."""
    sf = torch.from_numpy(GOLD[f"tbp{i}_in"])
    assert np.array_equal(F.swizzle_scales(sf[None]).numpy(), GOLD[f"tbp{i}_out"])


def test_permuted_view_matches_reference_scatter():
    idx = GOLD["scatter_index"]            # [mn, sf_k, l, 6]
    mn, sf_k, l = idx.shape[:3]
    sf = torch.randint(0, 256, (l, mn, sf_k), dtype=torch.uint8)
    pv = F.permuted_view(F.swizzle_scales(sf), mn, sf_k * 16, l).view(torch.uint8)
    assert pv.shape == (32, 4, mn // 128, 4, sf_k // 4, l)
    got = pv[tuple(torch.from_numpy(idx[..., d]).long() for d in range(6))]   # [mn, sf_k, l]
    assert torch.equal(got, sf.permute(1, 2, 0))


def test_swizzle_roundtrip_ragged():
    sf = torch.randint(0, 256, (3, 200, 10), dtype=torch.uint8)
    buf = F.swizzle_scales(sf)
    assert buf.numel() == F.sf_buffer_bytes(200, 160, 3) == 3 * 2 * 3 * 512
    assert torch.equal(F.unswizzle_scales(buf, 200, 160, 3), sf)


def test_e2m1_rounding_is_nearest_even():
    y = torch.tensor([0.0, 0.24, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.01, 7.0, -0.25, -0.75, -6.5, -0.1])
    want = [0, 0, 0, 1, 2, 2, 4, 4, 6, 6, 7, 7, 8, 8 | 2, 8 | 7, 8]
    assert F.round_to_e2m1_code(y).tolist() == want


def test_quantizer_properties(oracle):
    g = torch.Generator().manual_seed(0)
    x = torch.randn((64, 256), generator=g)
    x[3, 16:32] = 0                      # an all-zero block
    x[5, 0] = 1e4                        # a block whose scale would overflow e4m3 without the clamp
    packed, sf = F.quantize_nvfp4(x)
    assert packed.shape == (64, 128) and sf.shape == (64, 16)
    assert sf[3, 1] == 0 and (packed[3, 8:16] == 0).all()
    scale = torch.from_numpy(oracle.np_e4m3_decode(sf.numpy()))
    assert torch.isfinite(scale).all() and scale[5, 0] == 448
    deq = torch.from_numpy(oracle.np_unpack_e2m1(packed.numpy())).reshape(64, 16, 16) * scale[..., None]
    xb = x.reshape(64, 16, 16)
    amax = xb.abs().amax(-1, keepdim=True)
    ok = amax.squeeze(-1) <= 448 * 6
    # each value within half an e2m1 step (step <= 2 at the top of the grid) of x/scale, i.e. error <= scale
    assert ((deq - xb).abs() <= scale[..., None] * 1.0 + 1e-6)[ok].all()
    # scale is amax/6 rounded to e4m3: relative error at most 2^-4
    nz = (amax.squeeze(-1) > 1e-3) & ok
    assert ((scale - amax.squeeze(-1) / 6).abs() <= amax.squeeze(-1) / 6 / 16 + 1e-9)[nz].all()


def test_generators_shapes_and_strides():
    a, b, sfa, sfb, sfa_p, sfb_p, c = inputs.gemm_reference_style(128, 256, 512, 2, seed=1, device="cpu")
    assert a.shape == (128, 256, 2) and a.stride() == (256, 1, 128 * 256) and a.dtype == torch.float4_e2m1fn_x2
    assert b.shape == (256, 256, 2) and c.shape == (128, 256, 2) and c.stride() == (256, 1, 128 * 256)
    assert sfa.shape == (128, 32, 2) and sfa.dtype == torch.float8_e4m3fn
    assert sfa_p.shape == (32, 4, 1, 4, 8, 2) and sfb_p.shape == (32, 4, 2, 4, 8, 2)
    assert sfb_p.stride() == F.permuted_strides(256, 512)
    assert set(sfa.view(torch.uint8).unique().tolist()) <= {0x00, 0x38, 0x40, 0x44}   # 0, 1, 2, 3
    again = inputs.gemm_reference_style(128, 256, 512, 2, seed=1, device="cpu")
    assert torch.equal(again[0].view(torch.uint8), a.view(torch.uint8))
    other = inputs.gemm_reference_style(128, 256, 512, 2, seed=2, device="cpu")
    assert not torch.equal(other[0].view(torch.uint8), a.view(torch.uint8))

    a, b, *_, c = inputs.gemv_reference_style(256, 512, 2, seed=1, device="cpu")
    assert b.shape == (128, 256, 2) and c.shape == (256, 1, 2) and c.stride()[2] == 256
    assert int(a.view(torch.uint8).max()) <= 3

    d = inputs.dual_gemm_reference_style(128, 256, 256, 1, seed=1, device="cpu")
    assert len(d) == 10 and int((d[1].view(torch.uint8) & 0x44).max()) == 0

    abc, sfs, sfs_p, sizes = inputs.grouped_gemm_reference_style([96, 128], [128, 256], [256, 512], 2, 1, "cpu")
    assert sizes == [(96, 128, 256, 1), (128, 256, 512, 1)]
    assert abc[0][0].shape == (96, 128, 1) and sfs_p[0][0].shape == (32, 4, 1, 4, 4, 1)
    assert set(sfs_p[0][0].view(torch.uint8).unique().tolist()) <= {0x38, 0x40}        # padding rows included


def test_poisson_group_sizes_are_seeded_and_clipped():
    m = inputs.poisson_group_sizes(64, 128.0, 0, 1024, seed=0)
    assert m == inputs.poisson_group_sizes(64, 128.0, 0, 1024, seed=0)
    assert len(m) == 64 and all(0 <= v <= 1024 for v in m) and 100 < sum(m) / 64 < 160


def test_spec_parser():
    text = "m: 128; k: 256; l: 1; seed: 1111\nm: [96, 128]; n: (128, 256); g: 2; seed: 5; mode: fast"
    cases = spec.parse_cases(text)
    assert cases[0].args == {"m": 128, "k": 256, "l": 1, "seed": 1111}
    assert cases[1].args == {"m": [96, 128], "n": (128, 256), "g": 2, "seed": 5, "mode": "fast"}
    seeded = spec.parse_cases(text, seed=42)
    assert seeded[0].args["seed"] == spec.combine(1111, 42) == 1111 + (1153 * 1154) // 2
    for bad in ("m 128", "m: ", "m1: 3", "m: [1, 2", "m: a-b"):
        with pytest.raises(ValueError):
            spec.parse_cases(bad)


def test_checkers():
    ref = torch.tensor([1.0, 2.0, float("nan"), float("inf"), 0.0])
    assert check.verbose_allclose(ref.clone(), ref, 1e-3, 1e-3) == []
    off = ref.clone()
    off[1] = 2.01
    assert check.verbose_allclose(off, ref, 1e-3, 1e-3)[0] == "Number of mismatched elements: 1"
    nan_moved = torch.tensor([1.0, float("nan"), 2.0, float("inf"), 0.0])
    assert check.verbose_allclose(nan_moved, ref, 1e-3, 1e-3)
    assert check.verbose_allclose(ref[:3], ref, 1e-3, 1e-3) == ["SIZE MISMATCH"]
    assert check.compare_nested([ref, ref], [ref], 1e-3, 1e-3) == ["LENGTH MISMATCH"]
    assert check.compare_nested([ref, off], [ref, ref], 1e-3, 1e-3)[0].startswith("[1]: ")
    ok, msg = check.make_match_reference(lambda d: d, rtol=1e-3, atol=1e-3)(ref, ref.clone())
    assert ok and msg == ""
    assert check.max_delta_ok(torch.tensor([1.0, 100.5]), torch.tensor([1.0, 100.0]))[0]
    assert not check.max_delta_ok(torch.tensor([3.0, 100.0]), torch.tensor([1.0, 100.0]))[0]
