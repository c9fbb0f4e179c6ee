"""The CPU oracle against known answers and against itself (C restatement vs numpy restatement)."""
import numpy as np
import pytest
import torch

from _util import dual_oracle_args, gemm_oracle_args, grouped_oracle_args, operand_np, scales_np
from eval_test_b200 import formats as F, inputs


def test_e4m3_decode_all_codes_match_torch_cast(oracle):
    """All 256 e4m3fn codes against PyTorch's own CPU cast (the dtype the reference stores scales in,
    eval/common/scale_helpers.py:38)."""
    codes = torch.arange(256, dtype=torch.uint8)
    want = codes.view(torch.float8_e4m3fn).float().numpy()
    got_np = oracle.np_e4m3_decode(codes.numpy())
    got_c = np.array([oracle._load().oracle_e4m3_decode(int(c)) for c in codes], dtype=np.float32)
    for got in (got_np, got_c):
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert np.array_equal(got[~np.isnan(want)], want[~np.isnan(want)])


def test_e2m1_decode_table(oracle):
    want = [0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6]
    got = [oracle._load().oracle_e2m1_decode(c) for c in range(16)]
    assert got == want and np.signbit(got[8])
    assert oracle.np_unpack_e2m1(np.array([0x21, 0xF9], dtype=np.uint8)).tolist() == [0.5, 1.0, -0.5, -6.0]


def test_sf_offset_formula_matches_reference_layout(oracle):
    """oracle_sf_offset against the golden output of the reference's to_blocked."""
    from pathlib import Path
    gold = np.load(Path(__file__).parent / "golden" / "layout_golden.npz")
    sf, blocked = gold["tb2_in"], gold["tb2_out"]
    rows, kbs = sf.shape
    lib = oracle._load()
    for r in (0, 1, 31, 32, 127, 128, 200, rows - 1):
        for kb in (0, 1, 3, 4, 5, kbs - 1):
            assert blocked[lib.oracle_sf_offset(r, kb, 0, rows, kbs * 16)] == sf[r, kb]
    assert np.array_equal(oracle.np_unswizzle_sf(blocked, rows, kbs * 16, 1)[0], sf)


def test_known_answer_gemm(oracle):
    """Hand-computable case: A row = all 1.0 with scale 2, B row = all 1.5 with scale 3 -> 2*3*1.5*K."""
    M, N, K = 128, 128, 64
    a = np.full((1, M, K // 2), 0x22, dtype=np.uint8)       # 1.0, 1.0
    b = np.full((1, N, K // 2), 0x33, dtype=np.uint8)       # 1.5, 1.5
    b[0, 5] = 0xB3                                          # row 5: (+1.5, -1.5) pairs -> 0
    sfa = np.full(F.sf_buffer_bytes(M, K), 0x40, dtype=np.uint8)   # 2.0
    sfb = np.full(F.sf_buffer_bytes(N, K), 0x44, dtype=np.uint8)   # 3.0
    for fn in (oracle.c_gemm, oracle.np_gemm):
        c = fn(a, b, sfa, sfb, 0.5)
        assert c.shape == (1, M, N)
        assert (np.delete(c[0], 5, axis=1) == 0.5 * 2 * 3 * 1.5 * K).all()
        assert (c[0][:, 5] == 0).all()


def test_known_answer_gemv_uses_row_zero_only(oracle):
    M, K = 128, 128
    a = np.full((1, M, K // 2), 0x22, dtype=np.uint8)
    x = np.full((1, 128, K // 2), 0x77, dtype=np.uint8)     # rows 1..127 hold 6.0 and must be ignored
    x[0, 0] = 0x11                                          # the vector: 0.5
    one = np.full(F.sf_buffer_bytes(128, K), 0x38, dtype=np.uint8)
    for fn in (oracle.c_gemv, oracle.np_gemv):
        assert (fn(a, x, one, one) == 0.5 * K).all()


@pytest.mark.parametrize("gen", [inputs.gemm_reference_style, inputs.gemm_quantized])
def test_c_and_numpy_oracles_agree_gemm(oracle, gen):
    args = gemm_oracle_args(gen(128, 256, 512, 2, seed=0, device="cpu"))
    c1, c2 = oracle.c_gemm(*args, 0.5), oracle.np_gemm(*args, 0.5)
    assert np.abs(c1.astype(np.float32) - c2.astype(np.float32)).max() <= 1e-3 * np.abs(c2.astype(np.float32)).max()
    if gen is inputs.gemm_reference_style:       # dyadic data: fp32 accumulation is exact in any order
        assert np.array_equal(c1.view(np.uint16), c2.view(np.uint16))


def test_c_and_numpy_oracles_agree_gemv_dual(oracle):
    a, b, _, _, sa, sb, _ = inputs.gemv_reference_style(256, 512, 2, seed=0, device="cpu")
    args = (operand_np(a), operand_np(b), scales_np(sa), scales_np(sb))
    assert np.array_equal(oracle.c_gemv(*args).view(np.uint16), oracle.np_gemv(*args).view(np.uint16))
    args = dual_oracle_args(inputs.dual_gemm_reference_style(128, 256, 512, 1, seed=0, device="cpu"))
    c1, c2 = oracle.c_dual_gemm(*args).astype(np.float32), oracle.np_dual_gemm(*args).astype(np.float32)
    assert np.all(np.abs(c1 - c2) <= 1e-3 + 1e-3 * np.abs(c2))


def test_grouped_oracle_ragged_and_empty(oracle):
    data = inputs.grouped_gemm_quantized([40, 0, 200], [128, 256, 128], [256, 256, 512], 3, seed=0, device="cpu")
    outs = oracle.c_grouped_gemm(grouped_oracle_args(data))
    assert [o.shape for o in outs] == [(40, 128), (0, 256), (200, 128)]
    a, b, sa, sb = grouped_oracle_args(data)[2]
    want = oracle.np_gemm(a[None], b[None], sa, sb)[0].astype(np.float32)
    assert np.all(np.abs(outs[2].astype(np.float32) - want) <= 1e-3 + 1e-3 * np.abs(want))


def test_config0_gemm_oracle_self_consistency(oracle):
    """The CPU-runnable configuration: M=128, N=256, K=512, N(0,1) seed 0 through the quantiser, alpha = 1:
    the result must track the unquantised fp32 product within the quantisation noise."""
    g = torch.Generator().manual_seed(0)
    A, B = torch.randn((128, 512), generator=g), torch.randn((256, 512), generator=g)
    pa, sa = F.quantize_nvfp4(A)
    pb, sb = F.quantize_nvfp4(B)
    c = oracle.c_gemm(pa[None].numpy(), pb[None].numpy(), F.swizzle_scales(sa[None]).numpy(),
                      F.swizzle_scales(sb[None]).numpy())[0].astype(np.float32)
    exact = (A @ B.T).numpy()
    rel = np.linalg.norm(c - exact) / np.linalg.norm(exact)
    assert 0.05 < rel < 0.25     # fp4 quantisation noise of two operands (about 0.13), far from 0 or 1


# ------------------------------------------------------------------ pins against cuBLASLt outputs recorded on a B200
def _gold():
    from pathlib import Path
    return np.load(Path(__file__).parent / "golden" / "scaled_mm_golden.npz")


@pytest.mark.parametrize("tag", ["gemm0", "gemm1", "grp0", "grp1"])
def test_oracle_matches_recorded_scaled_mm_dyadic(oracle, tag):
    """Reference-style (dyadic) inputs: the oracle must reproduce torch._scaled_mm bit for bit - this pins the
    nibble order, the e2m1 / e4m3 tables, the transposition and the scale layout."""
    g = _gold()
    for fn in (oracle.c_gemm, oracle.np_gemm):
        got = fn(g[f"{tag}_a"], g[f"{tag}_b"], g[f"{tag}_sfa"], g[f"{tag}_sfb"])
        assert np.array_equal(got.view(np.uint16), g[f"{tag}_c"].view(np.uint16))


def test_oracle_matches_recorded_scaled_mm_gemv(oracle):
    g = _gold()
    for fn in (oracle.c_gemv, oracle.np_gemv):
        got = fn(g["gemv_a"], g["gemv_x"], g["gemv_sfa"], g["gemv_sfx"])
        assert np.array_equal(got.view(np.uint16), g["gemv_c"].view(np.uint16))


def test_oracle_matches_recorded_scaled_mm_inexact(oracle):
    """N(0,1)-quantised GEMM and the dual GEMM (U[0,1) scales): accumulation order inside the library is not
    specified, so the harness's own tolerance (rtol = atol = 1e-3) applies."""
    g = _gold()
    got = oracle.c_gemm(g["gemmq_a"], g["gemmq_b"], g["gemmq_sfa"], g["gemmq_sfb"]).astype(np.float32)
    want = g["gemmq_c"].astype(np.float32)
    assert np.all(np.abs(got - want) <= 1e-3 + 1e-3 * np.abs(want))
    got = oracle.c_dual_gemm(g["dual_a"], g["dual_b1"], g["dual_b2"], g["dual_sfa"], g["dual_sfb1"],
                             g["dual_sfb2"]).astype(np.float32)
    want = g["dual_c"].astype(np.float32)
    assert np.all(np.abs(got - want) <= 1e-3 + 1e-3 * np.abs(want))
