"""The bench's bookkeeping on CPU: algorithmic work per configuration (the roofline's numerator) and how the
configurations are split over ranks.  No kernel runs here."""
import importlib.util
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench_module"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_work_matches_the_configurations():
    b = _bench()
    assert b.GemvWorkload().work() == 604_147_712                      # 4 batches of 151 036 928 bytes
    assert b.GemmWorkload().work() == 2 * 8192 ** 3 == 1_099_511_627_776
    assert b.DualGemmWorkload().work() == 4 * 4096 * 14336 * 4096 == 962_072_674_304
    g = b.GroupedGemmWorkload()
    assert len(g.ms) == 64 and sum(m == 0 for m in g.ms) == 0 and 1.1e9 < g.work() < 1.2e9
    e = b.GroupedGemmWorkload(forced_empty=b.FORCED_EMPTY)
    assert sum(m == 0 for m in e.ms) == 5 and e.work() < g.work()
    assert e.name != g.name


def test_strong_scaling_splits_conserve_the_job():
    b = _bench()
    gemm = b.GemmWorkload()
    assert all(gemm.work(w) * w == gemm.job(w) == gemm.work(1) for w in (1, 2, 4, 8))
    rows = b.GemvWorkload(strong=True)
    assert rows.scaling == "strong" and rows._rows(8) == 2048
    assert rows.job(8) == 8 * rows.work(8) and abs(rows.job(8) - rows.job(1)) < 8 * 4 * (16384 // 2 + 16384 // 16)
    weak = b.GemvWorkload()
    assert weak.scaling == "weak" and weak.job(8) == 8 * weak.work(1)


def test_groups_are_dealt_by_weight_bytes():
    b = _bench()
    for wl in (b.GroupedGemmWorkload(), b.GroupedGemmWorkload(forced_empty=b.FORCED_EMPTY)):
        for world in (2, 4, 8):
            parts = [wl._mine(r, world) for r in range(world)]
            assert sorted(m for p in parts for m in p) == sorted(wl.ms)
            live = [sum(m > 0 for m in p) for p in parts]
            assert max(live) - min(live) <= 1                          # weights (non-empty groups) balanced
            assert wl.job(world) == wl._bytes(wl.ms) >= wl.work(world)


def test_default_run_covers_every_configuration():
    b = _bench()
    assert b.DEFAULT_SET == ("gemv", "gemm", "dual_gemm", "grouped_gemm", "grouped_gemm_empty")
    assert all(name in b.WORKLOADS for name in b.DEFAULT_SET + ("gemv_rowsplit", "gemm_gather_fused", "gemm_gather_nccl"))
