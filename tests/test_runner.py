"""The local runner: protocol pieces on CPU, whole runs on the GPU."""
import os

import pytest


def test_stats_match_the_reference_formula():
    from eval_test_b200 import runner
    st = runner.calculate_stats([100.0, 110.0, 90.0, 100.0])
    assert st.runs == 4 and st.mean == 100.0 and st.best == 90.0 and st.worst == 110.0
    assert abs(st.std - (200.0 / 3) ** 0.5) < 1e-12 and abs(st.err - st.std / 2.0) < 1e-12


def test_usage_and_bad_spec_exit_codes(tmp_path, capsys):
    from eval_test_b200 import runner
    assert runner.main(["nonsense"]) == 2
    assert runner.main(["test", "nvfp4_gemm", str(tmp_path / "missing.txt")]) == 113
    bad = tmp_path / "bad.txt"
    bad.write_text("m 128; n: 3")
    assert runner.main(["test", "nvfp4_gemm", str(bad)]) == 113
    capsys.readouterr()


def test_sampling_modes_follow_the_reference_runners():
    """GEMM one call per sample; GEMV and dual GEMM batches of 50; grouped GEMM batches of 15
    (eval/nvfp4_gemm/eval.py:13, eval/nvfp4_gemv/eval.py:11-12, eval/nvfp4_dual_gemm/eval.py:11-12,
    eval/common/eval_base.py:141-142)."""
    from eval_test_b200 import runner
    assert runner.SAMPLING == {"nvfp4_gemm": (False, 1), "nvfp4_gemv": (True, 50), "nvfp4_dual_gemm": (True, 50),
                               "nvfp4_grouped_gemm": (True, 15)}


def test_report_parses_a_log_and_renders_floors():
    from eval_test_b200 import report
    log = "\n".join([
        "benchmark-count: 1", "benchmark.0.spec: m: 128; n: 7168; k: 16384; l: 1; seed: 1111", "benchmark.0.runs: 5",
        "benchmark.0.mean: 29000.0", "benchmark.0.std: 100.0", "benchmark.0.err: 44.7", "benchmark.0.best: 28000.0",
        "benchmark.0.worst: 30000.0", "check: pass"])
    data = report.parse_log(log)
    assert data["check"] == "pass" and data["benchmark_count"] == 1 and data["benchmarks"][0]["runs"] == "5"
    by, fl = report.work_of("nvfp4_gemm", {"m": 128, "n": 7168, "k": 16384, "l": 1})
    assert fl == 2 * 128 * 7168 * 16384
    assert by == (128 + 7168) * (16384 // 2 + 16384 // 16) + 2 * 128 * 7168
    text = report.format_report(data, "benchmark", "nvfp4_gemm")
    assert "success" in text and "29.0" in text and "28.0" in text
    tests = report.parse_log("test-count: 2\ntest.0.spec: m: 1\ntest.0.status: pass\ntest.1.spec: m: 2\n"
                             "test.1.status: fail\ntest.1.error: mismatch\ncheck: fail")
    text = report.format_report(tests, "test", "nvfp4_gemm")
    assert "failure" in text and "fail: mismatch" in text
    by_g, fl_g = report.work_of("nvfp4_grouped_gemm", {"m": [0, 100], "n": [256, 256], "k": [512, 512]})
    assert fl_g == 2 * 100 * 256 * 512


def test_stop_rule_needs_three_samples_and_100_ms():
    import time
    from eval_test_b200 import runner
    start = time.perf_counter_ns()
    assert not runner._enough([1.0, 1.0, 1.0], 2, start, 1e9)            # wall time below 100 ms
    long_ago = start - int(2e8)
    assert not runner._enough([1.0, 1.0], 1, long_ago, 1e9)             # fewer than three samples
    assert runner._enough([100.0, 100.0, 100.0], 2, long_ago, 1e9)      # error of the mean below 0.1 %
    assert not runner._enough([100.0, 150.0, 50.0], 2, long_ago, 1e9)   # noisy, budget left
    assert runner._enough([100.0, 150.0, 50.0], 2, long_ago, 200.0)     # budget used up


def _run(mode, task, text, tmp_path, monkeypatch):
    from eval_test_b200 import runner
    specfile = tmp_path / "cases.txt"
    specfile.write_text(text)
    r, w = os.pipe()
    monkeypatch.setenv("POPCORN_FD", str(w))
    monkeypatch.setenv("POPCORN_SEED", "42")
    code = runner.main([mode, task, str(specfile)])
    with os.fdopen(r) as f:   # the runner closed its end when the Logger's file went away
        lines = dict(line.split(": ", 1) for line in f.read().splitlines() if ": " in line)
    return code, lines


@pytest.mark.gpu
@pytest.mark.parametrize("task,text", [
    ("nvfp4_gemv", "m: 128; k: 256; l: 1; seed: 1111\nm: 512; k: 1536; l: 2; seed: 1111"),
    ("nvfp4_gemm", "m: 128; n: 256; k: 256; l: 1; seed: 1111\nm: 512; n: 512; k: 7168; l: 1; seed: 1111"),
    ("nvfp4_dual_gemm", "m: 256; n: 512; k: 256; l: 1; seed: 1111"),
    ("nvfp4_grouped_gemm", "m: [96, 128]; n: [128, 256]; k: [256, 512]; g: 2; seed: 1111\n"
                           "m: [40, 56, 384, 512]; n: [512, 384, 256, 128]; k: [256, 256, 256, 256]; g: 4; seed: 1111"),
])
def test_test_mode_passes_against_scaled_mm(task, text, tmp_path, monkeypatch):
    """The kernels pass the harness's own acceptance check (torch._scaled_mm, rtol = atol = 1e-3) on shapes
    taken from its test lists."""
    code, lines = _run("test", task, text, tmp_path, monkeypatch)
    n = len(text.splitlines())
    assert code == 0, lines
    assert lines["test-count"] == str(n) and lines["check"] == "pass"
    assert all(lines[f"test.{i}.status"] == "pass" for i in range(n))


@pytest.mark.gpu
@pytest.mark.parametrize("mode,task,text", [
    ("benchmark", "nvfp4_gemv", "m: 7168; k: 2048; l: 4; seed: 1111"),          # batches of 50
    ("benchmark", "nvfp4_gemm", "m: 128; n: 4096; k: 7168; l: 1; seed: 1111"),   # one call per sample
    ("leaderboard", "nvfp4_gemm", "m: 128; n: 7168; k: 2048; l: 1; seed: 1111"), # fresh inputs and a re-check per repeat
    ("leaderboard", "nvfp4_grouped_gemm", "m: [128, 384]; n: [4096, 4096]; k: [1536, 1536]; g: 2; seed: 1111"),
])
def test_benchmark_modes_report_stats(mode, task, text, tmp_path, monkeypatch):
    code, lines = _run(mode, task, text, tmp_path, monkeypatch)
    assert code == 0, lines
    assert lines["check"] == "pass" and "benchmark.0.status" not in lines
    assert int(lines["benchmark.0.runs"]) >= 3 and 1e3 < float(lines["benchmark.0.mean"]) < 1e8


@pytest.mark.gpu
def test_profile_mode_logs_a_table(tmp_path, monkeypatch):
    import base64
    code, lines = _run("profile", "nvfp4_gemm", "m: 128; n: 256; k: 256; l: 1; seed: 1111", tmp_path, monkeypatch)
    assert code == 0, lines
    table = base64.b64decode(lines["benchmark.0.report"], b"+*").decode()
    assert "gemm" in table
