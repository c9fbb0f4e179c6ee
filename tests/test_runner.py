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
def test_benchmark_mode_reports_stats(tmp_path, monkeypatch):
    code, lines = _run("benchmark", "nvfp4_gemv", "m: 7168; k: 2048; l: 4; seed: 1111", tmp_path, monkeypatch)
    assert code == 0, lines
    assert int(lines["benchmark.0.runs"]) >= 3 and 1e3 < float(lines["benchmark.0.mean"]) < 1e8
