"""Local runner for the harness's shape-list files, in place of the remote launcher.

    python -m eval_test_b200.runner test      nvfp4_gemm  tests.txt
    python -m eval_test_b200.runner benchmark nvfp4_gemv  benchmarks.txt

It follows the reference's evaluation protocol (eval/common/eval_base.py): the same spec grammar and seed mixing
(``POPCORN_SEED``), ``key: value`` log lines written to the file descriptor named by ``POPCORN_FD`` (stdout when
unset), ``test.N.status: pass|fail`` with the checker's message on failure, and for benchmarks the statistics
``runs / mean / std / err / best / worst`` in nanoseconds measured with CUDA events around ``custom_kernel(data)``
on the current stream, after a correctness check, with a cold L2 before every timed call, until the relative error
of the mean is below 0.1 %, the time budget is used up or 120 s have passed (eval_base.py:229-295).
Exit codes: 0 all passed, 112 a test or benchmark failed, 113 malformed spec (eval_base.py:67,416).

Differences: everything runs in this process (the reference isolates each test in a spawned worker); the L2 is
flushed by writing a 512 MiB buffer, not by drawing 62.5 GiB of random numbers (eval/common/utils.py:158-160);
inputs come from this package's seeded generators.
"""
from __future__ import annotations

import copy
import math
import os
import sys
import time
from dataclasses import dataclass
from pathlib import Path

from . import spec

TASKS = ("nvfp4_gemv", "nvfp4_gemm", "nvfp4_dual_gemm", "nvfp4_grouped_gemm")


@dataclass
class Stats:
    runs: int
    mean: float
    std: float
    err: float
    best: float
    worst: float


def calculate_stats(durations: list[float]) -> Stats:
    """Mean, sample standard deviation, standard error, best and worst (eval_base.py:112-121)."""
    runs = len(durations)
    avg = sum(durations) / runs
    var = sum((x - avg) ** 2 for x in durations)
    std = math.sqrt(var / (runs - 1)) if runs > 1 else 0.0
    return Stats(runs, avg, std, std / math.sqrt(runs), float(min(durations)), float(max(durations)))


class Logger:
    """``key: value`` lines on the POPCORN file descriptor (eval_base.py:18-33)."""

    def __init__(self, fd: int | None):
        self.file = os.fdopen(fd, "w") if fd is not None else sys.stdout

    def log(self, key, value):
        print(f"{key}: {value}", file=self.file, flush=True)


def _task(task: str):
    """(custom_kernel, generate_input, check_implementation) of a task."""
    from . import inputs, reference_check
    from . import nvfp4_dual_gemm, nvfp4_gemm, nvfp4_gemv, nvfp4_grouped_gemm
    table = {
        "nvfp4_gemv": (nvfp4_gemv.custom_kernel, inputs.gemv_reference_style),
        "nvfp4_gemm": (nvfp4_gemm.custom_kernel, inputs.gemm_reference_style),
        "nvfp4_dual_gemm": (nvfp4_dual_gemm.custom_kernel, inputs.dual_gemm_reference_style),
        "nvfp4_grouped_gemm": (nvfp4_grouped_gemm.custom_kernel, inputs.grouped_gemm_reference_style),
    }
    kernel, gen = table[task]
    return kernel, gen, reference_check.check_implementation(task)


def clone_data(data):
    import torch
    if isinstance(data, torch.Tensor):
        # keep the strides: the kernels take the reference's layouts, not contiguous copies
        out = torch.empty_strided(data.shape, data.stride(), dtype=data.dtype, device=data.device)
        out.view(torch.uint8).copy_(data.view(torch.uint8)) if data.element_size() == 1 else out.copy_(data)
        return out
    if isinstance(data, (list, tuple)):
        return type(data)(clone_data(x) for x in data)
    return copy.copy(data)


class L2Flusher:
    def __init__(self):
        import torch
        self.buf = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self):
        self.buf.fill_(0)


def run_tests(task: str, cases, log: Logger) -> bool:
    import torch
    kernel, gen, check_impl = _task(task)
    ok_all = True
    log.log("test-count", len(cases))
    for i, case in enumerate(cases):
        log.log(f"test.{i}.spec", case.spec)
        try:
            data = gen(**case.args)
            torch.cuda.synchronize()
            out = kernel(clone_data(data))
            torch.cuda.synchronize()
            good, msg = check_impl(data, out)
        except Exception as e:  # a kernel error fails the test, as in the reference (eval_base.py:224-225)
            good, msg = False, f"{type(e).__name__}: {e}"
        log.log(f"test.{i}.status", "pass" if good else "fail")
        if not good:
            log.log(f"test.{i}.error", msg)
            ok_all = False
    log.log("check", "pass" if ok_all else "fail")
    return ok_all


def benchmark_case(task: str, args: dict, flush, max_time_ns: float = 10e9, max_repeats: int = 200):
    import torch
    kernel, gen, check_impl = _task(task)
    data = gen(**args)
    out = kernel(clone_data(data))
    torch.cuda.synchronize()
    good, msg = check_impl(data, out)
    if not good:
        return None, msg
    durations = []
    t_wall = time.perf_counter()
    for _ in range(max_repeats):
        torch.cuda.synchronize()
        flush()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        kernel(data)
        e.record()
        torch.cuda.synchronize()
        durations.append(s.elapsed_time(e) * 1e6)  # ns
        if len(durations) >= 3:
            st = calculate_stats(durations)
            total = st.mean * st.runs
            if (st.err / st.mean < 0.001 and total > 1e8) or total > max_time_ns or \
                    time.perf_counter() - t_wall > 120:
                break
    return calculate_stats(durations), ""


def run_benchmarks(task: str, cases, log: Logger) -> bool:
    flush = L2Flusher()
    ok_all = True
    if cases:
        benchmark_case(task, cases[0].args, flush, max_time_ns=1e8, max_repeats=10)  # warm-up
    log.log("benchmark-count", len(cases))
    for i, case in enumerate(cases):
        log.log(f"benchmark.{i}.spec", case.spec)
        try:
            stats, msg = benchmark_case(task, case.args, flush)
        except Exception as e:
            stats, msg = None, f"{type(e).__name__}: {e}"
        if stats is None:
            log.log(f"benchmark.{i}.status", "fail")
            log.log(f"benchmark.{i}.error", msg)
            ok_all = False
            continue
        for field in ("runs", "mean", "std", "err", "best", "worst"):
            log.log(f"benchmark.{i}.{field}", getattr(stats, field))
    log.log("check", "pass" if ok_all else "fail")
    return ok_all


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 3 or argv[0] not in ("test", "benchmark", "leaderboard") or argv[1] not in TASKS:
        print("usage: python -m eval_test_b200.runner test|benchmark|leaderboard <task> <spec file>\n"
              f"tasks: {', '.join(TASKS)}", file=sys.stderr)
        return 2
    mode, task, path = argv
    fd = os.getenv("POPCORN_FD")
    seed = os.getenv("POPCORN_SEED")
    try:
        cases = spec.parse_cases(Path(path).read_text(), int(seed) if seed else None)
    except (OSError, ValueError) as e:
        print(e, file=sys.stderr)
        return 113
    log = Logger(int(fd) if fd else None)
    ok = run_tests(task, cases, log) if mode == "test" else run_benchmarks(task, cases, log)
    return 0 if ok else 112


if __name__ == "__main__":
    sys.exit(main())
