"""Local runner for the harness's shape-list files, in place of the remote launcher.

    python -m eval_test_b200.runner test        nvfp4_gemm  tests.txt
    python -m eval_test_b200.runner benchmark   nvfp4_gemv  benchmarks.txt [--report] [--kernel-time]
    python -m eval_test_b200.runner leaderboard nvfp4_dual_gemm benchmarks.txt
    python -m eval_test_b200.runner profile     nvfp4_gemm  benchmarks.txt
    python -m eval_test_b200.runner benchmark   nvfp4_gemm  benchmarks.txt --eval-dir <eval/> --submission <eval/nvfp4_gemm/submission.py>

It follows the reference's evaluation protocol (eval/common/eval_base.py):

* the same spec grammar and seed mixing (``POPCORN_SEED``), ``key: value`` log lines on the file descriptor named by
  ``POPCORN_FD`` (stdout when unset), ``test.N.status: pass|fail`` with the checker's message on failure, exit codes
  0 / 112 (a test or benchmark failed) / 113 (malformed spec) / 2 (usage) (eval_base.py:67,416,525-549);
* ``benchmark``: a correctness check, then CUDA events around ``custom_kernel(data)`` on the current stream with a
  cold L2 before every sample, until the error of the mean is below 0.1 %, the time budget is used up or 120 s of
  wall time have passed (eval_base.py:229-295).  GEMV, dual GEMM and grouped GEMM are sampled in the reference's
  *batched* mode - 50 (GEMV, dual) or 15 (grouped) distinct inputs, seeds 42 apart, inside one event pair, per-call
  mean reported (eval_base.py:297-369; eval/nvfp4_gemv/eval.py:11-12, eval/nvfp4_dual_gemm/eval.py:11-12,
  eval_base.py:141-142) - the GEMM one call at a time (eval/nvfp4_gemm/eval.py:13);
* ``leaderboard``: every shape is warmed up first, then sampled with the output re-checked on every repeat; in
  single mode each repeat draws fresh inputs (``seed += 13``) so that a cached result cannot pass
  (eval_base.py:263-266,283-286,471-504);
* ``profile``: one call under ``torch.profiler``, the table base64-encoded into the log (eval_base.py:371-387,507-518).

``--eval-dir`` takes ``generate_input`` / ``check_implementation`` from the reference's own
``<eval-dir>/<task>/reference.py`` instead of this package's generators; ``--submission`` times any ``submission.py``
(for instance the reference's own kernels) with the same loop.  ``--report`` prints a markdown summary of the log.

Differences from the reference: everything runs in this process (the reference isolates each case in a spawned
worker); the L2 is flushed by writing a 512 MiB buffer, not by drawing 62.5 GiB of random numbers
(eval/common/utils.py:158-160).
"""
from __future__ import annotations

import argparse
import base64
import copy
import importlib
import importlib.util
import math
import os
import sys
import time
from dataclasses import dataclass, fields
from pathlib import Path

from . import spec

TASKS = ("nvfp4_gemv", "nvfp4_gemm", "nvfp4_dual_gemm", "nvfp4_grouped_gemm")
# (batched sampling?, inputs per batch) as the reference's per-task runners set them
SAMPLING = {"nvfp4_gemm": (False, 1), "nvfp4_gemv": (True, 50), "nvfp4_dual_gemm": (True, 50),
            "nvfp4_grouped_gemm": (True, 15)}


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
    """``key: value`` lines on the POPCORN file descriptor (eval_base.py:18-33); keeps a copy for ``--report``."""

    def __init__(self, fd: int | None):
        self.file = os.fdopen(fd, "w") if fd is not None else sys.stdout
        self.lines: list[str] = []

    def log(self, key, value):
        line = f"{key}: {value}"
        self.lines.append(line)
        print(line, file=self.file, flush=True)


@dataclass
class Task:
    name: str
    kernel: object
    compile_kernel: object
    generate_input: object
    check: object
    batched: bool
    batch_size: int


def _import_file(path: Path, name: str, extra_paths=()):
    """Import ``path`` the way the harness finds it: its own directory and ``extra_paths`` on ``sys.path`` while the
    module body runs, bare sibling names (``task``, ``utils``, ``reference``) not left behind in ``sys.modules``."""
    bare = ("task", "utils", "reference", "submission")
    saved = {b: sys.modules.pop(b, None) for b in bare}
    added = [str(path.parent), *map(str, extra_paths)]
    sys.path[:0] = added
    try:
        sp = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(sp)
        sp.loader.exec_module(mod)
    finally:
        for a in added:
            while a in sys.path:
                sys.path.remove(a)
        for b in bare:
            sys.modules.pop(b, None)
            if saved[b] is not None:
                sys.modules[b] = saved[b]
    return mod


def load_task(task: str, eval_dir: str | None = None, submission: str | None = None) -> Task:
    """The kernel, generator and checker of a task.  Defaults: this package's shim, its seeded reference-style
    generator and the ``torch._scaled_mm`` check of ``reference_check``."""
    from . import inputs, reference_check
    gens = {"nvfp4_gemv": inputs.gemv_reference_style, "nvfp4_gemm": inputs.gemm_reference_style,
            "nvfp4_dual_gemm": inputs.dual_gemm_reference_style, "nvfp4_grouped_gemm": inputs.grouped_gemm_reference_style}
    gen, chk = gens[task], reference_check.check_implementation(task)
    if eval_dir is not None:
        ref = _import_file(Path(eval_dir) / task / "reference.py", f"_harness_{task}_reference", [eval_dir])
        gen, chk = ref.generate_input, ref.check_implementation
    if submission is not None:
        sub_path = Path(submission).resolve()
        sub = _import_file(sub_path, f"_harness_{task}_submission", [sub_path.parent.parent])
        kernel, comp = sub.custom_kernel, getattr(sub, "compile_kernel", None)
    else:
        mod = importlib.import_module(f"{__package__}.{task}")
        kernel, comp = mod.custom_kernel, getattr(mod, "compile_kernel", None)
    batched, bs = SAMPLING[task]
    return Task(task, kernel, comp, gen, chk, batched, bs)


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


def _call_compile(t: Task):
    """``compile_kernel()`` when the submission has one that can be called without arguments
    (eval_base.py:182-199: ``use_loop=True`` is passed when the parameter exists)."""
    if t.compile_kernel is None:
        return
    import inspect
    params = inspect.signature(t.compile_kernel).parameters
    kwargs = {}
    for name, prm in params.items():
        if name == "use_loop":
            kwargs["use_loop"] = True
        elif prm.default is inspect.Parameter.empty:
            return
    t.compile_kernel(**kwargs)


def run_tests(t: Task, cases, log: Logger) -> bool:
    import torch
    ok_all = True
    log.log("test-count", len(cases))
    for i, case in enumerate(cases):
        log.log(f"test.{i}.spec", case.spec)
        try:
            data = t.generate_input(**case.args)
            torch.cuda.synchronize()
            out = t.kernel(clone_data(data))
            torch.cuda.synchronize()
            good, msg = t.check(data, out)
        except Exception as e:  # a kernel error fails the test, as in the reference (eval_base.py:224-225)
            good, msg = False, f"{type(e).__name__}: {e}"
        log.log(f"test.{i}.status", "pass" if good else "fail")
        if not good:
            log.log(f"test.{i}.error", msg)
            ok_all = False
    log.log("check", "pass" if ok_all else "fail")
    return ok_all


def _enough(durations, i, t_start_ns, max_time_ns) -> bool:
    """The reference's stop rule (eval_base.py:288-293): at least three samples and 100 ms of wall time, then stop
    when the error of the mean is below 0.1 %, the sampled time exceeds the budget or 120 s have passed."""
    wall = time.perf_counter_ns() - t_start_ns
    if i > 1 and wall > 1e8:
        st = calculate_stats(durations)
        return st.err / st.mean < 0.001 or st.mean * st.runs > max_time_ns or wall > 120e9
    return False


def benchmark_single(t: Task, args: dict, flush, recheck: bool, max_repeats: int, max_time_ns: float):
    """One call per sample (eval_base.py:229-295).  Returns (Stats | None, error message | None)."""
    import torch
    args = dict(args)
    data = t.generate_input(**args)
    check_copy = clone_data(data)
    try:
        _call_compile(t)
        torch.cuda.synchronize()
        out = t.kernel(clone_data(data))
    except Exception as e:
        return None, f"Encountered {type(e).__name__}: {e}"
    torch.cuda.synchronize()
    good, msg = t.check(check_copy, out)
    error = None if good else msg
    durations = []
    t0 = time.perf_counter_ns()
    for i in range(max_repeats):
        if recheck and "seed" in args:
            args["seed"] += 13
            data = t.generate_input(**args)
            check_copy = clone_data(data)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flush()
        s.record()
        out = t.kernel(data)
        e.record()
        torch.cuda.synchronize()
        durations.append(s.elapsed_time(e) * 1e6)  # ns
        if recheck:
            good, msg = t.check(check_copy, out)
            if not good and error is None:
                error = msg
        del out
        if _enough(durations, i, t0, max_time_ns):
            break
    return calculate_stats(durations), error


def benchmark_batched(t: Task, args: dict, flush, recheck: bool, max_repeats: int, max_time_ns: float):
    """``batch_size`` distinct inputs inside one event pair, per-call mean per sample (eval_base.py:297-369)."""
    import torch
    args = dict(args)
    batch = []
    for _ in range(t.batch_size):
        if "seed" in args:
            args["seed"] += 42
        batch.append(t.generate_input(**args))
    check_copy = clone_data(batch)
    try:
        outs = [t.kernel(clone_data(d)) for d in batch]
    except Exception as e:
        return None, f"Encountered {type(e).__name__}: {e}"
    torch.cuda.synchronize()
    error = None
    for ref_in, out in zip(check_copy, outs):
        good, msg = t.check(ref_in, out)
        if not good:
            error = msg
            break
    durations = []
    t0 = time.perf_counter_ns()
    for i in range(max_repeats):
        torch.cuda.synchronize()
        flush()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        outs = [t.kernel(d) for d in batch]
        e.record()
        torch.cuda.synchronize()
        durations.append(s.elapsed_time(e) / t.batch_size * 1e6)
        if recheck:
            for ref_in, out in zip(check_copy, outs):
                good, msg = t.check(ref_in, out)
                if not good and error is None:
                    error = msg
                    break
        if _enough(durations, i, t0, max_time_ns):
            break
    return calculate_stats(durations), error


def _benchmark(t: Task, args, flush, recheck, max_repeats, max_time_ns):
    fn = benchmark_batched if t.batched else benchmark_single
    try:
        return fn(t, args, flush, recheck, max_repeats, max_time_ns)
    except Exception as e:
        return None, f"{type(e).__name__}: {e}"


def kernel_only_us(t: Task, args: dict, flush) -> float | None:
    """Device time of the kernels of ONE call, cold L2, from the profiler's kernel records (no launch latency, no
    host time): what remains of a sample once everything but the GPU work is taken away."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    data = t.generate_input(**args)
    for _ in range(3):
        t.kernel(data)
    torch.cuda.synchronize()
    best = None
    for _ in range(5):
        flush()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            t.kernel(data)
            torch.cuda.synchronize()
        us = sum(e.device_time_total for e in prof.key_averages() if "memset" not in e.key.lower())
        if us > 0:
            best = us if best is None else min(best, us)
    return best


def run_benchmarks(t: Task, cases, log: Logger, leaderboard: bool = False, kernel_time: bool = False) -> bool:
    flush = L2Flusher()
    ok_all = True
    if leaderboard:      # warm every shape up, then sample with the output re-checked on every repeat
        for case in cases:
            _benchmark(t, case.args, flush, False, 50, 5e8)
    elif cases:
        _benchmark(t, cases[0].args, flush, False, 100, 1e8)
    log.log("benchmark-count", len(cases))
    for i, case in enumerate(cases):
        log.log(f"benchmark.{i}.spec", case.spec)
        stats, error = _benchmark(t, case.args, flush, leaderboard, 100, 30e9 if leaderboard else 10e9)
        if stats is not None:
            for f in fields(Stats):
                log.log(f"benchmark.{i}.{f.name}", getattr(stats, f.name))
        if kernel_time:
            try:
                us = kernel_only_us(t, case.args, flush)
                if us is not None:
                    log.log(f"benchmark.{i}.kernel_us", us)
            except Exception as e:
                log.log(f"benchmark.{i}.kernel_us_error", f"{type(e).__name__}: {e}")
        if error is not None or stats is None:
            ok_all = False
            log.log(f"benchmark.{i}.status", "fail")
            if error is not None:
                log.log(f"benchmark.{i}.error", error)
    log.log("check", "pass" if ok_all else "fail")
    return ok_all


def run_profile(t: Task, cases, log: Logger) -> bool:
    import torch
    from torch.profiler import ProfilerActivity, profile
    log.log("benchmark-count", len(cases))
    for i, case in enumerate(cases):
        log.log(f"benchmark.{i}.spec", case.spec)
        data = t.generate_input(**case.args)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            t.kernel(clone_data(data))
            torch.cuda.synchronize()
        table = prof.key_averages().table(sort_by="self_cuda_time_total", row_limit=20)
        log.log(f"benchmark.{i}.report", base64.b64encode(table.encode("utf-8"), b"+*").decode("utf-8"))
    log.log("check", "pass")
    return True


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    ap = argparse.ArgumentParser(prog="python -m eval_test_b200.runner", add_help=True)
    ap.add_argument("mode", choices=["test", "benchmark", "leaderboard", "profile"])
    ap.add_argument("task", choices=TASKS)
    ap.add_argument("spec_file")
    ap.add_argument("--eval-dir", help="take generate_input / check_implementation from <eval-dir>/<task>/reference.py")
    ap.add_argument("--submission", help="time the custom_kernel of this submission.py instead of the library's")
    ap.add_argument("--report", action="store_true", help="print a markdown summary of the log at the end")
    ap.add_argument("--kernel-time", action="store_true",
                    help="benchmark modes: also log the kernels' own device time of one call (profiler records)")
    try:
        a = ap.parse_args(argv)
    except SystemExit:
        return 2
    fd = os.getenv("POPCORN_FD")
    seed = os.getenv("POPCORN_SEED")
    try:
        cases = spec.parse_cases(Path(a.spec_file).read_text(), int(seed) if seed else None)
    except (OSError, ValueError) as e:
        print(e, file=sys.stderr)
        return 113
    log = Logger(int(fd) if fd else None)
    t = load_task(a.task, a.eval_dir, a.submission)
    if a.mode == "test":
        ok = run_tests(t, cases, log)
    elif a.mode == "profile":
        ok = run_profile(t, cases, log)
    else:
        ok = run_benchmarks(t, cases, log, leaderboard=a.mode == "leaderboard", kernel_time=a.kernel_time)
    if a.report:
        from . import report
        print(report.format_report(report.parse_log("\n".join(log.lines)), a.mode, a.task, report.system_info()))
    return 0 if ok else 112


if __name__ == "__main__":
    sys.exit(main())
