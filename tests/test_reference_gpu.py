"""The reference's own acceptance test, run with the reference's own code: for every line of every task's
``tests.txt`` and ``benchmarks.txt`` the unmodified ``reference.py`` generates the inputs
(``generate_input(**args)``, CUDA generator), this library's ``custom_kernel`` runs on a clone, and the reference's
``check_implementation`` (``ref_kernel`` = ``torch._scaled_mm``, ``rtol = atol = 1e-3``) judges the output - the
steps of ``run_single_test`` (eval/common/eval_base.py:212-227).  The reference files come from ``oracle/_ref``
(staged by ``oracle/make_ref.py``); nothing of them is restated here.

Where the reference's generator makes the arithmetic exact (GEMM, GEMV, grouped GEMM: small dyadic values and
scales), the output must in addition equal ``ref_kernel``'s bit for bit.

The last tests hand the whole job to the reference's ``eval.py test tests.txt`` with a one-line ``submission.py``
that re-exports this library's entry point, and read the result from its POPCORN log.
"""
import os
import subprocess
import sys

import pytest

import _reference as R

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not R.staged(), reason="reference harness not staged: python oracle/make_ref.py <checkout>")]

CASES = [(task, name, i, line) for task in R.TASKS if R.staged()
         for i, (name, line) in enumerate(R.spec_lines(task))]
EXACT = {"nvfp4_gemm", "nvfp4_gemv", "nvfp4_grouped_gemm"}


def _kernel(task):
    import importlib
    return importlib.import_module(f"eval_test_b200.{task}").custom_kernel


def _bits_equal(x, y) -> bool:
    import torch
    if isinstance(x, (list, tuple)):
        return len(x) == len(y) and all(_bits_equal(a, b) for a, b in zip(x, y))
    return x.shape == y.shape and torch.equal(x.contiguous().view(torch.int16), y.contiguous().view(torch.int16))


@pytest.mark.parametrize("task,name,idx,line", CASES, ids=[f"{t}-{n.split('.')[0]}{i}" for t, n, i, _ in CASES])
def test_reference_generate_input_and_check_implementation(task, name, idx, line):
    import torch
    from eval_test_b200 import _lib
    ref, base = R.load_reference(task), R.load_eval_base()
    case = next(c for c in base.get_test_cases(str(R.REF_EVAL / task / name), None) if c.spec == line)
    data = ref.generate_input(**case.args)
    torch.cuda.synchronize()
    out = _kernel(task)(base.clone_data(data))
    torch.cuda.synchronize()
    status = _lib.device_status(torch.cuda.current_device())
    assert status == 0, _lib.strerror(status)
    good, message = ref.check_implementation(data, out)
    assert good, message
    if task in EXACT:
        expected = ref.ref_kernel(data)          # written into data's own output tensors, not into `out`
        assert _bits_equal(out, expected), "differs from torch._scaled_mm in at least one bit"


def _cutlass_importable() -> bool:
    try:
        import cutlass  # noqa: F401
        return True
    except Exception:
        return False


@pytest.mark.parametrize("task", R.TASKS)
def test_reference_eval_py_drives_the_library(task, tmp_path):
    """``python eval.py test tests.txt`` of the reference (spawned worker, POPCORN log on a pipe) with
    ``submission.py`` = one line importing this library's ``custom_kernel``."""
    if task in ("nvfp4_gemm", "nvfp4_grouped_gemm") and not _cutlass_importable():
        pytest.skip("this task's eval.py initialises CUDA through the cutlass package, which is not importable here")
    task_dir = R.REF_HARNESS / task
    r, w = os.pipe()
    env = dict(os.environ, POPCORN_FD=str(w), PYTHONPATH=str(R.ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    env.pop("POPCORN_SEED", None)
    try:
        proc = subprocess.run([sys.executable, "eval.py", "test", "tests.txt"], cwd=task_dir, env=env, pass_fds=(w,),
                              capture_output=True, text=True, timeout=900)
    finally:
        os.close(w)
    with os.fdopen(r) as f:
        log = dict(line.split(": ", 1) for line in f.read().splitlines() if ": " in line)
    assert proc.returncode == 0, (log, proc.stderr[-2000:])
    n = int(log["test-count"])
    assert n == 10 and log["check"] == "pass"
    assert all(log[f"test.{i}.status"] == "pass" for i in range(n)), log
