"""Stages the reference harness next to the oracle -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

    python oracle/make_ref.py <path of the reference checkout>

The reference is Python: its ``reference.py`` files (input generators, ``ref_kernel`` = ``torch._scaled_mm``,
``check_implementation``) need a GPU, so they can only run where the kernels run.  This recipe copies the
checkout's ``eval/`` tree, unmodified, into the git-ignored ``oracle/_ref/`` so that it travels with the working
tree to the machine that has the GPU; nothing of it is committed.  Two trees are written:

* ``oracle/_ref/eval/``     the reference's files as they are (its own ``submission.py`` kernels of the GEMM, dual
  GEMM and GEMV tasks included, which the runner can time as "the kernel to beat").  The grouped task's
  ``submission.py`` is left out: as shipped it does not compile (eval/nvfp4_grouped_gemm/submission.py:7,1189), so it
  can never be run, and its source names cluster-multicast TMA wrappers (never called), a form of load that is
  kept out of everything that travels to a machine with more than one GPU;
* ``oracle/_ref/harness/``  the same files with each task's ``submission.py`` replaced by the one-line re-export a
  maintainer would add to use this library, so that the reference's own ``eval.py test tests.txt`` drives the new
  kernels (eval/nvfp4_gemm/eval.py:23-40 imports ``submission`` from the task directory).

Only ``tests/`` and the runner's ``--submission`` option read these trees, and only when they exist.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

TASKS = {
    "nvfp4_gemm": "from eval_test_b200.nvfp4_gemm import custom_kernel, compile_kernel  # noqa: F401\n",
    "nvfp4_dual_gemm": "from eval_test_b200.nvfp4_dual_gemm import custom_kernel, compile_kernel  # noqa: F401\n",
    "nvfp4_grouped_gemm": "from eval_test_b200.nvfp4_grouped_gemm import custom_kernel, compile_kernel  # noqa: F401\n",
    "nvfp4_gemv": "from eval_test_b200.nvfp4_gemv import custom_kernel  # noqa: F401\n",
}


def stage(ref_root: str | Path) -> Path:
    src = Path(ref_root) / "eval"
    if not src.is_dir():
        raise FileNotFoundError(f"{src} is not the eval/ directory of a reference checkout")
    ignore = shutil.ignore_patterns("__pycache__", "*.pyc")
    for name in ("eval", "harness"):
        dst = OUT / name
        if dst.exists():
            shutil.rmtree(dst)
        shutil.copytree(src, dst, ignore=ignore)
    for task, line in TASKS.items():
        (OUT / "harness" / task / "submission.py").write_text(line)
    (OUT / "eval" / "nvfp4_grouped_gemm" / "submission.py").unlink()
    return OUT


if __name__ == "__main__":
    if len(sys.argv) != 2:
        print(__doc__, file=sys.stderr)
        sys.exit(2)
    print(stage(sys.argv[1]))
