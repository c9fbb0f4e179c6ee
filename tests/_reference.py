"""Access to the staged reference harness (``oracle/_ref``, written by ``oracle/make_ref.py``) for the tests.

The reference's task directories all hold modules with the same bare names (``reference``, ``task``, ``utils``,
``submission``) and expect their own directory and ``eval/`` on ``sys.path``.  ``load_reference(task)`` imports one
task's ``reference.py`` the way the reference's ``eval.py`` would find it and then removes those bare names from
``sys.modules`` again, so that the next task gets its own.
"""
from __future__ import annotations

import functools
import importlib
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF_EVAL = ROOT / "oracle" / "_ref" / "eval"
REF_HARNESS = ROOT / "oracle" / "_ref" / "harness"
TASKS = ("nvfp4_gemm", "nvfp4_gemv", "nvfp4_dual_gemm", "nvfp4_grouped_gemm")
_BARE = ("reference", "task", "utils", "submission")


def staged() -> bool:
    return all((REF_EVAL / t / "reference.py").exists() for t in TASKS)


@functools.lru_cache(maxsize=None)
def load_reference(task: str):
    """The unmodified ``eval/<task>/reference.py`` as a module object."""
    task_dir, eval_dir = str(REF_EVAL / task), str(REF_EVAL)
    saved = {name: sys.modules.pop(name, None) for name in _BARE}
    sys.path[:0] = [task_dir, eval_dir]
    try:
        mod = importlib.import_module("reference")
    finally:
        for p in (task_dir, eval_dir):
            while p in sys.path:
                sys.path.remove(p)
        for name in _BARE:
            sys.modules.pop(name, None)
            if saved[name] is not None:
                sys.modules[name] = saved[name]
    return mod


@functools.lru_cache(maxsize=None)
def load_eval_base():
    """``eval/common/eval_base.py`` (spec parser, ``clone_data``) of the staged tree."""
    eval_dir = str(REF_EVAL)
    sys.path.insert(0, eval_dir)
    try:
        return importlib.import_module("common.eval_base")
    finally:
        sys.path.remove(eval_dir)


def spec_lines(task: str) -> list[tuple[str, str]]:
    """(file name, line) of every case in the task's ``tests.txt`` and ``benchmarks.txt``."""
    out = []
    for name in ("tests.txt", "benchmarks.txt"):
        path = REF_EVAL / task / name
        if path.exists():
            out += [(name, line) for line in path.read_text().splitlines() if line.strip()]
    return out
