"""B200-native NVFP4 kernels behind the entry points of the jIab-b/eval_test harness.

Each ``nvfp4_*`` module exposes ``custom_kernel(data)`` with the reference's input tuple; the work is done
by hand-written sm_100a CUDA kernels in ``csrc/`` reached through the C ABI of ``libnvfp4_b200.so``.
There is no CPU or library fallback: importing an op without the built library raises.
"""
from . import formats, inputs, check, spec  # noqa: F401

__all__ = ["formats", "inputs", "check", "spec"]
