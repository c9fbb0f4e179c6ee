"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "nvfp4_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nvfp4_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_four_entry_points():
    syms = _declared_symbols()
    for name in ("nvfp4_gemv", "nvfp4_gemm", "nvfp4_dual_gemm", "nvfp4_grouped_gemm", "nvfp4_strerror"):
        assert name in syms


def test_library_exports_every_declared_symbol(lib):
    for name in _declared_symbols():
        assert hasattr(lib, name), name


def test_strerror_and_version_need_no_gpu(lib):
    from eval_test_b200 import _lib
    assert lib.nvfp4_abi_version() == 1
    assert _lib.strerror(0) == "ok"
    assert "K" in _lib.strerror(-3) and "aligned" in _lib.strerror(-5)
    assert "expired" in _lib.strerror(101)


def test_group_struct_layout_matches_header():
    from eval_test_b200 import _lib
    assert ctypes.sizeof(_lib.Group) == 5 * 8 + 4 * 4
    assert _lib.Group.M.offset == 40 and _lib.Group.K.offset == 48


def test_argument_validation_needs_no_gpu(lib):
    """Rejected before any CUDA call is made."""
    assert lib.nvfp4_gemv(None, None, None, None, None, 128, 256, 1, 128, 1.0, None) == -1
    assert lib.nvfp4_gemv(16, 16, 16, 16, 16, 128, 100, 1, 128, 1.0, None) == -3
    assert lib.nvfp4_gemv(16, 16, 16, 16, 16, -1, 256, 1, 128, 1.0, None) == -2
    assert lib.nvfp4_gemv(8, 16, 16, 16, 16, 128, 256, 1, 128, 1.0, None) == -5


def test_shims_reject_wrong_layouts():
    import pytest
    import torch
    from eval_test_b200 import _args
    t = torch.zeros((128, 64, 1), dtype=torch.uint8)
    with pytest.raises(ValueError, match="CUDA"):
        _args.operand_ptr(t, 128, 64, 1, "a")
    with pytest.raises(ValueError, match="shape"):
        _args.operand_ptr(t, 256, 64, 1, "a")


def test_another_build_can_be_loaded_by_environment_variable(tmp_path):
    """NVFP4_B200_LIB names the library file that load() opens (an instrumented build, say); build() keeps writing
    the one next to the package."""
    import os
    import shutil
    import subprocess
    import sys
    from eval_test_b200 import _lib
    other = tmp_path / "libother.so"
    shutil.copy(_lib.BUILT_SO, other)
    code = ("from eval_test_b200 import _lib; lib = _lib.load(); "
            "print(_lib.SO_PATH, _lib.BUILT_SO, lib.nvfp4_abi_version())")
    out = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, NVFP4_B200_LIB=str(other)),
                         cwd=str(Path(__file__).resolve().parent.parent), capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    loaded, built, version = out.stdout.split()
    assert loaded == str(other.resolve()) and built == str(_lib.BUILT_SO) and int(version) >= 1
