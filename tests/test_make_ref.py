"""The recipe that stages the reference harness for the GPU tests, on a miniature stand-in checkout."""
import importlib.util
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _make_ref():
    spec = importlib.util.spec_from_file_location("make_ref_under_test", ROOT / "oracle" / "make_ref.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_stage_copies_the_tree_and_swaps_the_submissions(tmp_path, monkeypatch):
    mod = _make_ref()
    src = tmp_path / "checkout" / "eval"
    for task in mod.TASKS:
        (src / task).mkdir(parents=True)
        (src / task / "reference.py").write_text(f"# reference of {task}\n")
        (src / task / "submission.py").write_text("# the reference's own kernel\n")
        (src / task / "tests.txt").write_text("m: 128; seed: 1\n")
    (src / "common").mkdir()
    (src / "common" / "utils.py").write_text("# common\n")
    monkeypatch.setattr(mod, "OUT", tmp_path / "out")
    out = mod.stage(tmp_path / "checkout")
    for task, line in mod.TASKS.items():
        assert (out / "eval" / task / "reference.py").read_text() == f"# reference of {task}\n"
        assert (out / "harness" / task / "reference.py").read_text() == f"# reference of {task}\n"
        assert (out / "harness" / task / "submission.py").read_text() == line
        assert f"eval_test_b200.{task}" in line and "custom_kernel" in line
    assert (out / "eval" / "nvfp4_gemm" / "submission.py").read_text() == "# the reference's own kernel\n"
    assert not (out / "eval" / "nvfp4_grouped_gemm" / "submission.py").exists()
    assert (out / "harness" / "common" / "utils.py").exists()
    mod.stage(tmp_path / "checkout")            # staging again replaces the trees


def test_stage_rejects_something_that_is_not_a_checkout(tmp_path):
    import pytest
    with pytest.raises(FileNotFoundError):
        _make_ref().stage(tmp_path)
