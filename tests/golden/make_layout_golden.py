"""Generates ``layout_golden.npz``: the scale-factor layout as produced by the REFERENCE's own code.

Run where a checkout of the reference is at hand:

    python tests/golden/make_layout_golden.py <path of the reference checkout>

It imports ``to_blocked`` (eval/common/scale_helpers.py:10-17) and the padded variant of the grouped task
(eval/nvfp4_grouped_gemm/reference.py:14-36), feeds them seeded row-major scale matrices and stores inputs and
outputs.  It also stores a replay of the scatter of ``create_scale_factor_tensors``
(eval/common/scale_helpers.py:41-68) for one case: the 6-D index tuple each (row, k-block, batch) is written to.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root: str):
    ref = Path(ref_root)
    sh = _load(ref / "eval/common/scale_helpers.py", "ref_scale_helpers")
    out = {}
    g = torch.Generator().manual_seed(2024)
    for i, (rows, kbs) in enumerate([(128, 4), (256, 20), (384, 112), (128, 448)]):
        sf = torch.randint(0, 256, (rows, kbs), generator=g, dtype=torch.uint8)
        out[f"tb{i}_in"] = sf.numpy()
        out[f"tb{i}_out"] = sh.to_blocked(sf).numpy()
    # padded to_blocked of the grouped task: the file imports `task`/`utils` by bare name, so read only the function
    src = (ref / "eval/nvfp4_grouped_gemm/reference.py").read_text()
    start, end = src.index("def ceil_div"), src.index("def ref_kernel")
    ns = {"torch": torch}
    exec(compile(src[start:end], "grouped_reference_excerpt", "exec"), ns)
    for i, (rows, kbs) in enumerate([(40, 16), (200, 48), (72, 16)]):
        sf = torch.randint(0, 256, (rows, kbs), generator=g, dtype=torch.uint8)
        out[f"tbp{i}_in"] = sf.numpy()
        out[f"tbp{i}_out"] = ns["to_blocked"](sf).numpy()
    # the generator's scatter: destination index of every (i, j, b)
    mn, sf_k, l = 256, 24, 2
    i_grid, j_grid, b_grid = torch.meshgrid(torch.arange(mn), torch.arange(sf_k), torch.arange(l), indexing="ij")
    idx = torch.stack([i_grid % 32, (i_grid % 128) // 32, i_grid // 128, j_grid % 4, j_grid // 4, b_grid], dim=-1)
    out["scatter_index"] = idx.numpy().astype(np.int32)
    np.savez_compressed(Path(__file__).parent / "layout_golden.npz", **out)
    print("wrote layout_golden.npz:", sorted(out))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_layout_golden.py <path of the reference checkout>")
    main(sys.argv[1])
