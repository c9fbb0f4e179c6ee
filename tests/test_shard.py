"""Sharding logic on CPU: two gloo ranks each compute their shard (with the CPU oracle standing in for the GPU
kernel), the optional all-gather reassembles the result, and it must equal the unsharded result bit for bit
(no K split, so the accumulation order inside every output element is unchanged)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from _util import dual_oracle_args, gemm_oracle_args, grouped_oracle_args, operand_np, out_np, scales_np
    from eval_test_b200 import formats as F, inputs, shard
    from oracle import nvfp4_oracle as O
    O.set_num_threads(2)

    def to_c(arr):  # [L, M, N] float16 -> the [M, N, L] output layout
        return F.batch_last(torch.from_numpy(arr))

    # GEMM: column shards
    full = inputs.gemm_quantized(128, 512, 512, 2, seed=3, device="cpu")
    loc = shard.shard_gemm(full, rank, world)
    assert loc[1].shape == (512 // world, 256, 2) and loc[5].shape[2] == 512 // world // 128
    c = shard.gather_cols(to_c(O.c_gemm(*gemm_oracle_args(loc))), world)
    want = O.c_gemm(*gemm_oracle_args(full))
    assert np.array_equal(out_np(c).view(np.uint16), want.view(np.uint16))

    # dual GEMM
    full = inputs.dual_gemm_quantized(128, 256, 256, 1, seed=4, device="cpu")
    loc = shard.shard_dual_gemm(full, rank, world)
    c = shard.gather_cols(to_c(O.c_dual_gemm(*dual_oracle_args(loc))), world)
    assert np.array_equal(out_np(c).view(np.uint16), O.c_dual_gemm(*dual_oracle_args(full)).view(np.uint16))

    # GEMV: row shards
    full = inputs.gemv_quantized(512, 512, 2, seed=5, device="cpu")
    loc = shard.shard_gemv(full, rank, world)
    a, b, _, _, sa, sb, _ = loc
    got = O.c_gemv(operand_np(a), operand_np(b), scales_np(sa), scales_np(sb))       # [L, M/g]
    c = shard.gather_rows(to_c(got[:, :, None]), world)
    a, b, _, _, sa, sb, _ = full
    want = O.c_gemv(operand_np(a), operand_np(b), scales_np(sa), scales_np(sb))
    assert np.array_equal(out_np(c)[:, :, 0].view(np.uint16), want.view(np.uint16))

    # grouped GEMM: whole groups per rank; every group is computed exactly once across the ranks
    ms = [100, 0, 300, 40, 128, 0, 77]
    full = inputs.grouped_gemm_quantized(ms, [128] * 7, [256] * 7, 7, seed=6, device="cpu")
    loc, mine = shard.shard_grouped_gemm(full, rank, world)
    got = O.c_grouped_gemm(grouped_oracle_args(loc))
    want = O.c_grouped_gemm(grouped_oracle_args(full))
    for g, i in zip(got, mine):
        assert np.array_equal(g.view(np.uint16), want[i].view(np.uint16))
    owners = [None] * world
    dist.all_gather_object(owners, mine)
    assert sorted(i for o in owners for i in o) == list(range(7))

    dist.barrier()
    dist.destroy_process_group()
    (Path(out_dir) / f"ok{rank}").write_text("ok")


def test_two_rank_sharding_matches_unsharded(tmp_path):
    world, port = 2, 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_assign_groups_balances_weights():
    from eval_test_b200 import shard
    ms = [128, 0, 140, 99, 0, 157, 120, 131, 0, 125]
    for world in (1, 2, 4, 8):
        parts = shard.assign_groups(ms, world)
        assert sorted(i for p in parts for i in p) == list(range(len(ms)))
        live = [sum(ms[i] > 0 for i in p) for p in parts]
        assert max(live) - min(live) <= 1


def test_shard_rejects_uneven_split():
    from eval_test_b200 import inputs, shard
    data = inputs.gemm_reference_style(128, 384, 256, 1, seed=0, device="cpu")
    with pytest.raises(ValueError, match="multiple of 128"):
        shard.shard_gemm(data, 0, 2)
