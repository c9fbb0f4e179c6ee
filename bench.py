#!/usr/bin/env python
"""Benchmark of the NVFP4 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic input.  With no ``--workload`` the run prints ONE
JSON line whose headline (``metric`` / ``value`` / ``roofline`` / ``e2e`` / ``cpu_baseline`` / ``clocks``) is the
batched GEMV the metric is quoted on (M = K = 16384, L = 4, N(0,1) data through the block-16 quantiser, HBM-bound,
GB/s of algorithmic bytes) and whose ``workloads`` object holds the same record for the other configurations: the
8192^3 GEMM, the SwiGLU dual GEMM, the 64-group grouped GEMM with and without forced empty groups, and (N > 1) the
GEMV split M/N ways.  ``--workload NAME`` measures one of them alone.

N > 1 (torchrun, one process per GPU, no data-path collective): the headline GEMV is weak scaling (every rank owns
16384 more rows); the sub-records are strong scaling - GEMM and dual GEMM split the columns of C (rows of B),
the grouped GEMM deals whole groups to ranks balanced by weight bytes, the GEMV splits rows.  Every number is device
time (CUDA events on the launching stream), maximum over ranks.

Each record carries ``roofline`` (dominant kernel against the measured peak: copy bandwidth for the HBM-bound
workloads, 4 x the bf16 GEMM burst rate for the tensor-bound ones, with the fraction of the nominal 8 TB/s /
9 PFLOP/s beside it), ``e2e`` (the same metric through ``custom_kernel`` with pinned host inputs copied in and the
output copied out inside the timed region), ``cpu_baseline`` (N = 1, rank 0: the CPU oracle on the host cores, two
routes, see ``cpu_baseline()``) and ``clocks`` (NVML samples while the workload's launches run).

``--impl reference`` times the CPU restatement of the reference's arithmetic (the reference's own oracle is a GPU
library call and it has no CPU path) with all host threads on the same configurations.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HBM_FALLBACK_GBS = 6650.0
L2_BYTES = 126 * 1024 * 1024


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return HBM_FALLBACK_GBS, "fallback"


# ----------------------------------------------------------------------------------------------- workloads
def _util():
    from eval_test_b200 import hostviews
    return hostviews


class GemvWorkload:
    """Batched GEMV: A 16384 x 16384 e2m1 with block-16 e4m3 scales times a quantised vector, batch 4.
    N > 1: every rank owns 16384 more rows of A (weak scaling, nothing exchanged)."""
    name = "gemv_m16384_k16384_l4"
    metric = "nvfp4_gemv_hbm_gbs"
    unit, per = "GB/s", 1e9
    dtype = "e2m1 x ue4m3 scales, block-scaled tensor-core products, fp32 accumulate, fp16 out"
    bound, kernel, scaling = "hbm", "gemv_tc_kernel", "weak"

    def __init__(self, m=16384, k=16384, l=4, strong=False):
        self.m, self.k, self.l, self.strong = m, k, l, strong
        if strong:   # the same 16384 rows split M/N ways instead of 16384 rows per rank
            self.name, self.scaling = f"gemv_m{m}_k{k}_l{l}_rowsplit", "strong"

    def small(self):
        return GemvWorkload(m=4096, k=self.k, l=self.l, strong=self.strong)

    def _rows(self, world):
        return self.m // world if self.strong else self.m

    def work(self, world=1, m=None) -> int:
        """Algorithmic bytes per rank and step: A + its scales + the vector and its scales + the fp16 output."""
        m = self._rows(world) if m is None else m
        return self.l * (m * self.k // 2 + m * self.k // 16 + (self.k // 2 + self.k // 16) + 2 * m)

    def job(self, world=1) -> int:
        return self.work(world) * world

    def make(self, rank, world, device):
        from eval_test_b200 import inputs
        return inputs.gemv_quantized(self._rows(world), self.k, self.l, seed=rank, device=device)

    def run(self, data):
        from eval_test_b200 import nvfp4_gemv
        return nvfp4_gemv.custom_kernel(data)

    def io(self, data):
        a, b, _, _, sfa_p, sfb_p, c = data
        return [a, b, sfa_p, sfb_p], [c]

    def with_inputs(self, data, moved):
        a, b, sfa, sfb, sfa_p, sfb_p, c = data
        return (moved[0], moved[1], sfa, sfb, moved[2], moved[3], c)

    def config(self, world):
        rows = self._rows(world)
        mb = self.work(world) / 1e6
        return {"workload": self.name, "m_per_gpu": rows, "k": self.k, "l": self.l, "global_m": rows * world,
                "sharding": "rows of A per rank, no collective",
                "l2": (f"inputs ({mb:.0f} MB per step) larger than L2 (126 MB)" if mb > 132 else
                       f"inputs ({mb:.0f} MB per step) fit in L2 at this split: 512 MiB written between steps"),
                "generator": "N(0,1) seed = rank -> block-16 quantiser (scale = amax/6 as e4m3, RNE e2m1)"}

    def flush_l2(self, world):
        return self.work(world) < 132e6

    def cpu_samples(self, data):
        """(route, callable, units, description) per CPU route; see cpu_baseline()."""
        from oracle import nvfp4_oracle as O
        u = _util()
        a, b, _, _, sfa_p, sfb_p, _ = data
        out = []
        for route, rows, fn in (("fused_c", 8192, O.c_gemv), ("dequant_matmul", 2048, O.dq_gemv)):
            rows = min(rows, a.shape[0]) // 128 * 128
            args = (u.operand_np(a[:rows]), u.operand_np(b), u.scales_np(sfa_p[:, :, : rows // 128]), u.scales_np(sfb_p))
            out.append((route, (lambda fn=fn, args=args: fn(*args)), self.work(m=rows),
                        f"rows 0..{rows - 1} of each of the {self.l} batches, K = {self.k}"))
        return out


class GemmWorkload:
    """Large GEMM: M = N = K = 8192, alpha = 0.5.  N > 1: B, its scales and C are split along N (strong scaling,
    no K split, so nothing is reduced or exchanged)."""
    name = "gemm_m8192_n8192_k8192"
    metric = "nvfp4_gemm_tflops"
    unit, per = "TFLOPS", 1e12
    dtype = "e2m1 x ue4m3 scales on tcgen05 (kind::mxf4nvf4), fp32 accumulate, fp16 out"
    bound, kernel, scaling = "tensor", "gemm_pair_kernel", "strong"
    alpha = 0.5

    def __init__(self, m=8192, n=8192, k=8192):
        self.m, self.n, self.k = m, n, k

    def small(self):
        return GemmWorkload(m=4096, n=8192, k=4096)

    def work(self, world=1, m=None, n=None) -> int:
        return 2 * (self.m if m is None else m) * (self.n // world if n is None else n) * self.k

    def job(self, world=1) -> int:
        return self.work(1)

    def make(self, rank, world, device):
        from eval_test_b200 import inputs
        import torch
        a, _, sfa, _, sfa_p, _, _ = inputs.gemm_quantized(self.m, 128, self.k, 1, seed=0, device=device)
        g = torch.Generator(device=device).manual_seed(1000 + rank)
        b, sfb, sfb_p = inputs.quantized_operand(1, self.n // world, self.k, g, device)
        c = torch.empty((1, self.m, self.n // world), dtype=torch.float16, device=device).permute(1, 2, 0)
        return (a, b, sfa, sfb, sfa_p, sfb_p, c)

    def run(self, data):
        from eval_test_b200 import nvfp4_gemm
        return nvfp4_gemm.custom_kernel(data, alpha=self.alpha)

    def io(self, data):
        a, b, _, _, sfa_p, sfb_p, c = data
        return [a, b, sfa_p, sfb_p], [c]

    def with_inputs(self, data, moved):
        a, b, sfa, sfb, sfa_p, sfb_p, c = data
        return (moved[0], moved[1], sfa, sfb, moved[2], moved[3], c)

    def config(self, world):
        return {"workload": self.name, "m": self.m, "n": self.n, "k": self.k, "l": 1, "alpha": self.alpha,
                "n_per_gpu": self.n // world, "sharding": "columns of C (rows of B) per rank, A replicated, no collective",
                "l2": "operands + output (210 MB at 1 GPU) larger than L2 (126 MB)",
                "generator": "N(0,1) seeded -> block-16 quantiser"}

    def flush_l2(self, world):
        return False

    def cpu_samples(self, data):
        from oracle import nvfp4_oracle as O
        u = _util()
        a, b, _, _, sfa_p, sfb_p, _ = data
        out = []
        for route, rows, cols, fn in (("fused_c", 128, 1024, O.c_gemm), ("dequant_matmul", a.shape[0], b.shape[0], O.dq_gemm)):
            rows, cols = min(rows, a.shape[0]), min(cols, b.shape[0])
            args = (u.operand_np(a[:rows]), u.operand_np(b[:cols]), u.scales_np(sfa_p[:, :, : (rows + 127) // 128]),
                    u.scales_np(sfb_p[:, :, : cols // 128]), self.alpha)
            what = ("the whole problem" if (rows, cols) == (a.shape[0], b.shape[0]) else
                    f"rows 0..{rows - 1} of A against rows 0..{cols - 1} of B, K = {self.k}")
            out.append((route, (lambda fn=fn, args=args: fn(*args)), self.work(m=rows, n=cols), what))
        return out


class GemmGatherWorkload(GemmWorkload):
    """The same N-sharded GEMM with the full C assembled on every rank inside the timed step: either the kernel's
    fused all-gather epilogue (stores into every rank's copy over NVLink, then a barrier) or the kernel followed by
    an NCCL all-gather of the column shards.  The roofline target is the slower of the rank's flops at the tensor
    peak and the bytes the rank must send at 770 GB/s (measured peer-copy bandwidth per direction)."""
    metric = "nvfp4_gemm_allgather_tflops"
    kernel = "gemm_kernel"
    nvlink_gbs = 770.0

    def __init__(self, fused=True, m=8192, n=8192, k=8192):
        super().__init__(m, n, k)
        self.fused = fused
        self.name = f"gemm_m{m}_n{n}_k{k}_allgather_{'fused' if fused else 'nccl'}"

    def small(self):
        return GemmGatherWorkload(self.fused, m=4096, n=8192, k=4096)

    def make(self, rank, world, device):
        import torch
        from eval_test_b200 import shard
        data = super().make(rank, world, device)
        self.rank, self.world = rank, world
        if self.fused:
            if world > 1:
                self.out = shard.GatheredOutput(self.m, self.n, 1, device)
            else:
                buf = torch.empty((1, self.m, self.n), dtype=torch.float16, device=device)
                self.out = shard.GatheredOutput(self.m, self.n, 1, device, ptrs=[buf.data_ptr()], buf=buf)
        return data

    def run(self, data):
        from eval_test_b200 import nvfp4_gemm, shard
        if self.fused:
            # wait_all() orders "every rank has written" before the next thing on the stream; nothing reads C between
            # two steps here, so the second barrier of the protocol (GatheredOutput.release) has no reader to wait for
            shard.gemm_allgather(data, self.out, self.rank, alpha=self.alpha)
            self.out.wait_all()
            return self.out.view()
        self.last = shard.gather_cols(nvfp4_gemm.custom_kernel(data, alpha=self.alpha), self.world)
        return self.last

    def verify(self, data, ctx) -> str:
        """Every rank rebuilds all ranks' column shards of B from their seeds, computes the unsharded product with the
        plain kernel and compares its gathered copy of C with it bit for bit; "ok" only if all ranks agree."""
        import torch
        from eval_test_b200 import inputs, nvfp4_gemm
        a, _, sfa, _, sfa_p, _, _ = data
        dev, n_loc = a.device, self.n // self.world
        self.run(data)
        torch.cuda.synchronize()
        got = (self.out.view() if self.fused else self.last).clone()
        good = True
        for r in range(self.world):
            g = torch.Generator(device=dev).manual_seed(1000 + r)
            b, sfb, sfb_p = inputs.quantized_operand(1, n_loc, self.k, g, dev)
            c = torch.empty((1, self.m, n_loc), dtype=torch.float16, device=dev).permute(1, 2, 0)
            nvfp4_gemm.custom_kernel((a, b, sfa, sfb, sfa_p, sfb_p, c), alpha=self.alpha)
            good = good and torch.equal(got[:, r * n_loc:(r + 1) * n_loc].view(torch.int16), c.view(torch.int16))
        flag = torch.tensor([1.0 if good else 0.0], device=dev)
        if self.world > 1:
            ctx.dist.all_reduce(flag, op=ctx.dist.ReduceOp.MIN)
        return "ok" if bool(flag.item() == 1.0) else "MISMATCH"

    def io(self, data):
        ins, outs = super().io(data)
        return ins, ([self.out.buf] if self.fused else outs)

    def config(self, world):
        cfg = super().config(world)
        cfg["sharding"] = ("columns of C per rank; every rank ends with the full C: " +
                           ("fused all-gather epilogue (peer stores) + barrier" if self.fused
                            else "kernel, then NCCL all-gather of the shards"))
        return cfg

    def target_us(self, world, tensor_peak_tflops):
        send = 2 * self.m * (self.n // world) * (world - 1)
        return max(self.work(world) / (tensor_peak_tflops * 1e12), send / (self.nvlink_gbs * 1e9)) * 1e6


class DualGemmWorkload(GemmWorkload):
    """SwiGLU up-projection: C = silu(A.B1) * (A.B2), A 4096 x 4096, B1 and B2 14336 x 4096."""
    name = "dual_gemm_m4096_n14336_k4096"
    metric = "nvfp4_dual_gemm_tflops"
    kernel = "gemm_pair_kernel"
    alpha = 1.0

    def __init__(self, m=4096, n=14336, k=4096):
        super().__init__(m, n, k)

    def small(self):
        return DualGemmWorkload(m=2048, n=7168, k=4096)

    def work(self, world=1, m=None, n=None) -> int:
        return 2 * super().work(world, m, n)

    def make(self, rank, world, device):
        from eval_test_b200 import inputs
        import torch
        a, _, sfa, _, sfa_p, _, _ = inputs.gemm_quantized(self.m, 128, self.k, 1, seed=0, device=device)
        g = torch.Generator(device=device).manual_seed(1000 + rank)
        n = self.n // world
        b1, sfb1, sfb1_p = inputs.quantized_operand(1, n, self.k, g, device)
        b2, sfb2, sfb2_p = inputs.quantized_operand(1, n, self.k, g, device)
        c = torch.empty((1, self.m, n), dtype=torch.float16, device=device).permute(1, 2, 0)
        return (a, b1, b2, sfa, sfb1, sfb2, sfa_p, sfb1_p, sfb2_p, c)

    def run(self, data):
        from eval_test_b200 import nvfp4_dual_gemm
        return nvfp4_dual_gemm.custom_kernel(data)

    def io(self, data):
        a, b1, b2, _, _, _, sfa_p, sfb1_p, sfb2_p, c = data
        return [a, b1, b2, sfa_p, sfb1_p, sfb2_p], [c]

    def with_inputs(self, data, moved):
        return (moved[0], moved[1], moved[2], data[3], data[4], data[5], moved[3], moved[4], moved[5], data[9])

    def config(self, world):
        cfg = super().config(world)
        cfg.pop("alpha")
        cfg["l2"] = "operands + output (193 MB at 1 GPU) larger than L2 (126 MB)"
        return cfg

    def cpu_samples(self, data):
        from oracle import nvfp4_oracle as O
        u = _util()
        a, b1, b2, _, _, _, sfa_p, sfb1_p, sfb2_p, _ = data
        out = []
        for route, rows, cols, fn in (("fused_c", 128, 512, O.c_dual_gemm),
                                      ("dequant_matmul", a.shape[0], b1.shape[0], O.dq_dual_gemm)):
            rows, cols = min(rows, a.shape[0]), min(cols, b1.shape[0])
            nb = cols // 128
            args = (u.operand_np(a[:rows]), u.operand_np(b1[:cols]), u.operand_np(b2[:cols]),
                    u.scales_np(sfa_p[:, :, : (rows + 127) // 128]), u.scales_np(sfb1_p[:, :, :nb]),
                    u.scales_np(sfb2_p[:, :, :nb]))
            what = ("the whole problem" if (rows, cols) == (a.shape[0], b1.shape[0]) else
                    f"rows 0..{rows - 1} of A against rows 0..{cols - 1} of B1, B2")
            out.append((route, (lambda fn=fn, args=args: fn(*args)), self.work(m=rows, n=cols), what))
        return out

class DualGemmNvfp4Workload(DualGemmWorkload):
    """The same up-projection with the result emitted as NVFP4 (packed e2m1 + swizzled block scales) for the
    down-projection: the quantiser fused into the epilogue.  Same flops; 33 MB written per step instead of 117 MB."""
    name = "dual_gemm_nvfp4out_m4096_n14336_k4096"
    metric = "nvfp4_dual_gemm_nvfp4out_tflops"
    dtype = "e2m1 x ue4m3 scales on tcgen05 (kind::mxf4nvf4), fp32 accumulate, fp16 rounding, NVFP4 out"
    kernel = "gemm_kernel"

    def small(self):
        return DualGemmNvfp4Workload(m=2048, n=7168, k=4096)

    def run(self, data):
        from eval_test_b200 import nvfp4_dual_gemm
        self.last = nvfp4_dual_gemm.custom_kernel_nvfp4(data)
        return self.last

    def io(self, data):
        a, b1, b2, _, _, _, sfa_p, sfb1_p, sfb2_p, _ = data
        op, _, sf_p = getattr(self, "last", None) or self.run(data)
        return [a, b1, b2, sfa_p, sfb1_p, sfb2_p], [op, sf_p]


class GroupedGemmWorkload:
    """MoE expert layer: 64 groups, N = 4096, K = 7168, M_g ~ Poisson(128) clipped to [0, 1024] from
    numpy.random.default_rng(0).  At this M the layer is HBM-bound (every weight byte is read once), so the
    metric is algorithmic GB/s.  N > 1: the groups are dealt to the ranks by shard.assign_groups, balanced by weight
    bytes (strong scaling)."""
    name = "grouped_gemm_g64_n4096_k7168_poisson128"
    metric = "nvfp4_grouped_gemm_hbm_gbs"
    unit, per = "GB/s", 1e9
    dtype = "e2m1 x ue4m3 scales on tcgen05 (kind::mxf4nvf4), fp32 accumulate, fp16 out"
    bound, kernel, scaling = "hbm", "gemm_kernel", "strong"

    def __init__(self, g=64, n=4096, k=7168, mean=128.0, forced_empty=()):
        from eval_test_b200 import inputs
        self.g, self.n, self.k = g, n, k
        self.ms = inputs.poisson_group_sizes(g, mean, 0, 1024, seed=0)
        self.forced_empty = tuple(i for i in forced_empty if i < g)
        for i in self.forced_empty:   # a seeded Poisson(128) draw never gives an empty group: force some
            self.ms[i] = 0
        if self.forced_empty:
            self.name += f"_{len(self.forced_empty)}empty"

    def small(self):
        return GroupedGemmWorkload(g=16, forced_empty=self.forced_empty)

    def flush_l2(self, world):
        return self.work(world) < 132e6

    def _mine(self, rank, world):
        """Sizes of the groups of `rank`: whole groups, balanced by weight bytes (shard.assign_groups)."""
        from eval_test_b200 import shard
        return [self.ms[i] for i in shard.assign_groups(self.ms, world)[rank]]

    def _bytes(self, ms, n=None):
        n, k = (self.n if n is None else n), self.k
        w = sum(n * k // 2 + n * k // 16 for m in ms if m > 0)
        return w + sum(m * k // 2 + (m + 127) // 128 * 128 * k // 16 + 2 * m * n for m in ms)

    def work(self, world=1) -> int:
        """Algorithmic bytes of the busiest rank: weights and their scales of every non-empty group, activations,
        their (128-row padded) scales and the fp16 outputs."""
        return max(self._bytes(self._mine(r, world)) for r in range(world))

    def flops(self) -> int:
        return sum(2 * m * self.n * self.k for m in self.ms)

    def job(self, world=1) -> int:
        return self._bytes(self.ms)

    def make(self, rank, world, device):
        from eval_test_b200 import inputs
        ms = self._mine(rank, world)
        return inputs.grouped_gemm_quantized(ms, [self.n] * len(ms), [self.k] * len(ms), len(ms), seed=rank,
                                             device=device)

    def run(self, data):
        from eval_test_b200 import nvfp4_grouped_gemm
        return nvfp4_grouped_gemm.custom_kernel(data)

    def io(self, data):
        abc, _, sfs_p, _ = data
        ins = [t for (a, b, _), (sa, sb) in zip(abc, sfs_p) for t in (a, b, sa, sb) if t.numel()]
        return ins, [c for (_, _, c) in abc if c.numel()]

    def with_inputs(self, data, moved):
        abc, sfs, sfs_p, sizes = data
        it = iter(moved)
        new_abc, new_p = [], []
        for (a, b, c), (sa, sb) in zip(abc, sfs_p):
            a2, b2, sa2, sb2 = (next(it) if t.numel() else t for t in (a, b, sa, sb))
            new_abc.append((a2, b2, c))
            new_p.append((sa2, sb2))
        return (new_abc, sfs, new_p, sizes)

    def config(self, world):
        return {"workload": self.name, "groups": self.g, "n": self.n, "k": self.k, "sum_m": sum(self.ms),
                "min_m": min(self.ms), "max_m": max(self.ms), "empty_groups": sum(m == 0 for m in self.ms),
                "flop_per_step": sum(2 * m * self.n * self.k for m in self.ms),
                "forced_empty": list(self.forced_empty),
                "sharding": "whole groups per rank, balanced by weight bytes (non-empty groups), no collective",
                "l2": (f"weights ({self.work(world) / 1e6:.0f} MB per step and rank) larger than L2 (126 MB)"
                       if self.work(world) > 132e6 else
                       f"{self.work(world) / 1e6:.0f} MB per step and rank fit in L2: 512 MiB written between steps"),
                "generator": "M_g = clip(Poisson(128), 0, 1024), numpy default_rng(0); operands N(0,1) -> quantiser"}

    def cpu_samples(self, data):
        from oracle import nvfp4_oracle as O
        u = _util()
        abc, _, sfs_p, _ = data
        live = [i for i, (a, _, _) in enumerate(abc) if a.shape[0] > 0]
        out = []
        for route, groups, cols, fn in (("fused_c", 2, 256, O.c_grouped_gemm), ("dequant_matmul", 8, self.n, O.dq_grouped_gemm)):
            pick = live[:groups]
            args = [(u.operand_np(abc[i][0])[0], u.operand_np(abc[i][1][:cols])[0], u.scales_np(sfs_p[i][0]),
                     u.scales_np(sfs_p[i][1][:, :, : cols // 128])) for i in pick]
            ms = [g[0].shape[0] for g in args]
            what = f"the first {len(pick)} non-empty groups" + ("" if cols == self.n else f", rows 0..{cols - 1} of each B")
            out.append((route, (lambda fn=fn, args=args: fn(args)), self._bytes(ms, n=cols), what + f", K = {self.k}"))
        return out


class QuantizeWorkload:
    """fp32 -> NVFP4 quantiser in front of the path: one 16384 x 16384 fp32 operand per step (HBM-bound:
    4 bytes read, 0.5 + 1/16 bytes written per element).  N > 1: every rank quantises its own operand (weak)."""
    name = "quantize_f32_16384x16384"
    metric = "nvfp4_quantize_hbm_gbs"
    unit, per = "GB/s", 1e9
    dtype = "fp32 in, e2m1 + e4m3 block scales out"
    cpu_dtype = dtype
    bound, kernel, scaling = "hbm", "quantize_f32_kernel", "weak"

    def __init__(self, rows=16384, k=16384):
        self.rows, self.k = rows, k

    def small(self):
        return QuantizeWorkload(rows=4096)

    def work(self, world=1, rows=None) -> int:
        rows = self.rows if rows is None else rows
        return rows * self.k * 4 + rows * self.k // 2 + rows * self.k // 16

    def job(self, world=1) -> int:
        return self.work() * world

    def make(self, rank, world, device):
        import torch
        g = torch.Generator(device=device).manual_seed(rank)
        x = torch.randn((1, self.rows, self.k), generator=g, device=device)
        return [x, None]

    def run(self, data):
        from eval_test_b200 import quantize
        data[1] = quantize.quantize_operand(data[0], ref_scales=False)   # one launch: the kernel alone
        return data[1]

    def io(self, data):
        op, _, sf_p = data[1] if data[1] is not None else self.run(data)
        return [data[0]], [op, sf_p]

    def with_inputs(self, data, moved):
        return [moved[0], None]

    def config(self, world):
        return {"workload": self.name, "rows": self.rows, "k": self.k, "sharding": "one operand per rank",
                "l2": "1 GiB input larger than L2 (126 MB)", "generator": "N(0,1), seed = rank"}

    def flush_l2(self, world):
        return False

    def cpu_samples(self, data, rows=1024):
        from eval_test_b200 import formats as F
        x = data[0][:, :rows].cpu()

        def run():
            packed, sf = F.quantize_nvfp4(x)
            return packed, F.swizzle_scales(sf)
        return [("torch_ops", run, self.work(rows=rows),
                 f"rows 0..{rows - 1} (torch CPU ops, formats.quantize_nvfp4 + swizzle)")]


FORCED_EMPTY = (3, 17, 18, 40, 63)
WORKLOADS = {"gemv": GemvWorkload, "gemv_rowsplit": lambda: GemvWorkload(strong=True),
             "grouped_gemm_empty": lambda: GroupedGemmWorkload(forced_empty=FORCED_EMPTY),
             "gemm": GemmWorkload, "dual_gemm": DualGemmWorkload,
             "dual_gemm_nvfp4": DualGemmNvfp4Workload,
             "gemm_gather_fused": lambda: GemmGatherWorkload(True), "gemm_gather_nccl": lambda: GemmGatherWorkload(False),
             "grouped_gemm": GroupedGemmWorkload, "quantize": QuantizeWorkload}




# ----------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Polls NVML (SM clock, power, event reasons) for one GPU while launches run.  The timed region of a short run
    lasts a few milliseconds, less than one NVML refresh, so the record also covers an untimed continuation of the
    same launches (see measure()): what the clock settles at under this workload, power cap included."""
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        self.samples, self.power, self.reasons, self.max_mhz = [], [], set(), None
        self.in_timed = 0
        self.timed = False
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _poll(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                self.in_timed += 1 if self.timed else 0
                bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                for bit, name in self.REASONS.items():
                    if bits & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.001)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._poll, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self):
        s, w = sorted(self.samples), sorted(self.power)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_min_mhz": s[0] if s else None, "sm_max_mhz": self.max_mhz,
                "power_w": w[len(w) // 2] if w else None, "samples": len(s), "samples_in_timed_region": self.in_timed,
                "reasons": sorted(self.reasons),
                "window": "the timed region and an untimed continuation of the same launches (at least 0.25 s)"}


# ----------------------------------------------------------------------------------------------- CPU arm
def _host_threads() -> int:
    """All host cores, set explicitly: a launcher may have exported OMP_NUM_THREADS=1 for its workers."""
    import torch
    from oracle import nvfp4_oracle as O
    n = os.cpu_count() or 1
    O.set_num_threads(n)
    torch.set_num_threads(n)
    return n


def _time_cpu(fn, budget_s=8.0, max_runs=10):
    """One warm-up run (thread pools, page faults), then up to `max_runs` timed runs within the budget.  Returns the
    per-run seconds and, for routes that report them, the (dequantise, matmul) phase times."""
    time.sleep(0.3)          # let the worker threads of whatever ran before (another OpenMP runtime's pool) go idle
    t0 = time.perf_counter()
    fn()
    first = time.perf_counter() - t0
    runs, phases = [], []
    spent = first
    while len(runs) < max_runs and (not runs or spent + first <= budget_s):
        t0 = time.perf_counter()
        res = fn()
        dt = time.perf_counter() - t0
        runs.append(dt)
        spent += dt
        if isinstance(res, tuple) and len(res) == 3 and isinstance(res[1], float):
            phases.append((res[1], res[2]))
    return runs, phases


def _median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def cpu_baseline(wl, data):
    """The CPU restatement of the path on the host cores (all of them), two routes, median of up to 10 runs each:
    `fused_c`: the C oracle (exact integer block dot products, fp32 accumulation, OpenMP) on a bounded row sample;
    `dequant_matmul`: dequantise to fp32 (C, OpenMP) then torch.matmul in fp32 - the shape of computation the
    reference's oracle has - on the whole problem where that takes seconds, else on a sample; its two phases are
    listed apart.  `value` is the faster route's."""
    from oracle import nvfp4_oracle as O
    O.build()
    cores = _host_threads()
    routes = {}
    for route, fn, units, what in wl.cpu_samples(data):
        runs, phases = _time_cpu(fn)
        med = _median(runs)
        rec = {"value": units / med / wl.per, "best": units / min(runs) / wl.per, "seconds": med, "runs": len(runs),
               "spread": (max(runs) - min(runs)) / med, "sample": what}
        if phases:
            rec["dequantise_s"] = _median([p[0] for p in phases])
            rec["matmul_s"] = _median([p[1] for p in phases])
        routes[route] = rec
    best = max(routes, key=lambda r: routes[r]["value"])
    return {"value": routes[best]["value"], "unit": wl.unit, "cores": cores, "kind": "port", "route": best,
            "sample": routes[best]["sample"] + f"; median of {routes[best]['runs']} runs after a warm-up run",
            "routes": routes}


def cpu_c0():
    """BASELINE configuration 0, the CPU-runnable case, in full: GEMM 128 x 256 x 512, N(0,1) seed 0 through the
    quantiser, alpha = 1, both CPU routes."""
    from eval_test_b200 import inputs
    wl = GemmWorkload(128, 256, 512)
    wl.alpha = 1.0
    rec = cpu_baseline(wl, inputs.gemm_quantized(128, 256, 512, 1, seed=0, device="cpu"))
    rec["config"] = {"workload": "gemm_m128_n256_k512", "flop": wl.work()}
    return rec


def _reference_record(wl, args, steps, warmup):
    """K steps of the faster CPU route on this workload's sample (see cpu_baseline)."""
    import torch
    from oracle import nvfp4_oracle as O
    O.build()
    cores = _host_threads()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if torch.cuda.is_available() else "cpu"
    data = wl.make(0, 1, dev)     # the same seeded inputs as the GPU arm's rank 0; generated where it is fastest
    probes = []
    for route, fn, units, what in wl.cpu_samples(data):
        t0 = time.perf_counter()
        fn()
        probes.append((units / (time.perf_counter() - t0), route, fn, units, what))
    del data
    _, route, fn, units, what = max(probes, key=lambda p: p[0])
    for _ in range(max(0, min(warmup, 2) - 1)):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    val = units / dt / wl.per
    return {"impl": "reference", "metric": wl.metric, "value": val, "unit": wl.unit, "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": wl.scaling, "vs_baseline": None,
            "dtype": getattr(wl, "cpu_dtype", "e2m1 x ue4m3 scales, fp32 accumulate, fp16 out (CPU, " + route + ")"),
            "data": "synthetic", "config": wl.config(args.gpus),
            "cpu_baseline": {"value": val, "unit": wl.unit, "cores": cores, "kind": "port", "route": route,
                             "sample": "each step = " + what},
            "e2e": {"value": val, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def run_reference(args, names):
    """Reference arm: the reference has no CPU implementation of this path (its oracle is a cuBLASLt call), so this
    times the CPU restatement of it with all host threads, rank 0 only; the other ranks exit without work."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    head = _reference_record(WORKLOADS[names[0]](), args, args.steps, args.warmup)
    if len(names) > 1:
        head["workloads"] = {n: _reference_record(WORKLOADS[n](), args, max(1, min(args.steps, 5)), 1)
                             for n in names[1:] if not n.startswith("gemm_gather")}
    print(json.dumps(head), flush=True)


# ----------------------------------------------------------------------------------------------- GPU arm
NOMINAL = {"hbm": 8000.0, "tensor": 9000.0}   # GB/s and TFLOP/s the target statement quotes


def tensor_peak_tflops() -> tuple[float, str]:
    """Dense FP4 ceiling used for tensor-bound workloads: 4 x the measured bf16 GEMM rate of this pool (the
    FP4 tensor path issues 4 x the bf16 flops per clock: 9 vs 2.25 PFLOP/s nominal)."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return 4.0 * float(json.loads(p.read_text())["bf16_tflops"]), "4 x measured bf16 burst"
        except Exception:
            pass
    return 4.0 * 1590.0, "4 x fallback bf16"


class Ctx:
    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        assert self.world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={self.world}"
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = dist
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.flush_buf = None

    def barrier(self):
        import torch
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def flush(self):
        """Write 512 MiB (four times the L2) on the current stream."""
        import torch
        if self.flush_buf is None:
            self.flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=self.dev)
        self.flush_buf.fill_(0)

    def close(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def measure(wl, ctx, args, with_cpu=True):
    """All ranks run; rank 0 returns the record."""
    import torch
    from eval_test_b200 import _lib
    rank, world, dev = ctx.rank, ctx.world, ctx.dev
    data = wl.make(rank, world, dev)
    stream = torch.cuda.current_stream()
    flush = hasattr(wl, "flush_l2") and wl.flush_l2(world)

    for _ in range(args.warmup):
        wl.run(data)
    ctx.barrier()

    with ClockSampler(ctx.local_rank) as clocks:
        if not flush:
            # ---- timed region: K steps back to back, device-resident inputs larger than the L2 ----
            # One kernel launch per step and nothing else on the stream, so the average launch duration is the event
            # time over the region divided by the launches (launch gaps included: an upper bound of the kernel's own
            # time; an event pair around every launch would put two more stream operations between the kernels).
            t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ctx.barrier()
            clocks.timed = True
            t_begin.record(stream)
            for _ in range(args.steps):
                wl.run(data)
            t_end.record(stream)
            ctx.barrier()
            clocks.timed = False
            total_ms = t_begin.elapsed_time(t_end)
        else:
            # ---- this rank's inputs fit in the L2: 512 MiB are written before every step, outside its event pair ----
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
            ctx.barrier()
            clocks.timed = True
            for b, e in pairs:
                ctx.flush()
                b.record(stream)
                wl.run(data)
                e.record(stream)
            ctx.barrier()
            clocks.timed = False
            total_ms = sum(b.elapsed_time(e) for b, e in pairs)
        # ---- untimed continuation of the same launches, so that NVML sees the clock this workload settles at ----
        t0 = time.perf_counter()
        while not args.small and time.perf_counter() - t0 < 0.25:
            for _ in range(20):
                wl.run(data)
            torch.cuda.synchronize()
    kern_ms = total_ms / args.steps
    status = _lib.device_status(ctx.local_rank)
    assert status == 0, f"device status {status}: {_lib.strerror(status)}"
    check = wl.verify(data, ctx) if hasattr(wl, "verify") else None

    # ---- end to end: pinned host inputs -> device, kernel, outputs -> host, every step ----
    def flat(t):
        """All elements of a dense (possibly permuted) tensor as one 1-D view over its memory."""
        if t.element_size() == 1:
            t = t.view(torch.uint8)
        return torch.as_strided(t, (t.numel(),), (1,), t.storage_offset())

    ins, outs = wl.io(data)
    host_in = [torch.empty(t.numel(), dtype=flat(t).dtype).pin_memory() for t in ins]
    for h, t in zip(host_in, ins):
        h.copy_(flat(t))
    host_out = [torch.empty(o.numel(), dtype=flat(o).dtype).pin_memory() for o in outs]
    dev_in = [torch.empty_like(t) for t in ins]
    for d, t in zip(dev_in, ins):
        assert d.stride() == t.stride()
    e2e_data = wl.with_inputs(data, dev_in)
    h2d = sum(t.numel() * t.element_size() for t in ins)
    d2h = sum(o.numel() * o.element_size() for o in outs)

    def e2e_step():
        for d, h in zip(dev_in, host_in):
            flat(d).copy_(h, non_blocking=True)
        wl.run(e2e_data)
        for h, o in zip(host_out, wl.io(e2e_data)[1]):
            h.copy_(flat(o), non_blocking=True)

    e2e_steps = 1 if args.small else args.e2e_steps
    for _ in range(0 if args.small else 2):
        e2e_step()
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    ctx.barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    # ---- max over ranks ----
    t = torch.tensor([total_ms, kern_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        ctx.dist.all_reduce(t, op=ctx.dist.ReduceOp.MAX)
    total_ms, kern_ms, e2e_ms = (float(v) for v in t.tolist())

    line = None
    if rank == 0:
        if wl.bound == "hbm":
            peak, peak_kind = measured_peaks()
            peak_unit = "GB/s"
        else:
            peak, peak_kind = tensor_peak_tflops()
            peak_unit = "TFLOP/s"
        units = wl.work(world)               # per rank (the busiest one)
        job = wl.job(world)                  # whole job, all ranks
        ms_per_step = total_ms / args.steps
        achieved = units / (kern_ms * 1e-3) / wl.per
        line = {
            "metric": wl.metric, "value": job / (ms_per_step * 1e-3) / wl.per, "unit": wl.unit,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic", "config": wl.config(world),
            "roofline": {"bound": wl.bound, "kernel": wl.kernel, "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind if wl.bound == "tensor" else f"of {peak_kind}", "unit": peak_unit,
                         "frac": achieved / peak, "frac_of_nominal": achieved / NOMINAL[wl.bound],
                         "nominal": NOMINAL[wl.bound], "units_per_launch": units, "us_per_launch": kern_ms * 1e3,
                         "traffic": None},
            "e2e": {"value": job / (e2e_ms * 1e-3) / wl.per, "unit": wl.unit,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "steps": e2e_steps},
            "gpu_launches": args.steps, "clocks": clocks.summary(),
        }
        if check is not None:
            line["allgather_check"] = check
        if hasattr(wl, "flops"):            # an HBM-bound GEMM: the flop rate beside the byte rate
            line["tflops"] = wl.flops() / (ms_per_step * 1e-3) / 1e12
        if hasattr(wl, "target_us"):   # compute + collective: achieved time against the slower of the two floors
            tgt = wl.target_us(world, peak)
            line["roofline"].update({"bound": "tensor or nvlink", "target_us": tgt, "frac": tgt / (kern_ms * 1e3),
                                     "nvlink_gbs": wl.nvlink_gbs})
        traffic = ROOT / "profiles" / "traffic.json"
        if traffic.exists():
            try:
                line["roofline"]["traffic"] = json.loads(traffic.read_text()).get(wl.name)
            except Exception:
                pass
        if world == 1 and with_cpu and not args.no_cpu_baseline and not args.small:
            line["cpu_baseline"] = cpu_baseline(wl, data)
    del data, e2e_data, dev_in, host_in, host_out, ins, outs
    torch.cuda.empty_cache()
    return line


DEFAULT_SET = ("gemv", "gemm", "dual_gemm", "grouped_gemm", "grouped_gemm_empty")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="all", choices=["all"] + sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--small", action="store_true", help="shrink the workload (profiler captures); not a bench value")
    args = ap.parse_args()
    multi = ["gemv_rowsplit", "gemm_gather_fused", "gemm_gather_nccl"] if args.gpus > 1 else []
    names = list(DEFAULT_SET) + multi if args.workload == "all" else [args.workload]

    if args.impl == "reference":
        run_reference(args, names)
        return

    assert args.warmup >= 3 or args.small, "at least 3 warm-up steps"
    ctx = Ctx(args)
    from eval_test_b200 import _lib
    _lib.load()

    def wl_of(name):
        wl = WORKLOADS[name]()
        return wl.small() if args.small else wl

    head = measure(wl_of(names[0]), ctx, args)
    subs = {}
    for name in names[1:]:
        subs[name] = measure(wl_of(name), ctx, args)
    if ctx.rank == 0:
        if subs:
            head["workloads"] = subs
            head["gpu_launches_all_workloads"] = args.steps * len(names)
            if ctx.world == 1 and not args.no_cpu_baseline and not args.small:
                head["cpu_baseline_c0"] = cpu_c0()
        print(json.dumps(head), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
