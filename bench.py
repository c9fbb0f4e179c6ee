#!/usr/bin/env python
"""Benchmark of the NVFP4 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic input.  The default workload is the
batched GEMV the headline metric is quoted on (M = K = 16384, L = 4, N(0,1) data through the block-16
quantiser): HBM-bound, reported in GB/s of algorithmic bytes.  With N > 1 (launched by torchrun, one process
per GPU) every rank runs a shard of the same size (rows of A are independent, so nothing is exchanged): weak
scaling, value = bytes of all ranks / max-over-ranks device time.

The JSON line carries, besides the contract keys: ``roofline`` (dominant kernel, CUDA-event duration against
the measured HBM peak), ``e2e`` (same metric through ``custom_kernel`` with pinned host inputs copied in and
the output copied out inside the timed region), ``cpu_baseline`` (the CPU oracle on the host cores, rank 0,
N = 1) and ``clocks`` (NVML samples taken during the timed region).

``--impl reference`` times the CPU oracle (the reference has no CPU implementation of this path; the oracle is
the restatement of it) with all host threads on a bounded sample of the same workload.
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
    sys.path.insert(0, str(ROOT / "tests"))
    import _util
    return _util


class GemvWorkload:
    """Batched GEMV: A 16384 x 16384 e2m1 with block-16 e4m3 scales times a quantised vector, batch 4.
    N > 1: every rank owns 16384 more rows of A (weak scaling, nothing exchanged)."""
    name = "gemv_m16384_k16384_l4"
    metric = "nvfp4_gemv_hbm_gbs"
    unit, per = "GB/s", 1e9
    dtype = "e2m1 x ue4m3 scales, block-scaled tensor-core products, fp32 accumulate, fp16 out"
    bound, kernel, scaling = "hbm", "gemv_tc_kernel", "weak"

    def __init__(self, m=16384, k=16384, l=4):
        self.m, self.k, self.l = m, k, l

    def small(self):
        return GemvWorkload(m=4096, k=self.k, l=self.l)

    def work(self, world=1, m=None) -> int:
        """Algorithmic bytes per rank and step: A + its scales + the vector and its scales + the fp16 output."""
        m = self.m if m is None else m
        return self.l * (m * self.k // 2 + m * self.k // 16 + (self.k // 2 + self.k // 16) + 2 * m)

    def job(self, world=1) -> int:
        return self.work() * world

    def make(self, rank, world, device):
        from eval_test_b200 import inputs
        return inputs.gemv_quantized(self.m, self.k, self.l, seed=rank, device=device)

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
        return {"workload": self.name, "m_per_gpu": self.m, "k": self.k, "l": self.l, "global_m": self.m * world,
                "sharding": "rows of A per rank, no collective",
                "l2": f"inputs ({self.work() / 1e6:.0f} MB per step) larger than L2 (126 MB)",
                "generator": "N(0,1) seed = rank -> block-16 quantiser (scale = amax/6 as e4m3, RNE e2m1)"}

    def cpu_sample(self, data, rows=2048):
        u = _util()
        rows = min(rows, self.m)
        a, b, _, _, sfa_p, sfb_p, _ = data
        args = (u.operand_np(a[:rows]), u.operand_np(b), u.scales_np(sfa_p[:, :, : rows // 128]), u.scales_np(sfb_p))
        return args, self.work(m=rows), f"rows 0..{rows - 1} of each of the {self.l} batches, K = {self.k}"

    def cpu_data(self, rows=2048):
        from eval_test_b200 import inputs
        return inputs.gemv_quantized(min(rows, self.m), self.k, self.l, seed=0, device="cpu")

    def cpu_run(self, args):
        from oracle import nvfp4_oracle as O
        return O.c_gemv(*args)


class GemmWorkload:
    """Large GEMM: M = N = K = 8192, alpha = 0.5.  N > 1: B, its scales and C are split along N (strong scaling,
    no K split, so nothing is reduced or exchanged)."""
    name = "gemm_m8192_n8192_k8192"
    metric = "nvfp4_gemm_tflops"
    unit, per = "TFLOPS", 1e12
    dtype = "e2m1 x ue4m3 scales on tcgen05 (kind::mxf4nvf4), fp32 accumulate, fp16 out"
    bound, kernel, scaling = "tensor", "gemm_kernel", "strong"
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

    def cpu_sample(self, data, rows=128, cols=1024):
        u = _util()
        a, b, _, _, sfa_p, sfb_p, _ = data
        cols = min(cols, b.shape[0])
        args = (u.operand_np(a[:rows]), u.operand_np(b[:cols]), u.scales_np(sfa_p[:, :, : rows // 128]),
                u.scales_np(sfb_p[:, :, : cols // 128]), self.alpha)
        return args, self.work(m=rows, n=cols), f"rows 0..{rows - 1} of A against rows 0..{cols - 1} of B, K = {self.k}"

    def cpu_data(self, rows=128, cols=1024):
        from eval_test_b200 import inputs
        return inputs.gemm_quantized(rows, cols, self.k, 1, seed=0, device="cpu")

    def cpu_run(self, args):
        from oracle import nvfp4_oracle as O
        return O.c_gemm(*args)


class GemmGatherWorkload(GemmWorkload):
    """The same N-sharded GEMM with the full C assembled on every rank inside the timed step: either the kernel's
    fused all-gather epilogue (stores into every rank's copy over NVLink, then a barrier) or the kernel followed by
    an NCCL all-gather of the column shards.  The roofline target is the slower of the rank's flops at the tensor
    peak and the bytes the rank must send at 770 GB/s (measured peer-copy bandwidth per direction)."""
    metric = "nvfp4_gemm_allgather_tflops"
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
            shard.gemm_allgather(data, self.out, self.rank, alpha=self.alpha)
            self.out.wait_all()
            return self.out.view()
        return shard.gather_cols(nvfp4_gemm.custom_kernel(data, alpha=self.alpha), self.world)

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
    kernel = "gemm_kernel"
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

    def cpu_sample(self, data, rows=128, cols=512):
        u = _util()
        a, b1, b2, _, _, _, sfa_p, sfb1_p, sfb2_p, _ = data
        cols = min(cols, b1.shape[0])
        nb = cols // 128
        args = (u.operand_np(a[:rows]), u.operand_np(b1[:cols]), u.operand_np(b2[:cols]),
                u.scales_np(sfa_p[:, :, : rows // 128]), u.scales_np(sfb1_p[:, :, :nb]), u.scales_np(sfb2_p[:, :, :nb]))
        return args, self.work(m=rows, n=cols), f"rows 0..{rows - 1} of A against rows 0..{cols - 1} of B1, B2"

    def cpu_data(self, rows=128, cols=512):
        from eval_test_b200 import inputs
        return inputs.dual_gemm_quantized(rows, cols, self.k, 1, seed=0, device="cpu")

    def cpu_run(self, args):
        from oracle import nvfp4_oracle as O
        return O.c_dual_gemm(*args)

class DualGemmNvfp4Workload(DualGemmWorkload):
    """The same up-projection with the result emitted as NVFP4 (packed e2m1 + swizzled block scales) for the
    down-projection: the quantiser fused into the epilogue.  Same flops; 33 MB written per step instead of 117 MB."""
    name = "dual_gemm_nvfp4out_m4096_n14336_k4096"
    metric = "nvfp4_dual_gemm_nvfp4out_tflops"
    dtype = "e2m1 x ue4m3 scales on tcgen05 (kind::mxf4nvf4), fp32 accumulate, fp16 rounding, NVFP4 out"

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
    metric is algorithmic GB/s.  N > 1: groups are dealt round-robin to the ranks (strong scaling)."""
    name = "grouped_gemm_g64_n4096_k7168_poisson128"
    metric = "nvfp4_grouped_gemm_hbm_gbs"
    unit, per = "GB/s", 1e9
    dtype = "e2m1 x ue4m3 scales on tcgen05 (kind::mxf4nvf4), fp32 accumulate, fp16 out"
    bound, kernel, scaling = "hbm", "gemm_kernel", "strong"

    def __init__(self, g=64, n=4096, k=7168, mean=128.0):
        from eval_test_b200 import inputs
        self.g, self.n, self.k = g, n, k
        self.ms = inputs.poisson_group_sizes(g, mean, 0, 1024, seed=0)

    def small(self):
        return GroupedGemmWorkload(g=16)

    def _mine(self, rank, world):
        return self.ms[rank::world]

    def _bytes(self, ms, n=None):
        n, k = (self.n if n is None else n), self.k
        w = sum(n * k // 2 + n * k // 16 for m in ms if m > 0)
        return w + sum(m * k // 2 + (m + 127) // 128 * 128 * k // 16 + 2 * m * n for m in ms)

    def work(self, world=1) -> int:
        """Algorithmic bytes of the busiest rank: weights and their scales of every non-empty group, activations,
        their (128-row padded) scales and the fp16 outputs."""
        return max(self._bytes(self._mine(r, world)) for r in range(world))

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
                "sharding": "groups dealt round-robin to ranks, no collective",
                "l2": f"weights ({self.work() / 1e6:.0f} MB per step) larger than L2 (126 MB)",
                "generator": "M_g = clip(Poisson(128), 0, 1024), numpy default_rng(0); operands N(0,1) -> quantiser"}

    def cpu_sample(self, data, groups=2, cols=256):
        u = _util()
        abc, _, sfs_p, _ = data
        args = []
        for (a, b, _), (sa, sb) in list(zip(abc, sfs_p))[:groups]:
            args.append((u.operand_np(a)[0], u.operand_np(b[:cols])[0], u.scales_np(sa),
                         u.scales_np(sb[:, :, : cols // 128])))
        ms = [a[0].shape[0] for a in args]
        return args, self._bytes(ms, n=cols), f"groups 0..{groups - 1}, rows 0..{cols - 1} of each B, K = {self.k}"

    def cpu_data(self, groups=2, cols=256):
        from eval_test_b200 import inputs
        ms = self.ms[:groups]
        return inputs.grouped_gemm_quantized(ms, [cols] * groups, [self.k] * groups, groups, seed=0, device="cpu")

    def cpu_run(self, args):
        from oracle import nvfp4_oracle as O
        return O.c_grouped_gemm(args)


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

    def cpu_sample(self, data, rows=1024):
        x = data[0][:, :rows].cpu()
        return (x,), self.work(rows=rows), f"rows 0..{rows - 1} (torch CPU ops, formats.quantize_nvfp4 + swizzle)"

    def cpu_data(self, rows=1024):
        import torch
        return [torch.randn((1, rows, self.k), generator=torch.Generator().manual_seed(0)), None]

    def cpu_run(self, args):
        from eval_test_b200 import formats as F
        packed, sf = F.quantize_nvfp4(args[0])
        return packed, F.swizzle_scales(sf)


WORKLOADS = {"gemv": GemvWorkload, "gemm": GemmWorkload, "dual_gemm": DualGemmWorkload,
             "dual_gemm_nvfp4": DualGemmNvfp4Workload,
             "gemm_gather_fused": lambda: GemmGatherWorkload(True), "gemm_gather_nccl": lambda: GemmGatherWorkload(False),
             "grouped_gemm": GroupedGemmWorkload, "quantize": QuantizeWorkload}


# ----------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Polls NVML (SM clock, event reasons) for one GPU while the timed region runs."""
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
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
                bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                for bit, name in self.REASONS.items():
                    if bits & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.0005)

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
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "samples": len(s), "reasons": sorted(self.reasons)}


# ----------------------------------------------------------------------------------------------- CPU arm
def _time_cpu(wl, args, budget_s=20.0):
    t0 = time.perf_counter()
    wl.cpu_run(args)
    best = time.perf_counter() - t0
    for _ in range(2):
        if best * 3 > budget_s:
            break
        t0 = time.perf_counter()
        wl.cpu_run(args)
        best = min(best, time.perf_counter() - t0)
    return best


def cpu_baseline(wl, data):
    """The CPU oracle on the host cores over a bounded sample of the same inputs (best of 3)."""
    from oracle import nvfp4_oracle as O
    O.build()
    args, units, what = wl.cpu_sample(data)
    best = _time_cpu(wl, args)
    return {"value": units / best / wl.per, "unit": wl.unit, "cores": O.num_threads(), "kind": "port",
            "sample": what + "; best of 3", "seconds": best}


def run_reference(args, wl):
    """Reference arm: the reference has no CPU implementation of this path (its oracle is a cuBLASLt call), so
    this times the CPU restatement of it with all host threads; each step is a bounded sample (rank 0 only)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import nvfp4_oracle as O
    O.build()
    data = wl.cpu_data()
    sample, units, what = wl.cpu_sample(data)
    for _ in range(max(1, min(args.warmup, 2))):
        wl.cpu_run(sample)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        wl.cpu_run(sample)
    dt = (time.perf_counter() - t0) / args.steps
    val = units / dt / wl.per
    line = {"impl": "reference", "metric": wl.metric, "value": val, "unit": wl.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": wl.scaling, "vs_baseline": None,
            "dtype": getattr(wl, "cpu_dtype", "e2m1 x ue4m3 scales, exact int32 block dots, fp32 accumulate, fp16 out (CPU)"),
            "data": "synthetic",
            "config": wl.config(args.gpus),
            "cpu_baseline": {"value": val, "unit": wl.unit, "cores": O.num_threads(), "kind": "port",
                             "sample": "each step = " + what},
            "e2e": {"value": val, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------- GPU arm
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="gemv", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--small", action="store_true", help="shrink the workload (profiler captures); not a bench value")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]()
    if args.small:
        wl = wl.small()

    if args.impl == "reference":
        run_reference(args, wl)
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    assert args.warmup >= 3 or args.small, "at least 3 warm-up steps"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from eval_test_b200 import _lib
    _lib.load()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    data = wl.make(rank, world, dev)
    stream = torch.cuda.current_stream()

    for _ in range(args.warmup):
        wl.run(data)
    barrier()

    # ---- timed region: K steps, device-resident inputs ----
    # One kernel launch per step and nothing else on the stream, so the average launch duration is the event time
    # over the region divided by the launches (launch gaps included: an upper bound of the kernel's own time; an
    # event pair around every launch would put two more stream operations between the kernels).
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        t_begin.record(stream)
        for _ in range(args.steps):
            wl.run(data)
        t_end.record(stream)
        barrier()
    total_ms = t_begin.elapsed_time(t_end)
    kern_ms = total_ms / args.steps
    status = _lib.device_status(local_rank)
    assert status == 0, f"device status {status}: {_lib.strerror(status)}"

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
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    # ---- max over ranks ----
    t = torch.tensor([total_ms, kern_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, kern_ms, e2e_ms = (float(v) for v in t.tolist())

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
                         "frac": achieved / peak, "units_per_launch": units, "us_per_launch": kern_ms * 1e3,
                         "traffic": None},
            "e2e": {"value": job / (e2e_ms * 1e-3) / wl.per, "unit": wl.unit,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "steps": e2e_steps},
            "gpu_launches": args.steps, "clocks": clocks.summary(),
        }
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
        if world == 1 and not args.no_cpu_baseline and not args.small:
            line["cpu_baseline"] = cpu_baseline(wl, data)
        print(json.dumps(line), flush=True)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
