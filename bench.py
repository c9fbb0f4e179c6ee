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
class GemvWorkload:
    """c1: A 16384 x 16384 e2m1 with block-16 e4m3 scales times a quantised vector, batch 4."""
    name = "gemv_m16384_k16384_l4"
    metric = "nvfp4_gemv_hbm_gbs"
    unit = "GB/s"
    dtype = "e2m1 x ue4m3 scales, int32 block dot, fp32 accumulate, fp16 out"
    bound = "hbm"
    kernel = "gemv_kernel"

    def __init__(self, m=16384, k=16384, l=4):
        self.m, self.k, self.l = m, k, l

    def bytes_per_step(self, m=None) -> int:
        """Algorithmic bytes: A + its scales + the vector and its scales + the fp16 output, per batch."""
        m = self.m if m is None else m
        per_batch = m * self.k // 2 + m * self.k // 16 + (self.k // 2 + self.k // 16) + 2 * m
        return self.l * per_batch

    def make(self, seed, device):
        from eval_test_b200 import inputs
        return inputs.gemv_quantized(self.m, self.k, self.l, seed=seed, device=device)

    def run(self, data):
        from eval_test_b200 import nvfp4_gemv
        return nvfp4_gemv.custom_kernel(data)

    def io_tensors(self, data):
        a, b, _, _, sfa_p, sfb_p, c = data
        return [a, b, sfa_p, sfb_p], c

    def rebuild(self, data, moved):
        a, b, sfa, sfb, sfa_p, sfb_p, c = data
        return (moved[0], moved[1], sfa, sfb, moved[2], moved[3], c)

    def config(self, n_gpus):
        return {"workload": self.name, "m_per_gpu": self.m, "k": self.k, "l": self.l,
                "global_m": self.m * n_gpus, "sharding": "rows of A per rank, no collective",
                "l2": "inputs (604 MB per step) larger than L2 (126 MB)",
                "generator": "N(0,1) seed 0 -> block-16 quantiser (scale = amax/6 as e4m3, RNE e2m1)"}

    # CPU side (oracle) -----------------------------------------------------------------------------
    def cpu_sample(self, data, rows):
        """Rows [0, rows) of every batch as oracle arrays (rows is a multiple of 128)."""
        sys.path.insert(0, str(ROOT / "tests"))
        from _util import operand_np, scales_np
        a, b, _, _, sfa_p, sfb_p, _ = data
        a_np = operand_np(a[:rows])
        sfa = scales_np(sfa_p[:, :, : rows // 128])
        return a_np, operand_np(b), sfa, scales_np(sfb_p)

    def cpu_run(self, sample):
        from oracle import nvfp4_oracle as O
        return O.c_gemv(*sample)


WORKLOADS = {"gemv": GemvWorkload}


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
            time.sleep(0.002)

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
def cpu_baseline(wl, data, budget_s=20.0):
    """Oracle on the host cores over a bounded sample (whole 128-row blocks of every batch)."""
    from oracle import nvfp4_oracle as O
    O.build()
    rows = min(wl.m, 2048)
    sample = wl.cpu_sample(data, rows)
    t0 = time.perf_counter()
    wl.cpu_run(sample)
    dt = time.perf_counter() - t0
    # grow the sample towards a few seconds of work, then keep the best of 3
    while dt < 1.0 and rows < wl.m:
        rows = min(wl.m, rows * 4)
        sample = wl.cpu_sample(data, rows)
        t0 = time.perf_counter()
        wl.cpu_run(sample)
        dt = time.perf_counter() - t0
    best = dt
    for _ in range(2):
        if best * 3 > budget_s:
            break
        t0 = time.perf_counter()
        wl.cpu_run(sample)
        best = min(best, time.perf_counter() - t0)
    return {"value": wl.bytes_per_step(rows) / best / 1e9, "unit": wl.unit, "cores": O.num_threads(),
            "kind": "port", "sample": f"rows 0..{rows - 1} of each of the {wl.l} batches, K = {wl.k}; best of 3",
            "seconds": best}


def run_reference(args, wl):
    """Reference arm: the CPU oracle, all host threads, bounded sample per step (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from oracle import nvfp4_oracle as O
    O.build()
    rows = 2048
    small = type(wl)(m=rows, k=wl.k, l=wl.l)
    data = small.make(seed=0, device="cpu")
    sample = small.cpu_sample(data, rows)
    for _ in range(max(1, min(args.warmup, 2))):
        small.cpu_run(sample)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        small.cpu_run(sample)
    dt = (time.perf_counter() - t0) / args.steps
    val = small.bytes_per_step() / dt / 1e9
    line = {"impl": "reference", "metric": wl.metric, "value": val, "unit": wl.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": wl.config(args.gpus),
            "cpu_baseline": {"value": val, "unit": wl.unit, "cores": O.num_threads(), "kind": "port",
                             "sample": f"each step = rows 0..{rows - 1} of each of the {wl.l} batches, K = {wl.k}"},
            "e2e": {"value": val, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="gemv", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--small", action="store_true", help="shrink the workload (profiler captures); not a bench value")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]()
    if args.small:
        wl = GemvWorkload(m=4096, k=16384, l=4)

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

    data = wl.make(seed=rank, device=dev)
    stream = torch.cuda.current_stream()

    for _ in range(args.warmup):
        wl.run(data)
    barrier()

    # ---- timed region: K steps, device-resident inputs ----
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        t_begin.record(stream)
        for s, e in ev:
            s.record(stream)
            wl.run(data)
            e.record(stream)
        t_end.record(stream)
        barrier()
    total_ms = t_begin.elapsed_time(t_end)
    kern_ms = sum(s.elapsed_time(e) for s, e in ev) / args.steps
    status = _lib.device_status(local_rank)
    assert status == 0, f"device status {status}: {_lib.strerror(status)}"

    # ---- end to end: pinned host inputs -> device, kernel, output -> host, every step ----
    def flat(t):
        """All elements of a dense (possibly permuted) tensor as one 1-D view over its memory."""
        return torch.as_strided(t if t.dtype == torch.float16 else t.view(torch.uint8), (t.numel(),), (1,),
                                t.storage_offset())

    ins, out = wl.io_tensors(data)
    host_in = [torch.empty(t.numel(), dtype=torch.uint8).pin_memory() for t in ins]
    for h, t in zip(host_in, ins):
        h.copy_(flat(t))
    host_out = torch.empty(out.numel(), dtype=out.dtype).pin_memory()
    dev_in = [torch.empty_like(t) for t in ins]
    for d, t in zip(dev_in, ins):
        assert d.stride() == t.stride()
    e2e_data = wl.rebuild(data, dev_in)
    h2d = sum(t.numel() * t.element_size() for t in ins)
    d2h = out.numel() * out.element_size()

    def e2e_step():
        for d, h in zip(dev_in, host_in):
            flat(d).copy_(h, non_blocking=True)
        res = wl.run(e2e_data)
        host_out.copy_(flat(res), non_blocking=True)

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
        peak, peak_kind = measured_peaks()
        step_bytes = wl.bytes_per_step()
        ms_per_step = total_ms / args.steps
        achieved = step_bytes / (kern_ms * 1e-3) / 1e9
        line = {
            "metric": wl.metric, "value": world * step_bytes / (ms_per_step * 1e-3) / 1e9, "unit": wl.unit,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic", "config": wl.config(world),
            "roofline": {"bound": wl.bound, "kernel": wl.kernel, "achieved": achieved, "peak": peak,
                         "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                         "bytes_per_launch": step_bytes, "us_per_launch": kern_ms * 1e3, "traffic": None},
            "e2e": {"value": world * step_bytes / (e2e_ms * 1e-3) / 1e9, "unit": wl.unit,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "steps": e2e_steps},
            "gpu_launches": args.steps, "clocks": clocks.summary(),
        }
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
