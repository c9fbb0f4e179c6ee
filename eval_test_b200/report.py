"""Markdown summary of a POPCORN log, in the role of the reference launcher's result formatter
(modal/cli.py:77-125 parses the ``key: value`` log, modal/cli.py:128-264 renders status lines, the machine, and
per-case timings as mean +- err with best and worst in microseconds).

What is added here: for benchmark cases the algorithmic bytes and flops of the shape and the time floor they imply
on the measured peaks of this machine class, so that a timing can be read against its bound at a glance.
"""
from __future__ import annotations

import ast
import platform

# measured on B200: STREAM-style copy bandwidth and 4 x the bf16 GEMM burst rate (the FP4 path issues 4 x the flops)
HBM_GBS = 6550.7
FP4_TFLOPS = 4 * 1664.6


def parse_log(text: str) -> dict:
    """``{"compile": str?, "check": str?, "tests": {i: {field: value}}, "benchmarks": {i: {...}}}``."""
    data: dict = {"tests": {}, "benchmarks": {}}
    for raw in text.splitlines():
        key, sep, value = raw.strip().partition(":")
        if not sep:
            continue
        key, value = key.strip(), value.strip()
        head, _, rest = key.partition(".")
        if head in ("test", "benchmark") and rest:
            idx, _, field = rest.partition(".")
            if idx.isdigit() and field:
                data["tests" if head == "test" else "benchmarks"].setdefault(int(idx), {})[field] = value
        elif key in ("compile", "check"):
            data[key] = value
        elif key == "compile.error":
            data["compile_error"] = value
        elif key in ("test-count", "benchmark-count"):
            data[key.replace("-", "_")] = int(value) if value.isdigit() else value
    return data


def _spec_args(spec_line: str) -> dict:
    out = {}
    for part in spec_line.split(";"):
        k, sep, v = part.partition(":")
        if sep:
            v = v.strip()
            try:
                out[k.strip()] = ast.literal_eval(v)
            except (ValueError, SyntaxError):
                out[k.strip()] = v
    return out


def work_of(task: str, args: dict) -> tuple[int, int]:
    """(algorithmic bytes, flops) of one call: packed operands, their block scales (rows padded to 128), fp16 output."""
    def operand(rows, k, l=1):
        return l * (rows * k // 2 + (rows + 127) // 128 * 128 * k // 16)
    if task == "nvfp4_gemv":
        m, k, l = args["m"], args["k"], args["l"]
        return operand(m, k, l) + l * (k // 2 + k // 16) + 2 * m * l, 2 * m * k * l
    if task == "nvfp4_gemm":
        m, n, k, l = args["m"], args["n"], args["k"], args["l"]
        return operand(m, k, l) + operand(n, k, l) + 2 * m * n * l, 2 * m * n * k * l
    if task == "nvfp4_dual_gemm":
        m, n, k, l = args["m"], args["n"], args["k"], args["l"]
        return operand(m, k, l) + 2 * operand(n, k, l) + 2 * m * n * l, 4 * m * n * k * l
    if task == "nvfp4_grouped_gemm":
        by = fl = 0
        for m, n, k in zip(args["m"], args["n"], args["k"]):
            if m > 0:
                by += operand(m, k) + operand(n, k) + 2 * m * n
                fl += 2 * m * n * k
        return by, fl
    raise ValueError(task)


def floor_us(task: str, args: dict) -> float:
    by, fl = work_of(task, args)
    return max(by / (HBM_GBS * 1e9), fl / (FP4_TFLOPS * 1e12)) * 1e6


def system_info() -> dict:
    info = {"platform": platform.platform(), "cpu": platform.processor() or platform.machine()}
    try:
        import torch
        info["torch"] = torch.__version__
        if torch.cuda.is_available():
            info["gpu"] = torch.cuda.get_device_name(0)
            info["device_count"] = torch.cuda.device_count()
    except Exception:
        pass
    return info


def format_report(data: dict, mode: str, task: str, system: dict | None = None) -> str:
    ok = data.get("check") == "pass" and data.get("compile") != "fail"
    lines = [f"**{task} {mode}: {'success' if ok else 'failure'}**"]
    if "compile" in data:
        lines.append(f"> compilation {'successful' if data['compile'] == 'pass' else 'failed'}")
        if data.get("compile_error"):
            lines.append(f"> {data['compile_error']}")
    if system:
        lines += ["", "Running on: " + ", ".join(f"{k} `{v}`" for k, v in system.items())]
    if data["benchmarks"]:
        lines += ["", "| case | mean us | err us | best us | worst us | runs | kernel us | floor us | mean / floor | kernel / floor | status |",
                  "|---|---|---|---|---|---|---|---|---|---|---|"]
        for i, b in sorted(data["benchmarks"].items()):
            try:
                mean, err, best, worst = (float(b[f]) / 1e3 for f in ("mean", "err", "best", "worst"))
                kern = float(b["kernel_us"]) if "kernel_us" in b else None
                try:
                    fl = floor_us(task, _spec_args(b.get("spec", "")))
                    tail = f"{fl:.1f} | {mean / fl:.2f} | " + (f"{kern / fl:.2f}" if kern is not None else "-")
                except Exception:
                    tail = "- | - | -"
                row = (f"{mean:.1f} | {err:.2f} | {best:.1f} | {worst:.1f} | {b.get('runs', '-')} | "
                       + (f"{kern:.1f}" if kern is not None else "-") + f" | {tail}")
            except (KeyError, ValueError):
                row = "- | - | - | - | - | - | - | - | -"
            status = "fail: " + b.get("error", "failed") if b.get("status") == "fail" or "error" in b else "ok"
            lines.append(f"| `{b.get('spec', i)}` | {row} | {status} |")
    elif data["tests"]:
        lines += ["", "| case | status |", "|---|---|"]
        for i, t in sorted(data["tests"].items()):
            status = t.get("status", "?") + (": " + t["error"] if "error" in t else "")
            lines.append(f"| `{t.get('spec', i)}` | {status} |")
    return "\n".join(lines)
