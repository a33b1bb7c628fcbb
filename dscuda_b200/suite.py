"""Benchmark suite of the MLA path, in the shape of the reference's harness.

    python -m dscuda_b200.suite --suite b200 [--configs C2,C3] [--trials 5] [--report report.md]

The reference times each operator with `benchmarks/run.py <name>` and writes a markdown
table (`benchmarks/common.py:114-141`).  This does the same for the five B200
configurations: one row per configuration with the time per call, TFLOP/s or GB/s on the
algorithmic work, the bounding roofline and the fraction of the measured peak reached.
Timing: CUDA events around back-to-back calls after warm-up, median over trials.
Inputs are seeded synthetic tensors (`dscuda_b200.workloads`); every call goes through the
C ABI of `build/libdscuda_mla_bench.so`.
"""
from __future__ import annotations

import argparse
import json
import pathlib
import statistics
import sys
from typing import Callable, Dict, List

import torch

from . import mla, workloads

ROOT = pathlib.Path(__file__).resolve().parents[1]


def peaks() -> dict:
    """Measured copy bandwidth and sustained cuBLAS bf16 rate of this machine when a
    MEASURED_PEAKS.json sits at the repository root, else an earlier measurement of the same GPU type."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return dict(tensor=float(data["bf16_tflops_sustained"]), hbm=float(data["hbm_gbs"]), source="measured")
    return dict(tensor=1400.0, hbm=6650.0, source="fallback")


def time_call(call: Callable[[], None], launches: int, trials: int, warmup: int = 3) -> float:
    """Median over `trials` of the mean seconds per call over `launches` back-to-back calls."""
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    samples = []
    for _ in range(trials):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(launches):
            call()
        stop.record()
        stop.synchronize()
        samples.append(start.elapsed_time(stop) / 1e3 / launches)
    return statistics.median(samples)


def run_dense(name: str, config: dict, device: torch.device, trials: int) -> dict:
    x = workloads.dense_inputs(config, device)
    ins = (x["q_nope"], x["q_pe"], x["k_nope"], x["k_pe"], x["v"])
    out = torch.empty_like(x["v"])
    lse = torch.empty(config["batch"], config["heads"], config["seq"], device=device)
    if config["backward"]:
        workspace = mla.prefill_backward_workspace(config["batch"], config["seq"], config["batch"] * config["seq"], config["heads"], device)
        grads = (torch.empty(config["batch"], config["seq"], config["heads"], 192, device=device, dtype=torch.bfloat16),
                 torch.empty_like(x["k_nope"]), torch.empty_like(x["k_pe"]), torch.empty_like(x["v"]))

    def call():
        mla.prefill_forward(*ins, workloads.SCALE, output=out, lse=lse)
        if config["backward"]:
            mla.prefill_backward(x["dout"], out, lse, *ins, workloads.SCALE, workspace=workspace, grads=grads)

    flops = workloads.dense_flops(config)
    launches = 20 if flops < 1e12 else 5
    seconds = time_call(call, launches, trials)
    what = "forward + backward" if config["backward"] else "forward"
    return dict(config=name, workload=f"causal MLA {what}, B={config['batch']} S={config['seq']} H={config['heads']}", seconds=seconds,
                value=flops / seconds / 1e12, unit="TFLOP/s", bound="tensor")


def run_packed(name: str, config: dict, device: torch.device, trials: int) -> dict:
    lengths = workloads.varlen_lengths(config["seed"], config["sequences"], config["low"], config["high"])
    x, cu = workloads.packed_inputs(lengths, config["heads"], config["seed"], device, config["dout_std"])
    ins = (x["q_nope"], x["q_pe"], x["k_nope"], x["k_pe"], x["v"])
    total, longest = sum(lengths), max(lengths)
    out = torch.empty_like(x["v"])
    lse = torch.empty(config["heads"], total, device=device)
    workspace = mla.prefill_backward_workspace(len(lengths), longest, total, config["heads"], device)
    grads = (torch.empty(total, config["heads"], 192, device=device, dtype=torch.bfloat16), torch.empty_like(x["k_nope"]),
             torch.empty_like(x["k_pe"]), torch.empty_like(x["v"]))

    def call():
        mla.prefill_forward(*ins, workloads.SCALE, cu, longest, output=out, lse=lse)
        mla.prefill_backward(x["dout"], out, lse, *ins, workloads.SCALE, cu, longest, workspace=workspace, grads=grads)

    seconds = time_call(call, 3, trials, warmup=1)
    flops = workloads.packed_flops(lengths, config["heads"])
    return dict(config=name, workload=f"packed causal MLA forward + backward, {len(lengths)} sequences, {total} tokens, H={config['heads']} (one GPU's heads)",
                seconds=seconds, value=flops / seconds / 1e12, unit="TFLOP/s", bound="tensor")


def run_decode(name: str, config: dict, device: torch.device, trials: int) -> dict:
    query, cache, table, lengths = workloads.decode_inputs(config["seed"], config["batch"], config["heads"], config["low"], config["high"],
                                                           config["page"])
    q, c, t, n = (z.to(device) for z in (query, cache, table, lengths))
    workspace = mla.decode_workspace(config["batch"], config["heads"], config["splits"], 512, device)
    out = torch.empty(config["batch"], 1, config["heads"], 512, device=device, dtype=torch.bfloat16)
    lse = torch.empty(config["batch"], config["heads"], 1, device=device)

    def call():
        mla.mla_decode(q, c, t, n, workloads.SCALE, config["splits"], workspace, out, lse)

    seconds = time_call(call, 20, trials)
    moved = workloads.decode_bytes(lengths, table, config["batch"], config["heads"])
    return dict(config=name, workload=f"absorbed paged decode, batch {config['batch']}, H={config['heads']}, {int(lengths.sum())} cached tokens, "
                                      f"{config['page']}-token pages", seconds=seconds, value=moved / seconds / 1e9, unit="GB/s", bound="hbm")


RUNNERS = {"dense": run_dense, "packed": run_packed, "decode": run_decode}


def run_suite(names: List[str], device: torch.device, trials: int) -> List[dict]:
    top = peaks()
    rows = []
    for name in names:
        config = workloads.CONFIGS[name]
        row = RUNNERS[config["kind"]](name, config, device, trials)
        peak = top["tensor"] if row["bound"] == "tensor" else top["hbm"]
        row["peak"] = peak
        row["fraction"] = row["value"] / peak
        row["peak_source"] = top["source"]
        rows.append(row)
        if mla.device_status() != 0:
            raise RuntimeError(f"{name}: a kernel reported a device-side error status")
    return rows


def format_report(rows: List[dict]) -> str:
    lines = ["| config | workload | ms per call | throughput | roofline | fraction of peak |", "|---|---|---|---|---|---|"]
    for row in rows:
        lines.append(f"| {row['config']} | {row['workload']} | {row['seconds'] * 1e3:.3f} | {row['value']:.1f} {row['unit']} | "
                     f"{row['bound']} ({row['peak']:.0f} {row['unit']}, {row['peak_source']}) | {row['fraction']:.3f} |")
    return "\n".join(lines)


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--suite", default="b200", choices=["b200"])
    parser.add_argument("--configs", default="C1,C2,C3,C4,C5", help="comma-separated subset of C1..C5")
    parser.add_argument("--trials", type=int, default=5)
    parser.add_argument("--device", type=int, default=0)
    parser.add_argument("--report", default=None, help="write the markdown table to this file as well")
    args = parser.parse_args(argv)
    names = [name.strip() for name in args.configs.split(",") if name.strip()]
    for name in names:
        if name not in workloads.CONFIGS:
            parser.error(f"unknown configuration {name}")
    if not torch.cuda.is_available():
        raise RuntimeError("the suite runs the CUDA kernels; no GPU is visible")
    device = torch.device("cuda", args.device)
    torch.cuda.set_device(device)
    rows = run_suite(names, device, args.trials)
    report = format_report(rows)
    print(report)
    if args.report:
        pathlib.Path(args.report).write_text("# MLA on B200: suite `b200`\n\n" + report + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
