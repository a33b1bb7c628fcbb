"""Benchmark harness of the MLA path, in the shape of the reference's `benchmarks/run.py`.

    python -m dscuda_b200.suite --suite b200 [--configs C2,C3] [--test] [--operation forward|backward|decode]
                                [--graph-operations 10 --warmup-ms 1000 --sample-ms 20 --trials 9 | --eager]
                                [--gpus N] [--cpu-baseline] [--report-dir DIR]

What carries over from the reference (`benchmarks/run.py:12-26`, `benchmarks/common.py:68-141`):

* `--test`: correctness only.  Every configuration is run through the C ABI and compared with the
  CPU oracle (the role PyTorch expressions play in the reference's harness), no timing; prints
  "mla: N correctness checks passed" like the reference.
* timing: each call is captured `--graph-operations` times in a CUDA graph; the graph is replayed for
  `--warmup-ms`, then `--trials` samples of about `--sample-ms` each are taken and the median
  microseconds per call reported; the outputs are checked against the oracle before and after
  timing (`common.py:84-85,109-110`).  `--eager` times plain back-to-back launches instead.
* the report: one markdown table (one row per configuration: time per call, TFLOP/s or GB/s on the
  algorithmic work, the bounding roofline, the fraction of the measured peak, and with
  `--cpu-baseline` the CPU restatement's throughput on a bounded sample), plus with `--report-dir`
  a CSV and a samples JSON that records GPU, torch and CUDA versions (`common.py:114-141`).
* `--gpus N`: one worker process per GPU, each on its own shard (its own heads of the H = 128*N job,
  its share of the decode sequences); the row reports the slowest GPU's time and the job's
  throughput.  No collective is involved: the path has none.

This module is a harness around the product (the libraries and `dscuda_b200.mla`); like the
reference's harness it needs a checker, which is `oracle/` here.
"""
from __future__ import annotations

import argparse
import csv
import json
import math
import os
import pathlib
import statistics
import sys
import time
from typing import Callable, Dict, List, Optional

import torch

from . import mla, sharding, workloads

ROOT = pathlib.Path(__file__).resolve().parents[1]


def peaks() -> dict:
    """Measured copy bandwidth and sustained cuBLAS bf16 rate of this machine when a
    MEASURED_PEAKS.json sits at the repository root, else an earlier measurement of the same GPU type."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return dict(tensor=float(data["bf16_tflops_sustained"]), hbm=float(data["hbm_gbs"]), source="measured")
    return dict(tensor=1400.0, hbm=6650.0, source="fallback")


def _checks():
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    from oracle import checks          # the harness's checker
    return checks


# ---------------------------------------------------------------------------
# timing
# ---------------------------------------------------------------------------
def time_eager(call: Callable[[], None], launches: int, trials: int, warmup: int = 3) -> List[float]:
    """`trials` samples of the mean microseconds per call over `launches` back-to-back calls."""
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
        samples.append(start.elapsed_time(stop) * 1e3 / launches)
    return samples


def time_graph(call: Callable[[], None], operations: int, warmup_ms: float, sample_ms: float, trials: int) -> List[float]:
    """The reference's method (`benchmarks/common.py:68-111`): `operations` calls captured in one CUDA
    graph, replayed for `warmup_ms`, then `trials` samples of about `sample_ms`; microseconds per call."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(operations):
                call()
        deadline = time.perf_counter() + warmup_ms / 1e3
        graph.replay()
        torch.cuda.synchronize()
        while time.perf_counter() < deadline:
            graph.replay()
            torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def elapsed(repeats: int) -> float:
            start.record()
            for _ in range(repeats):
                graph.replay()
            stop.record()
            stop.synchronize()
            return start.elapsed_time(stop)

        repeats = max(1, math.ceil(sample_ms / max(elapsed(3) / 3, 1e-6)))
        samples = [1e3 * elapsed(repeats) / (repeats * operations) for _ in range(trials)]
    torch.cuda.current_stream().wait_stream(stream)
    return samples


# ---------------------------------------------------------------------------
# one configuration = tensors, a call, a check, a work count
# ---------------------------------------------------------------------------
class Case:
    def __init__(self, name, workload, call, check, work, unit, bound, launches=5):
        self.name, self.workload, self.call, self.check = name, workload, call, check
        self.work, self.unit, self.bound, self.launches = work, unit, bound, launches


def dense_case(name: str, config: dict, device: torch.device, operation: Optional[str], shard: int, world: int) -> Case:
    x = workloads.dense_inputs(config, device, shard=shard, rotate=mla.rope_apply)
    ins = (x["q_nope"], x["q_pe"], x["k_nope"], x["k_pe"], x["v"])
    out = torch.empty_like(x["v"])
    lse = torch.empty(config["batch"], config["heads"], config["seq"], device=device)
    backward = config["backward"] and operation != "forward"
    grads = workspace = None
    if backward:
        workspace = mla.prefill_backward_workspace(config["batch"], config["seq"], config["batch"] * config["seq"], config["heads"], device)
        grads = (torch.empty(config["batch"], config["seq"], config["heads"], 192, device=device, dtype=torch.bfloat16),
                 torch.empty_like(x["k_nope"]), torch.empty_like(x["k_pe"]), torch.empty_like(x["v"]))
    forward_in_call = operation != "backward"
    if not forward_in_call:
        mla.prefill_forward(*ins, workloads.SCALE, output=out, lse=lse)

    def call():
        if forward_in_call:
            mla.prefill_forward(*ins, workloads.SCALE, output=out, lse=lse)
        if backward:
            mla.prefill_backward(x["dout"], out, lse, *ins, workloads.SCALE, workspace=workspace, grads=grads)

    small = config["seq"] * config["heads"] <= 8192

    def check():
        checks = _checks()
        return checks.dense_full(x, out, lse, grads, workloads.SCALE) if small else checks.dense_slices(x, out, lse, grads, workloads.SCALE)

    pairs = workloads.causal_pairs(config["seq"]) * config["batch"] * config["heads"]
    flops = pairs * ((workloads.FWD_FLOP_PER_PAIR if forward_in_call else 0) + (workloads.BWD_FLOP_PER_PAIR if backward else 0))
    what = "forward + backward" if forward_in_call and backward else ("backward" if backward else "forward")
    heads = f"H={config['heads']}" + (f" per GPU (job H={config['heads'] * world})" if world > 1 else "")
    return Case(name, f"causal MLA {what}, B={config['batch']} S={config['seq']} {heads}", call, check, flops, "TFLOP/s", "tensor",
                launches=20 if flops < 1e12 else 5)


def packed_case(name: str, config: dict, device: torch.device, operation: Optional[str], shard: int, world: int) -> Case:
    lengths = workloads.varlen_lengths(config["seed"], config["sequences"], config["low"], config["high"])
    x, cu = workloads.packed_inputs(lengths, config["heads"], config["seed"], device, config["dout_std"], shard=shard, rotate=mla.rope_apply)
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

    def check():
        order = sorted(range(len(lengths)), key=lambda i: lengths[i])
        checks, result = _checks(), {}
        for label, index in (("shortest", order[0]), ("longest", order[-1])):
            for key, ok in checks.packed_slices(x, cu.cpu(), out, lse, grads, workloads.SCALE, index).items():
                result[f"{label}_{key}"] = ok
        return result

    return Case(name, f"packed causal MLA forward + backward, {len(lengths)} sequences, {total} tokens, H={config['heads']} per GPU", call, check,
                workloads.packed_flops(lengths, config["heads"]), "TFLOP/s", "tensor", launches=3)


def decode_case(name: str, config: dict, device: torch.device, operation: Optional[str], shard: int, world: int) -> Case:
    query, cache, table, lengths = workloads.decode_inputs(config["seed"], config["batch"], config["heads"], config["low"], config["high"],
                                                           config["page"])
    if world > 1:
        mine = sharding.decode_partition(lengths.tolist(), world)[shard]
        query, table, lengths = query[mine].contiguous(), table[mine].contiguous(), lengths[mine].contiguous()
    batch = query.shape[0]
    q, c, t, n = (z.to(device) for z in (query, cache, table, lengths))
    workspace = mla.decode_workspace(batch, config["heads"], config["splits"], 512, device)
    out = torch.empty(batch, 1, config["heads"], 512, device=device, dtype=torch.bfloat16)
    lse = torch.empty(batch, config["heads"], 1, device=device)

    def call():
        mla.mla_decode(q, c, t, n, workloads.SCALE, config["splits"], workspace, out, lse)

    def check():
        order = sorted(range(batch), key=lambda i: int(lengths[i]))
        return _checks().decode_sequences(query, cache, table, lengths, out, lse, workloads.SCALE, sorted({order[0], order[len(order) // 2], order[-1]}))

    moved = workloads.decode_bytes(lengths, table[:, : int(((lengths + config["page"] - 1) // config["page"]).max())], batch, config["heads"])
    return Case(name, f"absorbed paged decode, {batch} sequences, H={config['heads']}, {int(lengths.sum())} cached tokens, {config['page']}-token pages",
                call, check, moved, "GB/s", "hbm", launches=20)


BUILDERS = {"dense": dense_case, "packed": packed_case, "decode": decode_case}
OPERATIONS = {"dense": ("forward", "backward"), "packed": (), "decode": ("decode",)}


def run_cases(names: List[str], device: torch.device, args, shard: int = 0, world: int = 1) -> List[dict]:
    rows = []
    for name in names:
        config = workloads.CONFIGS[name]
        if args.operation and args.operation not in OPERATIONS[config["kind"]]:
            continue
        case = BUILDERS[config["kind"]](name, config, device, args.operation, shard, world)
        row = dict(config=name, workload=case.workload, unit=case.unit, bound=case.bound, work=case.work)
        case.call()
        torch.cuda.synchronize()
        row["checks_before"] = case.check()
        if not args.test:
            samples = (time_eager(case.call, case.launches, args.trials) if args.eager else
                       time_graph(case.call, args.graph_operations, args.warmup_ms, args.sample_ms, args.trials))
            torch.cuda.synchronize()
            row["samples_us"] = samples
            row["seconds"] = statistics.median(samples) / 1e6
            row["checks_after"] = case.check()
        if mla.device_status() != 0:
            raise RuntimeError(f"{name}: a kernel reported a device-side error status")
        rows.append(row)
        del case
        torch.cuda.empty_cache()
    return rows


def failed_checks(rows: List[dict]) -> List[str]:
    bad = []
    for row in rows:
        for stage in ("checks_before", "checks_after"):
            bad += [f"{row['config']} {stage} {key}" for key, ok in row.get(stage, {}).items() if not ok]
    return bad


def cpu_baseline_row(seconds_budget: float = 5.0) -> dict:
    """The CPU restatement on the reference's CPU-sized case (B=1, S=256, H=16, fp32, forward + backward)."""
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    from oracle import mla_oracle as oracle
    torch.set_num_threads(os.cpu_count() or 1)
    q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(0, 1, 256, 16, dtype=torch.float32)
    runs, start = 0, time.perf_counter()
    while time.perf_counter() - start < seconds_budget or runs < 3:
        out, lse = oracle.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, workloads.SCALE)
        oracle.prefill_backward(dout, out, lse, q_nope, q_pe, k_nope, k_pe, v, workloads.SCALE)
        runs += 1
    seconds = (time.perf_counter() - start) / runs
    flops = workloads.causal_pairs(256) * 16 * (workloads.FWD_FLOP_PER_PAIR + workloads.BWD_FLOP_PER_PAIR)
    return dict(tflops=flops / seconds / 1e12, cores=torch.get_num_threads(), sample="B=1 S=256 H=16 fp32 forward + backward")


def finish_rows(rows: List[dict], world: int = 1) -> List[dict]:
    top = peaks()
    for row in rows:
        peak = top["tensor"] if row["bound"] == "tensor" else top["hbm"]
        scale = 1e12 if row["unit"] == "TFLOP/s" else 1e9
        row["value"] = row["work"] / row["seconds"] / scale          # per GPU (slowest GPU's time)
        row["job_value"] = row["value"] * world if row["bound"] == "tensor" else row.get("job_work", row["work"]) / row["seconds"] / scale
        row["peak"], row["peak_source"] = peak, top["source"]
        row["fraction"] = row["value"] / peak
    return rows


def format_report(rows: List[dict], cpu: Optional[dict] = None, world: int = 1) -> str:
    header = "| config | workload | ms per call | throughput per GPU | roofline | fraction of peak |"
    rule = "|---|---|---|---|---|---|"
    if world > 1:
        header, rule = header + f" job throughput ({world} GPUs) |", rule + "---|"
    if cpu is not None:
        header, rule = header + f" CPU restatement ({cpu['cores']} cores, {cpu['sample']}) |", rule + "---|"
    lines = [header, rule]
    for row in rows:
        line = (f"| {row['config']} | {row['workload']} | {row['seconds'] * 1e3:.3f} | {row['value']:.1f} {row['unit']} | "
                f"{row['bound']} ({row['peak']:.0f} {row['unit']}, {row['peak_source']}) | {row['fraction']:.3f} |")
        if world > 1:
            line += f" {row['job_value']:.1f} {row['unit']} |"
        if cpu is not None:
            line += f" {cpu['tflops']:.3f} TFLOP/s |" if row["bound"] == "tensor" else " - |"
        lines.append(line)
    return "\n".join(lines)


def save_report(directory: pathlib.Path, rows: List[dict], report: str, method: str) -> None:
    """CSV + markdown + samples JSON with the versions, like `benchmarks/common.py:114-141`."""
    directory.mkdir(parents=True, exist_ok=True)
    fields = ["config", "workload", "seconds", "value", "unit", "bound", "peak", "peak_source", "fraction"]
    with (directory / "mla.csv").open("w", newline="") as file:
        writer = csv.DictWriter(file, fieldnames=fields, extrasaction="ignore")
        writer.writeheader()
        writer.writerows(rows)
    (directory / "mla.md").write_text("# MLA on B200: suite `b200`\n\n" + report + "\n")
    (directory / "mla_samples.json").write_text(json.dumps({
        "gpu": torch.cuda.get_device_name(), "torch": torch.__version__, "cuda": torch.version.cuda, "timing": method,
        "samples": [dict(config=row["config"], samples_us=row.get("samples_us")) for row in rows]}, indent=2) + "\n")


def _worker(rank: int, world: int, names: List[str], args, results) -> None:
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    results[rank] = [{k: v for k, v in row.items()} for row in run_cases(names, device, args, shard=rank, world=world)]


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--suite", default="b200", choices=["b200"])
    parser.add_argument("--configs", default="C1,C2,C3,C4,C5", help="comma-separated subset of C1..C5")
    parser.add_argument("--test", action="store_true", help="check every configuration against the CPU oracle; no timing")
    parser.add_argument("--operation", choices=("forward", "backward", "decode"), help="run only this operation")
    parser.add_argument("--graph-operations", type=int, default=10)
    parser.add_argument("--warmup-ms", type=int, default=1000)
    parser.add_argument("--sample-ms", type=int, default=20)
    parser.add_argument("--trials", type=int, default=9)
    parser.add_argument("--eager", action="store_true", help="time plain back-to-back launches instead of CUDA-graph replay")
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--device", type=int, default=0)
    parser.add_argument("--cpu-baseline", action="store_true", help="add a column with the CPU restatement's throughput")
    parser.add_argument("--report-dir", default=None, help="write mla.csv, mla.md and mla_samples.json here")
    parser.add_argument("--report", default=None, help="write the markdown table to this file")
    args = parser.parse_args(argv)
    names = [name.strip() for name in args.configs.split(",") if name.strip()]
    for name in names:
        if name not in workloads.CONFIGS:
            parser.error(f"unknown configuration {name}")
    if not torch.cuda.is_available():
        raise RuntimeError("the suite runs the CUDA kernels; no GPU is visible")
    if args.gpus > torch.cuda.device_count():
        parser.error(f"--gpus {args.gpus} but {torch.cuda.device_count()} visible")
    if args.gpus == 1:
        device = torch.device("cuda", args.device)
        torch.cuda.set_device(device)
        rows = run_cases(names, device, args)
    else:
        import torch.multiprocessing as mp
        manager = mp.Manager()
        results = manager.dict()
        mp.spawn(_worker, args=(args.gpus, names, args, results), nprocs=args.gpus, join=True)
        rows = [dict(row) for row in results[0]]
        for index, row in enumerate(rows):
            others = [results[r][index] for r in range(args.gpus)]
            if not args.test:
                row["seconds"] = max(o["seconds"] for o in others)          # the slowest GPU
            row["job_work"] = sum(o["work"] for o in others)
            for stage in ("checks_before", "checks_after"):
                if stage in row:
                    row[stage] = {f"gpu{r}_{k}": ok for r, o in enumerate(others) for k, ok in o[stage].items()}
    bad = failed_checks(rows)
    if bad:
        raise AssertionError("oracle checks failed: " + ", ".join(bad))
    count = sum(len(row["checks_before"]) for row in rows)
    if args.test:
        print(f"mla: {count} correctness checks passed")
        return 0
    cpu = cpu_baseline_row() if args.cpu_baseline else None
    report = format_report(finish_rows(rows, args.gpus), cpu, args.gpus)
    print(report)
    method = ("plain back-to-back launches; median microseconds" if args.eager else
              f"CUDA Graph replay of {args.graph_operations} captured calls; warmup and preparation excluded; median microseconds")
    if args.report:
        pathlib.Path(args.report).write_text("# MLA on B200: suite `b200`\n\n" + report + "\n")
    if args.report_dir:
        save_report(pathlib.Path(args.report_dir), rows, report, method)
    return 0


if __name__ == "__main__":
    sys.exit(main())
