"""Nsight Compute flow for the MLA kernels: run the launchers under ncu, then summarise.

    python -m dscuda_b200.profile mla [quick|full] [profile|extract|print] [--out-dir DIR] [--profiles-dir profiles]

Counterpart of the reference's `scripts/profile.sh mla` (`profile_mla`, scripts/profile.sh:281-296:
benchmark_mla at T in {128, 256, 512} with H=8 and benchmark_mla_decode at B=2, H=16, each profiled
twice, then `scripts/extract_ncu.py`).  Here every case is:

  1. the plain command (it must exit 0 before anything is profiled);
  2. the launch list: `ncu --metrics gpu__time_duration.sum` (one pass per launch);
  3. a counter capture of at most three launches of each kernel of the case: DRAM bytes read and
     written, DRAM throughput, tensor-pipe activity, issue slots, warps, registers, shared memory;
  4. `dscuda_b200.ncu_extract` on both outputs -> `<profiles-dir>/<case>_launches.md`,
     `<profiles-dir>/<case>_counters.md`, and for the training case `<profiles-dir>/traffic.json`.

Every ncu command carries `--clock-control none` (clocks are never touched) and
`--profile-from-start off` (the launchers bracket one call with cudaProfilerStart/Stop, so warm-up
launches are not captured).  The cases are small by design: a counter capture replays each launch
several times and saves and restores device memory around the passes.

Modes: `profile` runs everything (needs a B200 and ncu), `extract` only re-reads the reports in
--out-dir, `print` lists the commands without running them.
"""
from __future__ import annotations

import argparse
import pathlib
import shlex
import shutil
import subprocess
import sys
from typing import List

from . import ncu_extract

ROOT = pathlib.Path(__file__).resolve().parents[1]
BUILD = ROOT / "build"

COUNTERS = ",".join((
    "gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
    "smsp__issue_active.avg.pct_of_peak_sustained_active",
    "sm__warps_active.avg.pct_of_peak_sustained_active",
    "launch__registers_per_thread", "launch__shared_mem_per_block_dynamic", "launch__grid_size", "launch__block_size",
    "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio",
))


def cases(suite: str) -> List[dict]:
    """name, launcher command, kernel-name pattern, and (for the traffic file) work units per launch."""
    result = []
    sequences = (128,) if suite == "quick" else (128, 256, 512)
    for t in sequences:             # the reference's own sizes (scripts/profile.sh:282-290)
        result.append(dict(name=f"absorbed_T{t}_H8", command=[str(BUILD / "benchmark_mla"), "1", str(t), "8", "512", "64"],
                           pattern="regex:absorbed_(attention|backward_query|backward_key|backward_reduce|delta)_kernel"))
        result.append(dict(name=f"decode_KV{t}_H16", command=[str(BUILD / "benchmark_mla_decode"), "2", str(t), "16", "512", "64", "8"],
                           pattern="regex:(absorbed_decode|decode_combine)_kernel"))
    # B200-sized cases: inputs larger than the 126 MB L2, a few GB at most
    result.append(dict(name="absorbed_T2048_H16_B4", command=[str(BUILD / "benchmark_mla"), "4", "2048", "16", "512", "64"],
                       pattern="regex:absorbed_(attention|backward_query|backward_key|backward_reduce|delta)_kernel"))
    result.append(dict(name="decode_KV16384_H128_B16", command=[str(BUILD / "benchmark_mla_decode"), "16", "16384", "128", "512", "64", "8"],
                       pattern="regex:(absorbed_decode|decode_combine)_kernel"))
    # the training step at the benchmark's sequence length (the dS^T scratch grows with its square), 8 heads
    result.append(dict(name="train_S8192_H8", command=[str(BUILD / "benchmark_mla_prefill"), "1", "8192", "8", "1"],
                       pattern="regex:(attention_forward|backward_dq_stream|backward_dq|backward_dkdv)_kernel", traffic_key="train_step", units=8192 * 8,
                       unit_name="token_head"))
    return result


def commands(case: dict, out_dir: pathlib.Path, ncu: str):
    launches = out_dir / f"{case['name']}_launches.csv"
    report = out_dir / f"{case['name']}_counters"
    common = [ncu, "--clock-control", "none", "--profile-from-start", "off"]
    list_cmd = common + ["--metrics", "gpu__time_duration.sum", "--csv", "--log-file", str(launches)] + case["command"]
    count_cmd = common + ["--metrics", COUNTERS, "-k", case["pattern"], "-c", "12", "-f", "-o", str(report)] + case["command"]
    return launches, report.with_suffix(".ncu-rep"), list_cmd, count_cmd


def run(command: List[str], log: pathlib.Path) -> None:
    done = subprocess.run(command, capture_output=True, text=True)
    log.write_text(done.stdout + done.stderr)
    if done.returncode != 0:
        raise RuntimeError(f"{shlex.join(command)} exited {done.returncode}; see {log}")


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("family", choices=("mla",))
    parser.add_argument("suite", nargs="?", default="quick", choices=("quick", "full"))
    parser.add_argument("mode", nargs="?", default="profile", choices=("profile", "extract", "print"))
    parser.add_argument("--out-dir", type=pathlib.Path, default=ROOT / "gpurun_out", help="raw ncu output (reports, CSV, logs)")
    parser.add_argument("--profiles-dir", type=pathlib.Path, default=ROOT / "profiles", help="markdown summaries and traffic.json")
    parser.add_argument("--only", help="comma-separated case names")
    args = parser.parse_args(argv)
    ncu = shutil.which("ncu") or "/usr/local/cuda/bin/ncu"
    selected = [case for case in cases(args.suite) if not args.only or case["name"] in args.only.split(",")]
    args.out_dir.mkdir(parents=True, exist_ok=True)
    args.profiles_dir.mkdir(parents=True, exist_ok=True)
    for case in selected:
        launches, report, list_cmd, count_cmd = commands(case, args.out_dir, ncu)
        if args.mode == "print":
            print(shlex.join(case["command"]), "&&", shlex.join(list_cmd), "&&", shlex.join(count_cmd))
            continue
        if args.mode == "profile":
            run(case["command"], args.out_dir / f"{case['name']}_plain.log")          # must exit 0 before ncu sees it
            run(list_cmd, args.out_dir / f"{case['name']}_launches.log")
            run(count_cmd, args.out_dir / f"{case['name']}_counters.log")
        relative = [c.replace(str(ROOT) + "/", "") for c in list_cmd]
        ncu_extract.main(["launches", str(launches), "--title", f"Launch list: {case['name']}", "--command", shlex.join(relative),
                          "--out", str(args.profiles_dir / f"{case['name']}_launches.md")])
        relative = [c.replace(str(ROOT) + "/", "") for c in count_cmd]
        extract = ["counters", str(report), "--title", f"Counters: {case['name']}", "--command", shlex.join(relative),
                   "--out", str(args.profiles_dir / f"{case['name']}_counters.md")]
        if "traffic_key" in case:
            extract += ["--traffic-json", str(args.profiles_dir / "traffic.json"), "--traffic-key", case["traffic_key"], "--units", str(case["units"]),
                        "--unit-name", case["unit_name"]]
        ncu_extract.main(extract)
    return 0


if __name__ == "__main__":
    sys.exit(main())
