"""Turns Nsight Compute output for the MLA kernels into the tables under `profiles/`.

    python -m dscuda_b200.ncu_extract launches LAUNCHES.csv [--title T] [--command C] [--out profiles/x.md]
    python -m dscuda_b200.ncu_extract counters REPORT.ncu-rep|RAW.csv [--units N --unit-name NAME]
                                      [--title T] [--command C] [--out profiles/y.md]
                                      [--traffic-json profiles/traffic.json --traffic-key KEY]

It is the counterpart of the reference's `scripts/extract_ncu.py`: `short_kernel_name` maps a
demangled kernel name to a short label (there: lines 91-116, for the sm_89/sm_90 kernels; here: the
sm_100a kernels of this library), and rows of several reports are merged per label (there: lines
186-247).  Two kinds of input:

* `launches`: the CSV that `ncu --metrics gpu__time_duration.sum --csv --log-file F <command>` writes
  (one row per launch and metric).  Output: per kernel its launches, total time and share.  Per-launch
  times under ncu are cold-cache and serialised, so the share is what the table is for.
* `counters`: a `.ncu-rep` (read through `ncu -i F --page raw --csv`; needs `ncu` on PATH, no GPU) or
  that raw CSV saved to a file.  Output: per kernel duration, DRAM bytes read + written, DRAM
  throughput %, tensor-pipe active %, issue-slot %, registers, shared memory.  With `--traffic-json`
  the DRAM bytes per launch (and per `--units` when given) are stored under `--traffic-key`;
  `bench.py` reads that file for its `roofline.traffic` figure.

Nothing here needs a GPU.
"""
from __future__ import annotations

import argparse
import csv
import io
import json
import pathlib
import re
import shutil
import subprocess
import sys
from typing import Dict, Iterable, List, Optional

# (regular expression on the demangled name, short label).  First match wins.
KERNEL_PATTERNS = (
    (r"attention_forward_kernel<\(?int\)?3>|attention_forward_kernel<3>", "prefill_fwd"),
    (r"attention_forward_kernel<\(?int\)?2>|attention_forward_kernel<2>", "flash_fwd"),
    (r"attention_forward_kernel", "prefill_fwd"),
    (r"backward_dq_stream_kernel", "prefill_bwd_dq_stream"),
    (r"backward_dq_kernel", "prefill_bwd_dq"),
    (r"backward_dkdv_kernel", "prefill_bwd_dkdv"),
    (r"absorbed_delta_kernel", "absorbed_delta"),
    (r"sum_dk_pe_kernel", "dk_pe_sum"),
    (r"(?<!absorbed_)delta_kernel", "prefill_delta"),
    (r"absorbed_attention_kernel", "absorbed_fwd"),
    (r"absorbed_decode_kernel", "absorbed_decode"),
    (r"cache_dequantize_fp8_kernel", "cache_dequantize_fp8"),
    (r"decode_combine_kernel", "decode_combine"),
    (r"absorbed_backward_query_kernel", "absorbed_bwd_query"),
    (r"absorbed_backward_key_kernel", "absorbed_bwd_key"),
    (r"absorbed_backward_reduce_kernel", "absorbed_bwd_reduce"),
    (r"cache_append_fp8_kernel", "cache_append_fp8"),
    (r"cache_append_kernel", "cache_append"),
    (r"rope_apply_kernel", "rope_apply"),
    (r"projection_gemm_kernel", "projection_gemm"),
)
OTHER = "(other kernels)"

# raw-page column -> (field, scale to the field's unit by ncu unit)
BYTE_UNITS = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}
TIME_UNITS_US = {"ns": 1e-3, "nsecond": 1e-3, "us": 1.0, "usecond": 1.0, "ms": 1e3, "msecond": 1e3, "s": 1e6, "second": 1e6}
COUNTER_COLUMNS = {
    "gpu__time_duration.sum": "time_us",
    "dram__bytes_read.sum": "dram_read_bytes",
    "dram__bytes_write.sum": "dram_write_bytes",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed": "dram_pct",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active": "tensor_pct",
    "smsp__issue_active.avg.pct_of_peak_sustained_active": "issue_pct",
    "sm__warps_active.avg.pct_of_peak_sustained_active": "warps_pct",
    "launch__registers_per_thread": "registers",
    "launch__shared_mem_per_block_dynamic": "dynamic_smem_bytes",
    "launch__grid_size": "grid",
    "launch__block_size": "block",
    "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio": "stall_long_scoreboard",
}


def short_kernel_name(full_name: str) -> str:
    """Short label of one of this library's kernels, `OTHER` for anything else (torch, NCCL)."""
    for pattern, label in KERNEL_PATTERNS:
        if re.search(pattern, full_name):
            return label
    return OTHER


def _number(text: str) -> float:
    try:
        return float(text.replace(",", ""))
    except ValueError:
        return float("nan")


def _skip_banner(text: str) -> str:
    """ncu writes ==PROF== lines before the CSV header."""
    lines = text.splitlines()
    for index, line in enumerate(lines):
        if line.startswith('"ID"'):
            return "\n".join(lines[index:])
    raise ValueError("no CSV header (\"ID\",...) found in the ncu output")


# ---------------------------------------------------------------------------
# launch list
# ---------------------------------------------------------------------------
def read_launches(text: str) -> List[dict]:
    """Rows of `ncu --csv --metrics gpu__time_duration.sum`: one dict per launch (label, name, time_us)."""
    launches: Dict[str, dict] = {}
    for row in csv.DictReader(io.StringIO(_skip_banner(text))):
        if row.get("Metric Name") != "gpu__time_duration.sum":
            continue
        scale = TIME_UNITS_US.get(row.get("Metric Unit", "ns"), 1e-3)
        launches[row["ID"]] = dict(label=short_kernel_name(row["Kernel Name"]), name=row["Kernel Name"],
                                   time_us=_number(row["Metric Value"]) * scale)
    return [launches[key] for key in sorted(launches, key=int)]


def merge_by_label(rows: Iterable[dict], sum_fields=("time_us",), mean_fields=()) -> List[dict]:
    """One row per label: launches counted, `sum_fields` added, `mean_fields` averaged weighted by time."""
    merged: Dict[str, dict] = {}
    for row in rows:
        target = merged.setdefault(row["label"], dict(label=row["label"], launches=0, **{f: 0.0 for f in sum_fields},
                                                      **{f: 0.0 for f in mean_fields}, _weight=0.0))
        target["launches"] += 1
        for field in sum_fields:
            target[field] += row.get(field, 0.0)
        weight = row.get("time_us", 1.0)
        for field in mean_fields:
            target[field] += row.get(field, 0.0) * weight
        target["_weight"] += weight
    result = []
    for target in merged.values():
        for field in mean_fields:
            target[field] = target[field] / target["_weight"] if target["_weight"] else float("nan")
        del target["_weight"]
        result.append(target)
    return sorted(result, key=lambda r: -r["time_us"])


def launch_table(launches: List[dict]) -> str:
    rows = merge_by_label(launches)
    total = sum(row["time_us"] for row in rows) or 1.0
    lines = ["| kernel | launches | total ms | ms / launch | share |", "|---|---|---|---|---|"]
    for row in rows:
        lines.append(f"| `{row['label']}` | {row['launches']} | {row['time_us'] / 1e3:.2f} | {row['time_us'] / 1e3 / row['launches']:.3f} | "
                     f"{100 * row['time_us'] / total:.1f} % |")
    return "\n".join(lines)


# ---------------------------------------------------------------------------
# counters (raw page)
# ---------------------------------------------------------------------------
def raw_page(path: pathlib.Path) -> str:
    if path.suffix == ".ncu-rep":
        ncu = shutil.which("ncu") or "/usr/local/cuda/bin/ncu"
        done = subprocess.run([ncu, "-i", str(path), "--page", "raw", "--csv"], capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"ncu could not read {path}: {done.stderr[-500:]}")
        return done.stdout
    return path.read_text()


def read_counters(text: str) -> List[dict]:
    """Rows of the raw page: header line, unit line, then one line per captured launch."""
    rows = list(csv.reader(io.StringIO(_skip_banner(text))))
    header, units = rows[0], rows[1]
    name_column = header.index("Kernel Name")
    result = []
    for line in rows[2:]:
        if len(line) != len(header):
            continue
        entry = dict(label=short_kernel_name(line[name_column]), name=line[name_column])
        for index, column in enumerate(header):
            field = COUNTER_COLUMNS.get(column)
            if field is None:
                continue
            value = _number(line[index])
            if field == "time_us":
                value *= TIME_UNITS_US.get(units[index], 1e-3)
            elif field.endswith("_bytes"):
                value *= BYTE_UNITS.get(units[index].split("/")[0], 1.0)        # "Kbyte/block" -> "Kbyte"
            entry[field] = value
        result.append(entry)
    return result


def counter_table(captures: List[dict]) -> str:
    sums = ("time_us", "dram_read_bytes", "dram_write_bytes")
    means = ("dram_pct", "tensor_pct", "issue_pct", "registers", "dynamic_smem_bytes")
    for row in captures:
        for field in sums + means:
            row.setdefault(field, float("nan"))
    rows = merge_by_label(captures, sums, means)
    lines = ["| kernel | captured launches | us / launch | DRAM read MB / launch | DRAM written MB / launch | DRAM % of peak | tensor pipe active % | "
             "issue slots % | registers | dynamic smem KB |", "|---|---|---|---|---|---|---|---|---|---|"]
    for row in rows:
        n = row["launches"]
        lines.append(f"| `{row['label']}` | {n} | {row['time_us'] / n:.1f} | {row['dram_read_bytes'] / n / 1e6:.2f} | "
                     f"{row['dram_write_bytes'] / n / 1e6:.2f} | {row['dram_pct']:.1f} | {row['tensor_pct']:.1f} | {row['issue_pct']:.1f} | "
                     f"{row['registers']:.0f} | {row['dynamic_smem_bytes'] / 1024:.0f} |")
    return "\n".join(lines)


def traffic_entry(captures: List[dict], units: Optional[float], unit_name: str) -> dict:
    """DRAM bytes (read + written) per launch, per label, and per work unit when `units` is given."""
    entry = {}
    for row in merge_by_label(captures, ("time_us", "dram_read_bytes", "dram_write_bytes")):
        per_launch = (row["dram_read_bytes"] + row["dram_write_bytes"]) / row["launches"]
        item = dict(dram_bytes_per_launch=per_launch, captured_launches=row["launches"])
        if units:
            item[f"dram_bytes_per_{unit_name}"] = per_launch / units
            item["units_per_launch"] = units
        entry[row["label"]] = item
    return entry


def update_traffic_json(path: pathlib.Path, key: str, entry: dict, source: str) -> None:
    data = json.loads(path.read_text()) if path.exists() else {}
    data[key] = dict(kernels=entry, source=source)
    path.write_text(json.dumps(data, indent=1, sort_keys=True) + "\n")


def _document(title: str, command: str, note: str, table: str) -> str:
    parts = [f"# {title}", ""]
    if command:
        parts += ["Command (on a B200, after the same command exited 0 without ncu):", "", "```", command, "```", ""]
    if note:
        parts += [note, ""]
    parts += [table, ""]
    return "\n".join(parts)


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("mode", choices=("launches", "counters"))
    parser.add_argument("input", type=pathlib.Path)
    parser.add_argument("--title", default="ncu summary")
    parser.add_argument("--command", default="", help="the full command that produced the input (recorded in the summary)")
    parser.add_argument("--out", type=pathlib.Path, help="write the markdown summary here (default: stdout only)")
    parser.add_argument("--units", type=float, help="work units one captured launch processes (for per-unit traffic)")
    parser.add_argument("--unit-name", default="unit")
    parser.add_argument("--traffic-json", type=pathlib.Path)
    parser.add_argument("--traffic-key")
    args = parser.parse_args(argv)
    if args.mode == "launches":
        table = launch_table(read_launches(args.input.read_text()))
        note = "Per-launch times under ncu are cold-cache and serialised: compare shares, not absolutes."
    else:
        captures = read_counters(raw_page(args.input))
        table = counter_table(captures)
        note = "Counters of the captured launches (reduced size; see the command)."
        if args.traffic_json:
            if not args.traffic_key:
                parser.error("--traffic-json needs --traffic-key")
            update_traffic_json(args.traffic_json, args.traffic_key, traffic_entry(captures, args.units, args.unit_name), args.command)
    document = _document(args.title, args.command, note, table)
    print(document)
    if args.out:
        args.out.write_text(document)
    return 0


if __name__ == "__main__":
    sys.exit(main())
