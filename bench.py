"""Throughput of the MLA path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload train|prefill]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path over one
batch of seeded synthetic input:

* `train`   - causal MLA forward + backward, B=2, S=8192, H=128 per GPU, bf16
              (q/k/v ~ N(0,1), dO ~ N(0,0.1));
* `prefill` - causal MLA forward only, B=4, S=4096, H=128 per GPU.

`value` is TFLOP/s counted on the algorithmic work (640 FLOP per causal
(query,key) pair and head forward, 1664 backward), whole job, inputs resident in
HBM.  `e2e` is the same metric through the host-buffer API: pinned host inputs
copied to the device and the result read back inside the timed region.  The
`decode` object reports the absorbed paged decode (batch 64, lengths uniform in
[1024, 32768], 64-token pages, permuted page table) in GB/s of algorithmic
bytes.  There is no collective on the data path, and the job value is the sum
over ranks divided by the slowest rank's time.

With N > 1 GPUs the job is the head-sharded one: every rank owns its own 128 heads of an
H = 128*N job (its own draws; the shared rotary key is the same everywhere), the decode
benchmark's 64 sequences are dealt to the ranks by cache pages (with as many partial slots per
sequence as `mla.decode_splits` asks for that share), the packed long-context case
runs 16 heads per GPU, and a small head-sharded problem is gathered over NCCL and compared with
the CPU oracle on rank 0.  After the timed regions rank 0 also compares slices of the timed
outputs themselves with the oracle; the line carries the outcome as `verified`.

`--impl reference` times the CPU oracle port of the reference's
reference/python/mla.py on the host cores, on a bounded sample of the workload.
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import sys
import threading
import time

import torch

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from dscuda_b200 import workloads
from dscuda_b200.workloads import BWD_FLOP_PER_PAIR, FWD_FLOP_PER_PAIR, SCALE, causal_pairs

WORKLOADS = {"train": workloads.CONFIGS["C3"], "prefill": workloads.CONFIGS["C2"]}


def dram_traffic(kind: str, token_heads: int):
    """DRAM bytes (read + written) per launch of the dominant call, from the committed ncu capture
    summarised in profiles/traffic.json (written by `python -m dscuda_b200.ncu_extract counters ...
    --traffic-json`): bytes per (token, head) of the reduced-size capture (same sequence length, fewer
    heads) times the (token, head) pairs of this run; at a fixed sequence length the traffic grows in
    proportion to them.  None when the file has no entry."""
    path = ROOT / "profiles" / "traffic.json"
    if not path.exists():
        return None, None
    entry = json.loads(path.read_text()).get("train_step")
    if not entry:
        return None, None
    labels = ("prefill_bwd_dq_stream", "prefill_bwd_dkdv") if kind == "backward" else ("prefill_fwd",)
    try:
        per_unit = sum(entry["kernels"][label]["dram_bytes_per_token_head"] for label in labels)
    except KeyError:
        return None, None
    return per_unit * token_heads, "profiles/traffic.json (train_step): ncu capture at S=8192 with 8 heads, scaled by (token, head) pairs"


workload_flops = workloads.dense_flops


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return dict(tensor=float(data["bf16_tflops_sustained"]), tensor_burst=float(data["bf16_tflops"]),
                    hbm=float(data["hbm_gbs"]), source="measured")
    return dict(tensor=1400.0, tensor_burst=1590.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only) while the timed region runs."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index):
        self.index = index
        self.clocks, self.masks, self.max_clock = [], 0, None
        self.stop = threading.Event()
        self.thread = threading.Thread(target=self.run, daemon=True)

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_clock = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            while not self.stop.is_set():
                self.clocks.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                self.masks |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                self.stop.wait(0.01)
        except Exception as error:           # reported, never fatal: the clocks are evidence, not the measurement
            self.error = repr(error)

    def __enter__(self):
        self.thread.start()
        time.sleep(0.05)
        return self

    def __exit__(self, *exc):
        self.stop.set()
        self.thread.join(timeout=10)

    def summary(self):
        if not self.clocks:
            return dict(sm_mhz=None, sm_max_mhz=self.max_clock, reasons=[], samples=0, error=getattr(self, "error", None))
        reasons = [name for name, bit in self.REASONS.items() if self.masks & bit]
        return dict(sm_mhz=statistics.median(self.clocks), sm_min_mhz=min(self.clocks), sm_max_mhz=self.max_clock,
                    reasons=reasons, samples=len(self.clocks))


def time_steps(step, steps, warmup, barrier):
    for _ in range(warmup):
        step()
    barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    stop.synchronize()
    barrier()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / 1e3


def bind_to_gpu_numa_node(index):
    """Keeps this process (and the pinned buffers it allocates afterwards) on the CPU cores of the
    NUMA node its GPU hangs off.  CPU affinity of this process only; nothing on the GPU changes."""
    try:
        import pynvml
        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        physical = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(physical)).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        bus = bus.lower()
        if len(bus.split(":")[0]) == 8:                      # NVML pads the domain to eight digits, sysfs uses four
            bus = bus[4:]
        node = int(pathlib.Path(f"/sys/bus/pci/devices/{bus}/numa_node").read_text())
        if node < 0:
            return {"node": None, "bound": False}
        cpus = set()
        for piece in pathlib.Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
            low, _, high = piece.partition("-")
            cpus.update(range(int(low), int(high or low) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
        return {"node": node, "bound": bool(allowed), "cpus": len(allowed)}
    except Exception as error:                                   # evidence, never fatal
        return {"node": None, "bound": False, "error": repr(error)[:120]}


def verify_training(checks, w, x, out, lse, grads):
    """Slices of the timed step's own outputs against the CPU oracle (oracle/checks.py): batch 0,
    head 0, the last 256 query rows (O, LSE, dQ) and the first 128 keys (dK_nope, dV); dK_pe (summed
    over this GPU's heads) on the first 32 keys."""
    return checks.dense_slices(x, out, lse, grads if w["backward"] else None, SCALE)


def verify_sharded(mla, oracle, sharding, rank, world, device):
    """A small head-sharded problem over NCCL (B=1, S=1024, two heads per rank): every rank computes
    its own heads, O / LSE / dQ / dK_nope / dV are all-gathered, the fp32 dK_pe partial sums are
    added, and rank 0 compares the assembled result with the CPU oracle on the unsharded problem."""
    heads, seq = 2 * world, 1024
    q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(11, 1, seq, heads, dout_std=0.1)
    start, stop = sharding.head_range(heads, world, rank)
    mine = [t[:, :, start:stop].contiguous().to(device) for t in (q_nope, q_pe, k_nope)] + [k_pe.to(device), v[:, :, start:stop].contiguous().to(device)]
    out, lse = mla.prefill_forward(*mine, SCALE)
    workspace = mla.prefill_backward_workspace(1, seq, seq, stop - start, device)
    grads = mla.prefill_backward(dout[:, :, start:stop].contiguous().to(device), out, lse, *mine, SCALE, workspace=workspace)
    partial = workspace[: seq * 64 * 4].view(torch.float32).reshape(1, seq, 1, 64).clone()
    full_out = sharding.gather_heads(out, heads, 2)
    full_lse = sharding.gather_heads(lse, heads, 1)
    full = [sharding.gather_heads(grads[i], heads, 2) for i in (0, 1, 3)]
    dk_pe = sharding.sum_dk_pe_partials(partial)
    torch.cuda.synchronize()
    if rank != 0:
        return None
    ref_out, ref_lse = oracle.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, SCALE)
    ref = oracle.prefill_backward(dout, full_out.cpu(), full_lse.cpu(), q_nope, q_pe, k_nope, k_pe, v, SCALE)

    def rel(got, want):
        return float((got.double().cpu() - want.double()).norm() / want.double().norm())

    return {"out": float((full_out.float().cpu() - ref_out).abs().max()) <= 1e-2 * float(ref_out.abs().max()),
            "lse": float((full_lse.cpu() - ref_lse).abs().max()) <= 1e-3,
            "dq": rel(full[0].float(), ref[0]) <= 1e-2, "dk_nope": rel(full[1].float(), ref[1]) <= 1e-2,
            "dk_pe_sum_over_ranks": rel(dk_pe, ref[2]) <= 1e-2, "dv": rel(full[2].float(), ref[3]) <= 1e-2}


def run_ours(args, rank, world, device):
    from dscuda_b200 import mla, sharding
    from oracle import checks, mla_oracle as oracle  # checker (verification) and the cpu_baseline leg only

    w = dict(WORKLOADS[args.workload])
    for key in ("batch", "seq", "heads"):
        if getattr(args, key) is not None:          # reduced sizes for profiler captures; the line names them
            w[key] = getattr(args, key)
    peaks = measured_peaks()
    if world > 1:
        import torch.distributed as dist
        barrier = dist.barrier

        def reduce_max(values):
            t = torch.tensor(values, device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return [float(v) for v in t]

        def reduce_sum(values):
            t = torch.tensor(values, device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            return [float(v) for v in t]
    else:
        def barrier():
            return None

        def reduce_max(values):
            return list(values)

        reduce_sum = reduce_max
    if args.only_decode:
        decode = bench_decode(mla, checks, sharding, device, peaks, rank, world, barrier, reduce_max, reduce_sum, steps=args.steps,
                              warmup=args.warmup, batch=args.decode_batch)
        return {"metric": decode["metric"], "value": decode["value"], "unit": decode["unit"], "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": decode["us_per_step"] / 1e3, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"decode only: batch {args.decode_batch}, heads 128, lengths uniform in [1024, 32768], seed 3"},
                "gpu_launches": 2 * args.steps, "roofline": decode["roofline"], "decode": decode} if rank == 0 else None
    numa = bind_to_gpu_numa_node(device.index)
    x = workloads.dense_inputs(w, device, shard=rank, rotate=mla.rope_apply)
    fwd_in = (x["q_nope"], x["q_pe"], x["k_nope"], x["k_pe"], x["v"])
    out = torch.empty_like(x["v"])
    lse = torch.empty(w["batch"], w["heads"], w["seq"], device=device)
    launches = 1
    grads = None
    if w["backward"]:
        workspace = mla.prefill_backward_workspace(w["batch"], w["seq"], w["batch"] * w["seq"], w["heads"], device)
        grads = (torch.empty(w["batch"], w["seq"], w["heads"], 192, device=device, dtype=torch.bfloat16),
                 torch.empty_like(x["k_nope"]), torch.empty_like(x["k_pe"]), torch.empty_like(x["v"]))
        launches += mla.prefill_backward_launches(w["batch"], w["seq"], w["batch"] * w["seq"], w["heads"])

    def forward():
        mla.prefill_forward(*fwd_in, SCALE, output=out, lse=lse)

    def backward():
        mla.prefill_backward(x["dout"], out, lse, *fwd_in, SCALE, workspace=workspace, grads=grads)

    def step():
        forward()
        if w["backward"]:
            backward()

    with ClockSampler(device.index) as sampler:
        seconds = time_steps(step, args.steps, args.warmup, barrier)
    clocks = sampler.summary()
    assert mla.device_status() == 0, "a kernel reported a bounded-wait timeout"
    verified = {"train_step_slices": verify_training(checks, w, x, out, lse, grads)} if rank == 0 and not args.skip_verify else {}

    # dominant call timed alone (same stream, CUDA events) for the roofline object
    dominant = backward if w["backward"] else forward
    dominant_seconds = time_steps(dominant, max(2, args.steps), 1, lambda: None) / max(2, args.steps)
    dominant_flops = causal_pairs(w["seq"]) * w["batch"] * w["heads"] * (BWD_FLOP_PER_PAIR if w["backward"] else FWD_FLOP_PER_PAIR)

    # end to end: pinned host inputs -> device -> kernels -> result back to the host, every step.
    # The copy of step i+1 overlaps the kernels of step i (two staging sets, one copy stream).
    from dscuda_b200.host_pipeline import HostPipeline
    host = {k: torch.empty(v.shape, dtype=v.dtype, pin_memory=True).copy_(v) for k, v in x.items()}
    result_host = torch.empty(lse.shape, dtype=lse.dtype, pin_memory=True)
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = result_host.numel() * result_host.element_size()

    def e2e_run(steps, compute=True):
        pipe = HostPipeline(x, device)
        pipe.stage(host)
        for i in range(steps):
            if i + 1 < steps:
                pipe.stage(host)
            staged = pipe.acquire()
            if compute:
                ins = (staged["q_nope"], staged["q_pe"], staged["k_nope"], staged["k_pe"], staged["v"])
                mla.prefill_forward(*ins, SCALE, output=out, lse=lse)
                if w["backward"]:
                    mla.prefill_backward(staged["dout"], out, lse, *ins, SCALE, workspace=workspace, grads=grads)
                result_host.copy_(lse, non_blocking=True)
            pipe.release()

    def timed(function, steps):
        barrier()
        torch.cuda.synchronize()
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record()
        function(steps)                              # every copy is enqueued after `first` and finishes before `last`
        last.record()
        last.synchronize()
        barrier()
        torch.cuda.synchronize()
        return first.elapsed_time(last) / 1e3

    e2e_steps = max(2, min(args.steps, 8))
    e2e_run(2)                                       # warm-up
    e2e_seconds = timed(e2e_run, e2e_steps)
    # the host link alone, all ranks at once: the ceiling of any pipeline that feeds every step from the host
    copy_seconds = timed(lambda steps: e2e_run(steps, compute=False), e2e_steps)

    flops = workload_flops(w)
    seconds, e2e_seconds, copy_seconds = reduce_max([seconds, e2e_seconds, copy_seconds])
    del host

    prefill = None
    if w["backward"] and not args.skip_decode:
        del x, out, lse, grads, workspace
        torch.cuda.empty_cache()
        prefill = bench_prefill(mla, checks, device, peaks, rank, barrier, reduce_max, verify=rank == 0 and not args.skip_verify)
    decode = bench_decode(mla, checks, sharding, device, peaks, rank, world, barrier, reduce_max, reduce_sum) if not args.skip_decode else None
    varlen = bench_varlen(mla, device, peaks, rank, world, barrier, reduce_max) if not args.skip_decode else None
    append = bench_cache_append(mla, device, peaks) if world == 1 and not args.skip_decode else None
    rope = bench_rope(mla, device, peaks) if world == 1 and not args.skip_decode else None
    projection = bench_projection(mla, device, peaks) if world == 1 and not args.skip_decode else None
    absorbed = bench_absorbed(mla, device, peaks) if world == 1 and not args.skip_decode else None
    flash = bench_flash(mla, device, peaks) if world == 1 and not args.skip_decode else None
    cpu = cpu_baseline(oracle, 12.0) if world == 1 and not args.skip_cpu else None
    if world > 1 and not args.skip_verify:
        verified["head_sharded_over_nccl"] = verify_sharded(mla, oracle, sharding, rank, world, device)
    assert mla.device_status() == 0, "a kernel reported a device-side error status"

    if rank != 0:
        return None
    if decode is not None and "verified" in decode:
        verified["decode"] = decode.pop("verified")
    if prefill is not None and "verified" in prefill:
        verified["prefill"] = prefill.pop("verified")
    value = flops * world * args.steps / seconds / 1e12
    achieved = dominant_flops / dominant_seconds / 1e12
    traffic, traffic_source = dram_traffic("backward" if w["backward"] else "forward", w["batch"] * w["seq"] * w["heads"])
    e2e_value = flops * world * e2e_steps / e2e_seconds / 1e12
    ceiling_value = flops * world * e2e_steps / copy_seconds / 1e12
    all_checks = [ok for group in verified.values() if group for ok in group.values()]
    line = {
        "metric": "MLA fwd+bwd TFLOP/s (bf16 causal)" if w["backward"] else "MLA prefill fwd TFLOP/s (bf16 causal)",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload}: causal non-absorbed MLA, B={w['batch']} S={w['seq']} H={w['heads']} per GPU, "
                               f"qk=128+64 (shared k_pe), v=128, seed {w['seed']}",
                   "per_gpu_tflops": value / world,
                   "sharding": f"rank r owns heads 128r..128r+127 of the H={128 * world} job (own draws, shared k_pe); no collective on the data path",
                   "l2": "inputs (>= 1.9 GB per step) exceed the 126 MB L2; no flush needed"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "h2d_gbs_per_rank": h2d * e2e_steps / e2e_seconds / 1e9,
                "host_link_ceiling": {"value": ceiling_value, "unit": "TFLOP/s", "h2d_gbs_per_rank": h2d * e2e_steps / copy_seconds / 1e9,
                                      "how": "the same staged copies with no kernels, all ranks at once"},
                "fraction_of_ceiling": e2e_value / ceiling_value, "numa": numa},
        "gpu_launches": launches * args.steps,
        "verified": bool(all_checks) and all(all_checks), "verified_checks": verified,
        "roofline": {"bound": "tensor", "kernel": "prefill backward (dK/dV kernel, then dQ streamed from the stored dS)" if w["backward"] else "attention_forward_kernel<3>",
                     "achieved": achieved, "peak": peaks["tensor"], "unit": "TFLOP/s", "frac": achieved / peaks["tensor"],
                     "peak_source": peaks["source"] + " sustained cuBLAS bf16", "frac_of_burst_peak": achieved / peaks["tensor_burst"],
                     "traffic": traffic, "traffic_source": traffic_source},
        "cpu_baseline": cpu, "prefill": prefill, "decode": decode, "varlen": varlen, "cache_append": append, "rope": rope, "projection": projection,
        "absorbed": absorbed, "flash": flash,
    }
    return line


def bench_prefill(mla, checks, device, peaks, rank, barrier, reduce_max, steps=10, warmup=3, verify=True):
    """Causal forward alone at B=4, S=4096, H=128 per GPU (the prefill configuration)."""
    w = workloads.CONFIGS["C2"]
    x = workloads.dense_inputs(w, device, shard=rank, rotate=mla.rope_apply)
    fwd_in = (x["q_nope"], x["q_pe"], x["k_nope"], x["k_pe"], x["v"])
    out = torch.empty_like(x["v"])
    lse = torch.empty(w["batch"], w["heads"], w["seq"], device=device)
    seconds = reduce_max([time_steps(lambda: mla.prefill_forward(*fwd_in, SCALE, output=out, lse=lse), steps, warmup, barrier) / steps])[0]
    tflops = workloads.dense_flops(w) / seconds / 1e12
    result = {"metric": "MLA prefill fwd TFLOP/s per GPU (bf16 causal)", "value": tflops, "unit": "TFLOP/s", "ms_per_step": seconds * 1e3,
              "workload": f"B={w['batch']} S={w['seq']} H={w['heads']} per GPU, seed {w['seed']}", "timing": "slowest rank",
              "frac_of_measured_sustained_peak": tflops / peaks["tensor"], "frac_of_measured_burst_peak": tflops / peaks["tensor_burst"]}
    if verify:
        result["verified"] = verify_training(checks, w, x, out, lse, None)
    return result


def bench_decode(mla, checks, sharding, device, peaks, rank, world, barrier, reduce_max, reduce_sum, steps=20, warmup=3, splits=8, batch=64):
    """Absorbed paged decode at batch 64, heads 128, lengths uniform in [1024, 32768] (seed 3).  With
    several GPUs the sequences are dealt to the ranks by cache pages (`sharding.decode_partition`),
    every cached token is still read by exactly one GPU, and the job's GB/s is all bytes over the
    slowest rank's time."""
    query, cache, table, lengths = workloads.decode_inputs(seed=3, batch=batch, heads=128)
    mine = sharding.decode_partition(lengths.tolist(), world)[rank] if world > 1 else list(range(batch))
    query, table, lengths = query[mine].contiguous(), table[mine].contiguous(), lengths[mine].contiguous()
    total_tokens = int(lengths.sum())
    if world > 1:
        # a rank's share is a small batch of long sequences: more partial slots than the harness's 8, so that the
        # kernel can still hand every pair of SMs an equal range of tiles
        splits = mla.decode_splits(lengths.tolist(), 128, minimum=splits)
    q, c, t, n = (z.to(device) for z in (query, cache, table, lengths))
    local = len(mine)
    workspace = mla.decode_workspace(local, 128, splits, 512, device)
    out = torch.empty(local, 1, 128, 512, device=device, dtype=torch.bfloat16)
    lse = torch.empty(local, 128, 1, device=device)

    def step():
        mla.mla_decode(q, c, t, n, SCALE, splits=splits, workspace=workspace, output=out, lse=lse)

    seconds = reduce_max([time_steps(step, steps, warmup, barrier) / steps])[0]
    algorithmic = workloads.decode_bytes(lengths, table[:, : int(((lengths + 63) // 64).max())], local, 128)
    flops = workloads.decode_flops(lengths, 128)
    own_gbs = algorithmic / seconds / 1e9
    algorithmic_all, flops_all, tokens_all = reduce_sum([algorithmic, flops, total_tokens])
    gbs = algorithmic_all / seconds / 1e9
    # the shortest and the longest of this rank's sequences against the oracle
    torch.cuda.synchronize()
    order = sorted(range(local), key=lambda i: int(lengths[i]))
    ok = checks.decode_sequences(query, cache, table, lengths, out, lse, SCALE, sorted({order[0], order[-1]})).values()
    ok = reduce_sum([0.0 if all(ok) else 1.0])[0] == 0.0
    return {"metric": "absorbed MLA decode HBM GB/s", "value": gbs, "unit": "GB/s", "us_per_step": seconds * 1e6, "timing": "slowest rank",
            "tokens": int(tokens_all), "algorithmic_bytes": int(algorithmic_all), "splits": splits, "tflops": flops_all / seconds / 1e12,
            "sequences_per_gpu": local if world == 1 else "dealt by cache pages", "per_gpu_gbs": gbs / world, "rank0_gbs": own_gbs,
            "verified": {"shortest_and_longest_sequence_of_every_rank": ok},
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / world / peaks["hbm"],
                         "peak_source": peaks["source"] + " copy bandwidth", "tensor_frac": flops_all / world / seconds / 1e12 / peaks["tensor_burst"]}}


def bench_varlen(mla, device, peaks, rank, world, barrier, reduce_max, heads=16, steps=3, warmup=1):
    """Packed long-context forward+backward: the 16 sequence lengths of seed 4 (log-uniform in
    [512, 32768], 121 320 tokens), 16 heads per GPU (each rank its own 16 heads of the 128-head job)."""
    lengths = workloads.varlen_lengths()
    total = sum(lengths)
    tensors, cu = workloads.packed_inputs(lengths, heads, 4, device, shard=rank, rotate=mla.rope_apply)
    x = (tensors["q_nope"], tensors["q_pe"], tensors["k_nope"], tensors["k_pe"], tensors["v"])
    dout = tensors["dout"]
    out = torch.empty_like(x[4])
    lse = torch.empty(heads, total, device=device)
    workspace = mla.prefill_backward_workspace(len(lengths), max(lengths), total, heads, device)
    grads = (torch.empty(total, heads, 192, device=device, dtype=torch.bfloat16), torch.empty_like(x[2]), torch.empty_like(x[3]), torch.empty_like(x[4]))

    def step():
        mla.prefill_forward(*x, SCALE, cu, max(lengths), output=out, lse=lse)
        mla.prefill_backward(dout, out, lse, *x, SCALE, cu, max(lengths), workspace=workspace, grads=grads)

    seconds = reduce_max([time_steps(step, steps, warmup, barrier) / steps])[0]
    tflops = workloads.packed_flops(lengths, heads) / seconds / 1e12
    return {"metric": "packed long-context MLA fwd+bwd TFLOP/s per GPU", "value": tflops, "unit": "TFLOP/s", "ms_per_step": seconds * 1e3,
            "timing": "slowest rank", "job_tflops": tflops * world, "tokens": total, "sequences": len(lengths), "heads_per_gpu": heads,
            "frac_of_measured_sustained_peak": tflops / peaks["tensor"]}


def bench_cache_append(mla, device, peaks, batch=64, tokens=4096, steps=20, warmup=3):
    """Appending `tokens` new rows per sequence to the paged cache (a prefill's worth): 1152 bytes
    read and 1152 written per token; the rows (302 MB) and the pages they land in exceed the L2."""
    g = torch.Generator(device=device).manual_seed(5)
    latent = torch.randn(batch, tokens, 512, device=device, generator=g).bfloat16()
    rope = torch.randn(batch, tokens, 64, device=device, generator=g).bfloat16()
    pages = tokens // 64
    cache = torch.empty(batch * pages, 64, 1, 576, device=device, dtype=torch.bfloat16)
    table = torch.randperm(batch * pages, device=device, generator=g).to(torch.int32).reshape(batch, pages).contiguous()

    def step():
        mla.cache_append(cache, latent, rope, table)

    seconds = time_steps(step, steps, warmup, lambda: None) / steps
    moved = 2 * batch * tokens * 576 * 2
    gbs = moved / seconds / 1e9
    return {"metric": "paged cache append HBM GB/s", "value": gbs, "unit": "GB/s", "us_per_step": seconds * 1e6, "tokens": batch * tokens,
            "algorithmic_bytes": moved, "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                                                     "frac": gbs / peaks["hbm"], "peak_source": peaks["source"] + " copy bandwidth"}}


def bench_absorbed(mla, device, peaks, shapes=((1, 512, 8), (4, 2048, 16)), steps=10, warmup=3):
    """Absorbed causal forward and backward (the reference's four-argument-pair API): its own largest
    prefill shape (B=1, T=512, H=8) and a larger one.  FLOPs per causal (query, key) pair and head:
    forward 2*(576+512), backward 2*(576+512+576+576+512)."""
    rows = []
    for b, t, h in shapes:
        g = torch.Generator(device=device).manual_seed(7)

        def draw(*shape):
            return (torch.randn(*shape, device=device, generator=g) * 0.25).bfloat16()

        q, qr, kv, kr = draw(b, t, h, 512), draw(b, t, h, 64), draw(b, t, 512), draw(b, t, 64)
        scale = 576 ** -0.5
        out, lse = mla.mla_forward(q, qr, kv, kr, scale)
        dout = draw(b, t, h, 512)
        fwd = time_steps(lambda: mla.mla_forward(q, qr, kv, kr, scale), steps, warmup, lambda: None) / steps
        bwd = time_steps(lambda: mla.mla_backward(dout, out, lse, q, qr, kv, kr, scale), steps, warmup, lambda: None) / steps
        pairs = causal_pairs(t) * b * h
        rows.append({"shape": f"B={b} T={t} H={h}", "forward_us": fwd * 1e6, "backward_us": bwd * 1e6,
                     "forward_tflops": pairs * 2 * (576 + 512) / fwd / 1e12,
                     "backward_tflops": pairs * 2 * (576 + 512 + 576 + 576 + 512) / bwd / 1e12})
    return {"metric": "absorbed MLA causal forward / backward", "kernels": "forward and backward tcgen05", "shapes": rows}


def bench_flash(mla, device, peaks, batch=4, seq=4096, q_heads=64, kv_heads=8, steps=10, warmup=3):
    """Causal D=128 grouped-query forward (the flash_attention.h contract): 4*128 FLOP per causal pair and query head."""
    g = torch.Generator(device=device).manual_seed(9)
    q = torch.randn(batch, seq, q_heads, 128, device=device, generator=g).bfloat16()
    k = torch.randn(batch, seq, kv_heads, 128, device=device, generator=g).bfloat16()
    v = torch.randn(batch, seq, kv_heads, 128, device=device, generator=g).bfloat16()
    scale = 128 ** -0.5
    seconds = time_steps(lambda: mla.flash_forward(q, k, v, scale), steps, warmup, lambda: None) / steps
    tflops = causal_pairs(seq) * batch * q_heads * 4 * 128 / seconds / 1e12
    return {"metric": "flash attention forward TFLOP/s (D=128 GQA, causal)", "value": tflops, "unit": "TFLOP/s", "ms_per_step": seconds * 1e3,
            "shape": f"B={batch} T={seq} Hq={q_heads} Hkv={kv_heads}", "frac_of_measured_sustained_peak": tflops / peaks["tensor"]}


def bench_projection(mla, device, peaks, rows=16384, heads=128, steps=10, warmup=3):
    """The projection GEMMs either side of the path at the prefill configuration's size (rows = 4 x 4096 tokens, H = 128):
    latent -> per-head keys and values (tensor-bound), W_UK folded into the query and W_UV applied to the latent
    output (both bound by HBM: their larger side is read or written once)."""
    g = torch.Generator(device=device).manual_seed(10)
    latent = torch.randn(rows, 512, device=device, generator=g).bfloat16()
    w_uk = (torch.randn(heads * 128, 512, device=device, generator=g) * 0.05).bfloat16()
    w_uv = (torch.randn(heads * 128, 512, device=device, generator=g) * 0.05).bfloat16()
    q_nope = torch.randn(rows, heads, 128, device=device, generator=g).bfloat16()
    o_latent = torch.randn(rows, heads, 512, device=device, generator=g).bfloat16()
    up = time_steps(lambda: mla.up_project(latent, w_uk, w_uv, heads), steps, warmup, lambda: None) / steps
    absorb = time_steps(lambda: mla.absorb_query(q_nope, w_uk), steps, warmup, lambda: None) / steps
    unabsorb = time_steps(lambda: mla.unabsorb_output(o_latent, w_uv), steps, warmup, lambda: None) / steps
    flops = 2 * rows * heads * 128 * 512
    moved = rows * heads * (128 + 512) * 2 + heads * 128 * 512 * 2
    return {"metric": "MLA projection GEMMs", "rows": rows, "heads": heads,
            "up_project": {"ms": up * 1e3, "tflops": 2 * flops / up / 1e12, "bound": "tensor", "frac_of_measured_burst_peak": 2 * flops / up / 1e12 / peaks["tensor_burst"]},
            "absorb_query": {"ms": absorb * 1e3, "gbs": moved / absorb / 1e9, "bound": "hbm", "frac": moved / absorb / 1e9 / peaks["hbm"]},
            "unabsorb_output": {"ms": unabsorb * 1e3, "gbs": moved / unabsorb / 1e9, "bound": "hbm", "frac": moved / unabsorb / 1e9 / peaks["hbm"]}}


def bench_rope(mla, device, peaks, batch=2, seq=8192, heads=128, steps=20, warmup=3):
    """Rotary embedding in place of the training step's q_pe and k_pe (270 MB read and written)."""
    g = torch.Generator(device=device).manual_seed(6)
    q_pe = torch.randn(batch, seq, heads, 64, device=device, generator=g).bfloat16()
    k_pe = torch.randn(batch, seq, 1, 64, device=device, generator=g).bfloat16()

    def step():
        mla.rope_apply(q_pe, k_pe)

    seconds = time_steps(step, steps, warmup, lambda: None) / steps
    moved = 2 * (q_pe.numel() + k_pe.numel()) * 2
    gbs = moved / seconds / 1e9
    return {"metric": "rotary embedding HBM GB/s", "value": gbs, "unit": "GB/s", "us_per_step": seconds * 1e6, "algorithmic_bytes": moved,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / peaks["hbm"],
                         "peak_source": peaks["source"] + " copy bandwidth"}}


def cpu_baseline(oracle, budget_seconds):
    """The oracle port on the host cores: B=1, S=256, H=16 fp32 forward+backward, repeated for about `budget_seconds`."""
    torch.set_num_threads(os.cpu_count() or 1)
    q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(0, 1, 256, 16, dtype=torch.float32)
    flops = causal_pairs(256) * 16 * (FWD_FLOP_PER_PAIR + BWD_FLOP_PER_PAIR)

    def once():
        out, lse = oracle.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, SCALE)
        oracle.prefill_backward(dout, out, lse, q_nope, q_pe, k_nope, k_pe, v, SCALE)

    once()
    runs, start = 0, time.perf_counter()
    while time.perf_counter() - start < budget_seconds or runs < 3:
        once()
        runs += 1
    seconds = (time.perf_counter() - start) / runs
    return {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{runs} runs of B=1 S=256 H=16 fp32 forward+backward (oracle port of reference/python/mla.py), {seconds * 1e3:.1f} ms each"}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    from oracle import mla_oracle as oracle
    w = WORKLOADS[args.workload]
    torch.set_num_threads(os.cpu_count() or 1)
    # bounded sample of the workload: the first 512 tokens of one sequence, 8 heads
    seq, heads = 512, 8
    q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(w["seed"], 1, seq, heads, dtype=torch.bfloat16, dout_std=w["dout_std"])
    flops = causal_pairs(seq) * heads * (FWD_FLOP_PER_PAIR + (BWD_FLOP_PER_PAIR if w["backward"] else 0))

    def step():
        out, lse = oracle.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, SCALE)
        if w["backward"]:
            oracle.prefill_backward(dout, out.bfloat16(), lse, q_nope, q_pe, k_nope, k_pe, v, SCALE)

    for _ in range(args.warmup):
        step()
    start = time.perf_counter()
    for _ in range(args.steps):
        step()
    seconds = time.perf_counter() - start
    value = flops * args.steps / seconds / 1e12
    sample = f"B=1 S={seq} H={heads} slice of the {args.workload} workload per step"
    return {
        "impl": "reference", "metric": "MLA fwd+bwd TFLOP/s (bf16 causal)" if w["backward"] else "MLA prefill fwd TFLOP/s (bf16 causal)",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: causal non-absorbed MLA, B={w['batch']} S={w['seq']} H={w['heads']} per GPU, "
                               f"qk=128+64 (shared k_pe), v=128, seed {w['seed']}", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--workload", default="train", choices=tuple(WORKLOADS))
    parser.add_argument("--batch", type=int, default=None, help="override the workload's batch (profiler captures)")
    parser.add_argument("--seq", type=int, default=None, help="override the workload's sequence length (profiler captures)")
    parser.add_argument("--heads", type=int, default=None, help="override the workload's heads (profiler captures)")
    parser.add_argument("--only-decode", action="store_true", help="time the paged decode alone")
    parser.add_argument("--decode-batch", type=int, default=64)
    parser.add_argument("--skip-decode", action="store_true")
    parser.add_argument("--skip-cpu", action="store_true")
    parser.add_argument("--skip-verify", action="store_true", help="leave out the oracle checks of the timed outputs (profiler captures)")
    args = parser.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    try:
        line = run_ours(args, rank, world, device)
        if line is not None:
            print(json.dumps(line), flush=True)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
