"""`dscuda_b200.ncu_extract` on small committed samples of Nsight Compute output (no GPU, no ncu):
kernel names map to the short labels, launches merge per label with shares that add up, the
counter table and the traffic file carry DRAM bytes per launch and per work unit."""

import json
import pathlib

from dscuda_b200 import ncu_extract

GOLDEN = pathlib.Path(__file__).resolve().parent / "golden"


def test_short_kernel_names():
    name = ncu_extract.short_kernel_name
    assert name("dscuda::<unnamed>::attention_forward_kernel<3>(dscuda::<unnamed>::ForwardParams)") == "prefill_fwd"
    assert name("dscuda::<unnamed>::attention_forward_kernel<(int)2>(dscuda::<unnamed>::ForwardParams)") == "flash_fwd"
    assert name("dscuda::<unnamed>::backward_dq_kernel(dscuda::<unnamed>::BackwardParams)") == "prefill_bwd_dq"
    assert name("dscuda::<unnamed>::backward_dkdv_kernel(dscuda::<unnamed>::BackwardParams)") == "prefill_bwd_dkdv"
    assert name("dscuda::<unnamed>::delta_kernel(float *, ...)") == "prefill_delta"
    assert name("dscuda::<unnamed>::absorbed_delta_kernel(__nv_bfloat16 *, ...)") == "absorbed_delta"
    assert name("dscuda::<unnamed>::absorbed_attention_kernel(dscuda::<unnamed>::AbsorbedParams)") == "absorbed_fwd"
    assert name("dscuda::<unnamed>::decode_combine_kernel(__nv_bfloat16 *, float *, const float *, const int *, int, int)") == "decode_combine"
    assert name("dscuda::<unnamed>::absorbed_backward_key_kernel(dscuda::<unnamed>::AbsorbedBackwardParams)") == "absorbed_bwd_key"
    assert name("dscuda::<unnamed>::absorbed_backward_query_kernel(dscuda::<unnamed>::AbsorbedBackwardParams)") == "absorbed_bwd_query"
    assert name("void at::native::vectorized_elementwise_kernel<4, ...>(int, T2, T3)") == ncu_extract.OTHER


def test_launch_list_merges_per_label():
    launches = ncu_extract.read_launches((GOLDEN / "ncu_launches_sample.csv").read_text())
    assert launches and all(row["time_us"] > 0 for row in launches)
    labels = {row["label"] for row in launches}
    assert {"absorbed_bwd_key", "absorbed_bwd_query", "absorbed_fwd", "absorbed_delta"} <= labels
    merged = ncu_extract.merge_by_label(launches)
    assert sum(row["launches"] for row in merged) == len(launches)
    assert abs(sum(row["time_us"] for row in merged) - sum(row["time_us"] for row in launches)) < 1e-6
    table = ncu_extract.launch_table(launches)
    shares = [float(line.split("|")[-2].strip().rstrip(" %")) for line in table.splitlines()[2:]]
    assert abs(sum(shares) - 100.0) < 0.5


def test_counter_table_and_traffic_file(tmp_path):
    captures = ncu_extract.read_counters((GOLDEN / "ncu_raw_sample.csv").read_text())
    assert [row["label"] for row in captures] == ["prefill_fwd", "prefill_bwd_dq", "prefill_bwd_dkdv"]
    forward = captures[0]
    assert 100e6 < forward["dram_read_bytes"] < 130e6 and 50 < forward["tensor_pct"] < 70 and forward["registers"] == 168
    assert "prefill_bwd_dkdv" in ncu_extract.counter_table(captures)
    target = tmp_path / "traffic.json"
    ncu_extract.update_traffic_json(target, "train_step", ncu_extract.traffic_entry(captures, 131072, "token_head"), "sample")
    entry = json.loads(target.read_text())["train_step"]["kernels"]["prefill_fwd"]
    assert abs(entry["dram_bytes_per_launch"] - (forward["dram_read_bytes"] + forward["dram_write_bytes"])) < 1
    assert abs(entry["dram_bytes_per_token_head"] * 131072 - entry["dram_bytes_per_launch"]) < 1
