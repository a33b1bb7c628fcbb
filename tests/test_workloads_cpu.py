"""Benchmark workloads and the suite's host side (no GPU): the package's input generators
agree with the oracle's, the work counts are the documented ones, the report is well formed."""

import pytest
import torch

from dscuda_b200 import suite, workloads
from oracle import mla_oracle as oracle


def test_generators_agree_with_the_oracle():
    assert workloads.varlen_lengths() == oracle.varlen_lengths()
    assert sum(workloads.varlen_lengths()) == 121320
    ours = workloads.decode_inputs(seed=3, batch=3, heads=2, low=10, high=200)
    theirs = oracle.decode_inputs(seed=3, batch=3, heads=2, low=10, high=200)
    for a, b in zip(ours, theirs):
        assert torch.equal(a, b)


def test_work_counts():
    assert workloads.FWD_FLOP_PER_PAIR == 640 and workloads.BWD_FLOP_PER_PAIR == 1664
    assert abs(workloads.dense_flops(workloads.CONFIGS["C2"]) / 1e12 - 2.7495) < 1e-3
    assert abs(workloads.dense_flops(workloads.CONFIGS["C3"]) / 1e12 - 19.7936) < 1e-3
    c5 = workloads.CONFIGS["C5"]
    assert abs(workloads.packed_flops(workloads.varlen_lengths(), c5["heads"]) / 1e12 - 38.00) < 1e-2
    # C4: the lengths are the first draw of the seed-3 generator
    g = torch.Generator().manual_seed(3)
    lengths = torch.randint(1024, 32769, (64,), generator=g)
    assert int(lengths.sum()) == 1131680
    pages = int(((lengths + 63) // 64).max())
    table = torch.zeros(64, pages, dtype=torch.int32)
    assert workloads.decode_bytes(lengths.to(torch.int32), table, 64, 128) == 1321683456
    assert abs(workloads.decode_flops(lengths, 128) / 1e12 - 0.3152) < 1e-3


def test_report_and_arguments():
    rows = [dict(config="C4", workload="decode", seconds=5e-4, value=2600.0, unit="GB/s", bound="hbm", peak=6540.2, peak_source="measured",
                 fraction=2600.0 / 6540.2)]
    text = suite.format_report(rows)
    assert text.splitlines()[0].startswith("| config |") and "2600.0 GB/s" in text and "0.398" in text
    with pytest.raises(SystemExit):
        suite.main(["--configs", "C9"])
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no GPU"):
            suite.main(["--configs", "C1"])
    assert set(workloads.CONFIGS) == {"C1", "C2", "C3", "C4", "C5"}
