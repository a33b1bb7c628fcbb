"""The harness (`python -m dscuda_b200.suite`) on a GPU: `--test` checks configurations against the
oracle without timing, the timing mode replays CUDA graphs and checks before and after, and the
report files carry the versions."""

import json

import pytest

pytestmark = pytest.mark.gpu


def test_correctness_mode(gpu, capsys):
    from dscuda_b200 import suite
    assert suite.main(["--configs", "C1,C4", "--test"]) == 0
    printed = capsys.readouterr().out
    assert "correctness checks passed" in printed and "|" not in printed


def test_graph_replay_timing_and_report_files(gpu, capsys, tmp_path):
    from dscuda_b200 import suite
    assert suite.main(["--configs", "C1", "--warmup-ms", "50", "--sample-ms", "5", "--trials", "3", "--cpu-baseline", "--report-dir", str(tmp_path)]) == 0
    printed = capsys.readouterr().out
    assert printed.splitlines()[0].startswith("| config |") and "C1" in printed and "CPU restatement" in printed
    samples = json.loads((tmp_path / "mla_samples.json").read_text())
    assert samples["gpu"] and samples["torch"] and "CUDA Graph replay" in samples["timing"]
    assert len(samples["samples"][0]["samples_us"]) == 3
    assert (tmp_path / "mla.csv").read_text().startswith("config,workload,seconds")
    assert (tmp_path / "mla.md").exists()


def test_single_operation_eager(gpu, capsys):
    from dscuda_b200 import suite
    assert suite.main(["--configs", "C1,C4", "--operation", "backward", "--eager", "--trials", "2"]) == 0
    printed = capsys.readouterr().out
    assert "C1" in printed and "C4" not in printed and "backward" in printed
