"""The benchmark suite end to end on the GPU, on the small configuration."""

import pytest

pytestmark = pytest.mark.gpu


def test_suite_runs_the_small_configuration(gpu, tmp_path):
    from dscuda_b200 import suite
    report = tmp_path / "report.md"
    assert suite.main(["--configs", "C1", "--trials", "2", "--report", str(report)]) == 0
    text = report.read_text()
    assert "| C1 |" in text and "TFLOP/s" in text
