"""The reference's own harness, unchanged, against these libraries.

`benchmarks/run.py mla --test` and `benchmarks/run.py flash_attention --test` of the reference
load `build/libdscuda_{mla,flash_attention}_bench.so` relative to their own checkout
(benchmarks/common.py:19-20), bind the bridge symbols with their own ctypes signatures
(benchmarks/mla.py:27-32, benchmarks/flash_attention.py:37) and compare with their own PyTorch
expressions at their own tolerances (benchmarks/mla.py:103-105,122-125).  This test copies the
harness files of a reference checkout to a temporary directory, puts this repository's libraries
in its build/ and runs both commands.

The checkout is looked for in $DSCUDA_REFERENCE_ROOT, then in baseline/_ref/dscuda at the
repository root (a git-ignored staging copy made by `__graft_entry__.build()` on a machine that has
the reference); without either the test is skipped.
"""

import os
import pathlib
import shutil
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = pathlib.Path(__file__).resolve().parents[1]
HARNESS_FILES = ("benchmarks/run.py", "benchmarks/common.py", "benchmarks/mla.py", "benchmarks/flash_attention.py",
                 "reference/python/__init__.py", "reference/python/mla.py")


def reference_root():
    for candidate in (os.environ.get("DSCUDA_REFERENCE_ROOT"), ROOT / "baseline" / "_ref" / "dscuda"):
        if candidate and all((pathlib.Path(candidate) / name).exists() for name in HARNESS_FILES):
            return pathlib.Path(candidate)
    return None


@pytest.mark.parametrize("family,checks", [("mla", 10), ("flash_attention", 4)])
def test_reference_harness_passes_against_these_libraries(gpu, tmp_path, family, checks):
    source = reference_root()
    if source is None:
        pytest.skip("no reference checkout (set DSCUDA_REFERENCE_ROOT)")
    for name in HARNESS_FILES:
        target = tmp_path / name
        target.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(source / name, target)
    (tmp_path / "build").mkdir()
    for name in ("mla", "flash_attention"):
        shutil.copyfile(ROOT / "build" / f"libdscuda_{name}_bench.so", tmp_path / "build" / f"libdscuda_{name}_bench.so")
    done = subprocess.run([sys.executable, "benchmarks/run.py", family, "--test"], cwd=tmp_path, capture_output=True, text=True, timeout=600)
    log = ROOT / "gpurun_out"
    if log.is_dir():
        (log / f"reference_harness_{family}.log").write_text(done.stdout + done.stderr)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert f"{family}: {checks} correctness checks passed" in done.stdout
