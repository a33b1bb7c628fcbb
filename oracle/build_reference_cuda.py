"""Builds the reference's own CUDA implementation of the MLA path for sm_100a, as a second checker.

    python oracle/build_reference_cuda.py [REFERENCE_ROOT]

Test infrastructure, like the rest of `oracle/`: the product never loads what this builds.  The
sources are compiled where they lie in the reference checkout (nothing is copied): the MLA kernels
`kernels/attention/mla/{sm89.cu,dispatch.cu}`, `kernels/common/cuda_common.cu` and the C bridge
`benchmarks/bindings/mla_bridge.cu`, against the reference's own `include/`.  These are the kernels the
reference runs on any GPU without an sm_90 path (`kernels/attention/mla/dispatch.cu:5-31`); they use
`mma.sync` and plain loads and compile unchanged for sm_100a.  The output is
`oracle/_ref/libdscuda_mla_reference.so` (git-ignored), exporting the bridge's symbols
(`benchmarks/bindings/mla_bridge.cu:12-63`).

`tests/test_reference_cuda_gpu.py` compares this repository's kernels with it on the reference's own
benchmark shapes, and `bench.py` times it beside them (`reference_cuda` in the line); both skip when the
library has not been built (no reference checkout at build time).
"""
from __future__ import annotations

import os
import pathlib
import shutil
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parents[1]
OUTPUT = ROOT / "oracle" / "_ref" / "libdscuda_mla_reference.so"
SOURCES = ("kernels/attention/mla/sm89.cu", "kernels/attention/mla/dispatch.cu", "kernels/common/cuda_common.cu",
           "benchmarks/bindings/mla_bridge.cu")


def build(reference_root: pathlib.Path) -> pathlib.Path | None:
    """Compiles the library; returns its path, or None when the checkout or nvcc is missing."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not all((reference_root / name).exists() for name in SOURCES) or not pathlib.Path(nvcc).exists():
        return None
    OUTPUT.parent.mkdir(parents=True, exist_ok=True)
    newest = max((reference_root / name).stat().st_mtime for name in SOURCES)
    if OUTPUT.exists() and OUTPUT.stat().st_mtime >= newest:
        return OUTPUT
    command = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
               "-cudart", "static", f"-I{reference_root / 'include'}", f"-I{reference_root / 'kernels' / 'attention' / 'mla'}",
               *[str(reference_root / name) for name in SOURCES], "-o", str(OUTPUT)]
    subprocess.run(command, check=True)
    return OUTPUT


if __name__ == "__main__":
    root = pathlib.Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DSCUDA_REFERENCE_ROOT", "/root/reference"))
    result = build(root)
    print(result if result is not None else f"nothing built: no reference checkout at {root} (or no nvcc)")
