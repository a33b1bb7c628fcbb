"""Build the native libraries with CMake (sm_100a only).

    python -m dscuda_b200.build

Outputs `build/libdscuda_mla_bench.so` and
`build/libdscuda_flash_attention_bench.so` at the repository root, the names the
reference's harness loads (`benchmarks/common.py:19-20`).  nvcc cross-compiles,
so no GPU is needed to build.
"""

from __future__ import annotations

import os
import pathlib
import shutil
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parents[1]
BUILD = ROOT / "build"
# the two product libraries, then the test-only probe library (tests/csrc)
LIBRARIES = ("libdscuda_mla_bench.so", "libdscuda_flash_attention_bench.so", "libdscuda_test_probes.so")


def _tool(name: str) -> str:
    beside_python = pathlib.Path(sys.executable).parent / name
    if beside_python.exists():
        return str(beside_python)
    found = shutil.which(name)
    if found is None:
        raise RuntimeError(f"{name} not found")
    return found


def build(verbose: bool = False) -> list[pathlib.Path]:
    """Configure and build; returns the library paths."""
    nvcc = os.environ.get("CUDACXX") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    work = BUILD / "cmake"
    work.mkdir(parents=True, exist_ok=True)
    cmake = _tool("cmake")
    configure = [cmake, "-S", str(ROOT), "-B", str(work), "-DCMAKE_BUILD_TYPE=Release", f"-DCMAKE_CUDA_COMPILER={nvcc}"]
    if shutil.which("ninja") or (pathlib.Path(sys.executable).parent / "ninja").exists():
        configure += ["-G", "Ninja", f"-DCMAKE_MAKE_PROGRAM={_tool('ninja')}"]
    sink = None if verbose else subprocess.PIPE
    for command in (configure, [cmake, "--build", str(work), "-j", str(os.cpu_count() or 4)]):
        done = subprocess.run(command, stdout=sink, stderr=subprocess.STDOUT, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"{' '.join(command)} failed:\n{done.stdout or ''}")
    paths = [BUILD / name for name in LIBRARIES]
    for path in paths:
        if not path.exists():
            raise RuntimeError(f"build finished without producing {path}")
    return paths


if __name__ == "__main__":
    for built in build(verbose=True):
        print(built)
