"""Builds the reference's own CUDA implementation of the MLA path for sm_100a, as a second checker.

    python oracle/build_reference_cuda.py [REFERENCE_ROOT]

Test infrastructure, like the rest of `oracle/`: the product never loads what this builds.  The
sources are compiled where they lie in the reference checkout (nothing is copied): the MLA kernels
`kernels/attention/mla/{sm89.cu,dispatch.cu}`, `kernels/common/cuda_common.cu` and the C bridge
`benchmarks/bindings/mla_bridge.cu`, against the reference's own `include/`.  These are the kernels the
reference runs on any GPU without an sm_90 path (`kernels/attention/mla/dispatch.cu:5-31`); they use
`mma.sync` and plain loads and compile unchanged for sm_100a.  The output is
`oracle/_ref/libdscuda_mla_reference.so` (git-ignored), exporting the bridge's symbols
(`benchmarks/bindings/mla_bridge.cu:12-63`).  The D=128 flash-attention forward is built the same way
(`kernels/attention/flash_attention/{sm89_forward.cu,dispatch.cu}` and its bridge) into
`oracle/_ref/libdscuda_flash_attention_reference.so`; the dispatcher also names an sm_90 function whose
source needs wgmma, so `oracle/flash_sm90_stub.cu` supplies that symbol (never reached on sm_100a).

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
OUTPUT_DIR = ROOT / "oracle" / "_ref"
# library name -> (sources inside the checkout, extra include directory inside the checkout, sources of this directory)
LIBRARIES = {
    "libdscuda_mla_reference.so": (
        ("kernels/attention/mla/sm89.cu", "kernels/attention/mla/dispatch.cu", "kernels/common/cuda_common.cu", "benchmarks/bindings/mla_bridge.cu"),
        "kernels/attention/mla", ()),
    # flash attention: the sm_89 path (what the dispatcher runs on anything but compute capability 9.x) plus a stub
    # for the sm_90 symbol the dispatcher names
    "libdscuda_flash_attention_reference.so": (
        ("kernels/attention/flash_attention/sm89_forward.cu", "kernels/attention/flash_attention/dispatch.cu", "kernels/common/cuda_common.cu",
         "benchmarks/bindings/flash_attention_bridge.cu"),
        "kernels/attention/flash_attention", ("flash_sm90_stub.cu",)),
}


def build(reference_root: pathlib.Path):
    """Compiles the libraries; returns their paths (an empty list when the checkout or nvcc is missing)."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    built = []
    for name, (sources, include, local_sources) in LIBRARIES.items():
        if not all((reference_root / source).exists() for source in sources) or not pathlib.Path(nvcc).exists():
            continue
        output = OUTPUT_DIR / name
        OUTPUT_DIR.mkdir(parents=True, exist_ok=True)
        inputs = [reference_root / source for source in sources] + [ROOT / "oracle" / source for source in local_sources]
        if not output.exists() or output.stat().st_mtime < max(path.stat().st_mtime for path in inputs):
            command = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
                       "-cudart", "static", f"-I{reference_root / 'include'}", f"-I{reference_root / include}", *[str(path) for path in inputs],
                       "-o", str(output)]
            subprocess.run(command, check=True)
        built.append(output)
    return built


if __name__ == "__main__":
    root = pathlib.Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DSCUDA_REFERENCE_ROOT", "/root/reference"))
    result = build(root)
    print("\n".join(str(path) for path in result) if result else f"nothing built: no reference checkout at {root} (or no nvcc)")
