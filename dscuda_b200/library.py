"""ctypes bindings of the C ABI declared in `include/dscuda_c_api.h`.

Mirrors the helpers of the reference's `benchmarks/common.py:19-40`
(`library`, `bind`, `checked`): a non-zero status becomes a RuntimeError
carrying `dscuda_<prefix>_last_error()`.
"""

from __future__ import annotations

import ctypes
import functools
import os
import pathlib

ROOT = pathlib.Path(__file__).resolve().parents[1]
P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

# name -> (argument types, result type); the order is the C declaration order.
MLA_SYMBOLS = {
    "dscuda_mla_last_error": ([], ctypes.c_char_p),
    "dscuda_mla_forward": ([P] * 6 + [I] * 5 + [F, P], I),
    "dscuda_mla_backward": ([P] * 11 + [I] * 5 + [F, P], I),
    "dscuda_mla_workspace_elements": ([I] * 4, ctypes.c_size_t),
    "dscuda_mla_decode": ([P] * 7 + [I] * 7 + [F, P], I),
    "dscuda_mla_decode_checked": ([P] * 7 + [I] * 8 + [F, P], I),
    "dscuda_mla_decode_static_capacity": ([], ctypes.c_size_t),
    "dscuda_mla_decode_static": ([P] * 6 + [I] * 7 + [F, P], I),
    "dscuda_mla_cache_append": ([P] * 6 + [I] * 7 + [P], I),
    "dscuda_mla_cache_append_fp8": ([P] * 6 + [I] * 7 + [P], I),
    "dscuda_mla_cache_dequantize_fp8": ([P] * 2 + [ctypes.c_longlong] * 2 + [P], I),
    "dscuda_mla_rope_apply": ([P] * 3 + [ctypes.c_longlong] + [I] * 3 + [F, P], I),
    "dscuda_mla_prefill_forward": ([P] * 8 + [I] * 7 + [F, P], I),
    "dscuda_mla_prefill_backward_workspace_bytes": ([I] * 4, ctypes.c_size_t),
    "dscuda_mla_prefill_backward_scratch_limit": ([ctypes.c_longlong], ctypes.c_size_t),
    "dscuda_mla_prefill_backward_launches": ([I] * 5, I),
    "dscuda_mla_prefill_backward": ([P] * 14 + [I] * 7 + [F, P], I),
    "dscuda_mla_up_project": ([P] * 5 + [ctypes.c_longlong, I, P], I),
    "dscuda_mla_absorb_query": ([P] * 3 + [ctypes.c_longlong, I, P], I),
    "dscuda_mla_unabsorb_output": ([P] * 3 + [ctypes.c_longlong, I, P], I),
    "dscuda_mla_device_status": ([I], I),
}
FLASH_SYMBOLS = {
    "dscuda_flash_last_error": ([], ctypes.c_char_p),
    "dscuda_flash_forward": ([P] * 5 + [I] * 5 + [F, P], I),
    "dscuda_flash_device_status": ([I], I),
}


def library_path(name: str) -> pathlib.Path:
    """`build/` at the repository root, or the directory named by DSCUDA_BUILD_DIR."""
    directory = pathlib.Path(os.environ["DSCUDA_BUILD_DIR"]) if os.environ.get("DSCUDA_BUILD_DIR") else ROOT / "build"
    return directory / f"libdscuda_{name}_bench.so"


@functools.lru_cache(maxsize=None)
def library(name: str) -> ctypes.CDLL:
    """Load `build/libdscuda_<name>_bench.so` and set every prototype."""
    path = library_path(name)
    if not path.exists():
        raise RuntimeError(f"{path} is missing: run `python -m dscuda_b200.build` (there is no fallback path)")
    lib = ctypes.CDLL(str(path))
    for symbol, (arguments, result) in (MLA_SYMBOLS if name == "mla" else FLASH_SYMBOLS).items():
        function = getattr(lib, symbol)
        function.argtypes, function.restype = arguments, result
    return lib


def checked(lib: ctypes.CDLL, prefix: str, status: int) -> None:
    if status:
        raise RuntimeError(getattr(lib, f"dscuda_{prefix}_last_error")().decode())
