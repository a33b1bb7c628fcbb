"""CPU-side checks of the C-ABI libraries: they load, they export every symbol
the public header declares, and argument validation fails on the host with the
reference's status/last-error convention (no GPU needed: a rejected call never
reaches a launch)."""

import ctypes
import pathlib
import re

import pytest

from dscuda_b200 import library

ROOT = pathlib.Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "dscuda_c_api.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dscuda_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_reference_bridge_symbols():
    names = declared_symbols()
    # the five MLA symbols and two flash symbols the reference's harness binds
    for required in ("dscuda_mla_last_error", "dscuda_mla_forward", "dscuda_mla_backward", "dscuda_mla_workspace_elements",
                     "dscuda_mla_decode", "dscuda_flash_last_error", "dscuda_flash_forward"):
        assert required in names


def test_libraries_export_every_declared_symbol():
    mla = ctypes.CDLL(str(library.library_path("mla")))
    flash = ctypes.CDLL(str(library.library_path("flash_attention")))
    for name in declared_symbols():
        lib = flash if name.startswith("dscuda_flash") else mla
        assert hasattr(lib, name), name
    assert set(library.MLA_SYMBOLS) | set(library.FLASH_SYMBOLS) == set(declared_symbols())


def test_workspace_sizes_are_host_only():
    lib = library.library("mla")
    # reference: kernels/attention/mla/sm89.cu:539-541 -> B*H*splits*(C+2)
    assert lib.dscuda_mla_workspace_elements(64, 128, 8, 512) == 64 * 128 * 8 * 514
    assert lib.dscuda_mla_prefill_backward_workspace_bytes(2, 8192, 16384, 128) >= 16384 * 64 * 4 + 16384 * 128 * 4


def test_backward_workspace_follows_the_scratch_limit():
    """Host-only arithmetic of the backward's dS^T scratch: 16 KB per (128-key tile, 64-query tile at or after it), as many
    heads at a time as the limit holds, the recomputing route (small workspace, four launches) when not even one fits."""
    lib = library.library("mla")
    batch, seq, heads = 2, 8192, 128
    fixed = 16384 * 64 * 4 + 16384 * heads * 4 + 16384 * heads * 64 * 4          # dk_pe sums, delta, per-head dk_pe contributions
    key_tiles = seq // 128
    per_head = batch * (key_tiles * key_tiles + key_tiles) * 16384              # 2 bytes per causal pair, tile-rounded
    previous = lib.dscuda_mla_prefill_backward_scratch_limit(-1)
    try:
        assert lib.dscuda_mla_prefill_backward_scratch_limit(-1) == previous                       # a negative value only reads
        for limit, group in ((0, 0), (per_head - 1, 0), (per_head, 1), (5 * per_head + 7, 5), (1 << 40, heads)):
            lib.dscuda_mla_prefill_backward_scratch_limit(limit)
            size = lib.dscuda_mla_prefill_backward_workspace_bytes(batch, seq, batch * seq, heads)
            assert fixed + group * per_head <= size <= fixed + group * per_head + 4096, (limit, group)
            launches = lib.dscuda_mla_prefill_backward_launches(batch, seq, batch * seq, heads, 0)
            assert launches == (4 if group == 0 else 2 + 2 * -(-heads // group))
        # packed batches: the bound needs no lengths and is never above the dense figure for the same longest sequence
        lib.dscuda_mla_prefill_backward_scratch_limit(1 << 40)
        packed = lib.dscuda_mla_prefill_backward_workspace_bytes(16, 32768, 121320, 16)
        tokens_fixed = 121320 * 64 * 4 + 121320 * 16 * 4 + 121320 * 16 * 64 * 4
        assert packed - tokens_fixed <= 16 * (32768 * 121320 + 4 * 121320 * 128 + 64 * 16384) + 8192
        assert packed - tokens_fixed >= 16 * sum(n * n for n in (25869, 26465)) + 0          # at least what its two longest sequences need
    finally:
        lib.dscuda_mla_prefill_backward_scratch_limit(previous)
    assert lib.dscuda_mla_prefill_backward_scratch_limit(-1) == previous


@pytest.mark.parametrize("rank,rope", [(256, 64), (512, 32)])
def test_absorbed_entry_points_reject_other_head_sizes(rank, rope):
    lib = library.library("mla")
    # reference: kernels/attention/mla/sm89.cu:20-24 -> invalid_argument -> status 1 + message
    assert lib.dscuda_mla_forward(None, None, None, None, None, None, 1, 4, 2, rank, rope, 0.1, None) == 1
    assert b"C=512 and RoPE=64" in lib.dscuda_mla_last_error()
    assert lib.dscuda_mla_backward(*([None] * 11), 1, 4, 2, rank, rope, 0.1, None) == 1
    assert b"C=512 and RoPE=64" in lib.dscuda_mla_last_error()
    assert lib.dscuda_mla_decode(*([None] * 7), 1, 2, rank, rope, 64, 1, 8, 0.1, None) == 1
    with pytest.raises(RuntimeError, match="C=512"):
        library.checked(lib, "mla", 1)


def test_prefill_entry_points_validate_on_the_host():
    lib = library.library("mla")
    args = [None] * 8
    assert lib.dscuda_mla_prefill_forward(*args, 1, 16, 16, 2, 64, 64, 128, 0.1, None) == 1
    assert b"nope=128" in lib.dscuda_mla_last_error()
    assert lib.dscuda_mla_prefill_forward(*args, 1, 16, 17, 2, 128, 64, 128, 0.1, None) == 1
    assert b"total_tokens" in lib.dscuda_mla_last_error()
    assert lib.dscuda_mla_prefill_forward(*args, 1, 16, 16, 2, 128, 64, 128, -1.0, None) == 1
    assert b"positive softmax scale" in lib.dscuda_mla_last_error()
    assert lib.dscuda_mla_prefill_forward(*args, 1, 16, 16, 2, 128, 64, 128, 0.1, None) == 1
    assert b"null tensor pointer" in lib.dscuda_mla_last_error()
    assert lib.dscuda_mla_prefill_backward(*([None] * 14), 1, 16, 16, 2, 128, 64, 128, 0.1, None) == 1
    assert b"null tensor pointer" in lib.dscuda_mla_last_error()


def test_flash_entry_point_validates_on_the_host():
    lib = library.library("flash_attention")
    assert lib.dscuda_flash_forward(None, None, None, None, None, 1, 64, 4, 2, 64, 0.1, None) == 1
    assert b"head_size 128" in lib.dscuda_flash_last_error()
    assert lib.dscuda_flash_forward(None, None, None, None, None, 1, 64, 3, 2, 128, 0.1, None) == 1
    assert b"divisible" in lib.dscuda_flash_last_error()


def test_host_wrappers_refuse_cpu_tensors():
    import torch
    from dscuda_b200 import mla
    x = torch.zeros(1, 4, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        mla.flash_forward(x, x, x, 0.1)


def test_cache_append_validates_on_the_host():
    lib = library.library("mla")
    args = [None] * 6
    assert lib.dscuda_mla_cache_append(*args, 1, 4, 256, 64, 64, 2, 8, None) == 1
    assert b"KV rank 512" in lib.dscuda_mla_last_error()
    assert lib.dscuda_mla_cache_append(*args, 1, 0, 512, 64, 64, 2, 8, None) == 1
    assert b"positive batch" in lib.dscuda_mla_last_error()
    assert lib.dscuda_mla_cache_append(*args, 1, 4, 512, 64, 64, 2, 8, None) == 1
    assert b"null tensor pointer" in lib.dscuda_mla_last_error()


def test_rope_validates_on_the_host():
    lib = library.library("mla")
    assert lib.dscuda_mla_rope_apply(None, None, None, 4, 2, 4, 32, 10000.0, None) == 1
    assert b"RoPE size 64" in lib.dscuda_mla_last_error()
    assert lib.dscuda_mla_rope_apply(None, None, None, 4, 2, 0, 64, 10000.0, None) == 1
    assert b"positions" in lib.dscuda_mla_last_error()
    assert lib.dscuda_mla_rope_apply(None, None, None, 4, 2, 4, 64, 10000.0, None) == 1
    assert b"null tensor pointer" in lib.dscuda_mla_last_error()
