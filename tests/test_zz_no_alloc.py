"""The workspace-free decode entry point (`dscuda_mla_decode_static`).

Some hosts cannot allocate device memory at the place they call the decode from
(a serving loop that pre-sizes its pool, a plugin inside another allocator).
For them the library keeps the split partials in a fixed array of its own.  This
file checks, through the C ABI, that the workspace-free call returns what the
regular call returns, twice in a row on the same array, and that it refuses
requests beyond the array's capacity.  It is named so that pytest collects it
last."""

import pytest
import torch

from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu


def call_static(lib, out, lse, query, cache, table, lengths, splits, scale):
    b, _, h, _ = query.shape
    return lib.dscuda_mla_decode_static(
        out.data_ptr(), lse.data_ptr(), query.data_ptr(), cache.data_ptr(), table.data_ptr(), lengths.data_ptr(),
        b, h, 512, 64, cache.shape[1], table.shape[1], splits, scale, torch.cuda.current_stream().cuda_stream)


def test_static_scratch_decode_matches_workspace_decode_twice(gpu):
    from dscuda_b200 import mla
    from dscuda_b200.library import checked, library
    lib = library("mla")
    scale = 192 ** -.5
    for seed, batch, heads, splits in ((3, 4, 128, 8), (5, 6, 64, 4)):       # two calls in a row, different shapes
        query, cache, table, lengths = (t.to(gpu) for t in oracle.decode_inputs(seed=seed, batch=batch, heads=heads, low=40, high=1500))
        assert batch * heads * splits <= lib.dscuda_mla_decode_static_capacity()
        expected_out, expected_lse = mla.mla_decode(query, cache, table, lengths, scale, splits=splits)
        out = torch.zeros_like(expected_out)
        lse = torch.zeros_like(expected_lse)
        # Free device memory as the driver reports it (cudaMemGetInfo) sees every allocation of the process, not
        # only those of torch's caching allocator.  The first call on a device also resolves the array's address,
        # so the comparison is made around a second call.
        checked(lib, "mla", call_static(lib, out, lse, query, cache, table, lengths, splits, scale))
        torch.cuda.synchronize()
        before_torch = torch.cuda.memory_allocated()
        before_free, _ = torch.cuda.mem_get_info()
        checked(lib, "mla", call_static(lib, out, lse, query, cache, table, lengths, splits, scale))
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before_torch
        assert torch.cuda.mem_get_info()[0] == before_free
        assert mla.device_status() == 0
        # tolerances of the decode tests (benchmarks/mla.py:103-105 of the reference)
        torch.testing.assert_close(out.float(), expected_out.float(), atol=8e-3, rtol=8e-3)
        torch.testing.assert_close(lse, expected_lse, atol=1e-4, rtol=1e-4)
        # and against the CPU oracle, so the pair cannot agree on a wrong answer
        ref_out, ref_lse = oracle.paged_decode(query.cpu(), cache.cpu(), table.cpu(), lengths.cpu(), scale)
        assert float((out.float().cpu() - ref_out).abs().max()) <= 1e-2 * float(ref_out.abs().max())
        assert float((lse.cpu() - ref_lse).abs().max()) <= 1e-3


def test_static_scratch_decode_rejects_requests_beyond_capacity(gpu):
    from dscuda_b200.library import library
    lib = library("mla")
    capacity = lib.dscuda_mla_decode_static_capacity()
    assert capacity == 8192
    # 128 heads x 8 splits x 9 sequences = 9216 partials > 8192: refused on the host, nothing is launched
    status = lib.dscuda_mla_decode_static(None, None, None, None, None, None, 9, 128, 512, 64, 64, 4, 8, 0.1, None)
    assert status == 1
    message = lib.dscuda_mla_last_error().decode()
    assert "at most 8192" in message and "9216" in message
