"""The FP8 cache variant on the GPU, through the C ABI: appended rows are bit-identical to the CPU restatement of the
format (e4m3 codes, group scales, rotary values), dequantised rows likewise, the quantisation error stays inside what
three mantissa bits allow, and decode over the dequantised cache equals the oracle's decode over the same values."""

import pytest
import torch

from conftest import max_err_ratio
from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu


def rows_of(fp8_cache, table, b, count):
    """The first `count` token rows of sequence b from a paged byte cache [blocks, page, 656]."""
    page = fp8_cache.shape[1]
    pages = (count + page - 1) // page
    gathered = fp8_cache[table[b, :pages].long()].reshape(pages * page, -1)
    return gathered[:count]


@pytest.mark.parametrize("batch,tokens,page", [(1, 1, 64), (3, 130, 64), (2, 300, 128)])
def test_append_and_dequantize_are_bit_exact(gpu, batch, tokens, page):
    from dscuda_b200 import mla
    g = torch.Generator().manual_seed(tokens)
    kv = (torch.randn(batch, tokens, 576, generator=g) * torch.rand(batch, tokens, 1, generator=g) * 3).bfloat16()
    kv[0, 0, 128:256] = 0                                           # a zero group: scale 1
    pages = (tokens + page - 1) // page
    table = torch.randperm(batch * pages, generator=g).to(torch.int32).reshape(batch, pages)
    fp8 = torch.zeros(batch * pages, page, 656, dtype=torch.uint8, device=gpu)
    mla.cache_append_fp8(fp8, kv[..., :512].contiguous().to(gpu), kv[..., 512:].contiguous().to(gpu), table.to(gpu))
    dequantised = mla.cache_dequantize_fp8(fp8)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    codes, scales, rope = oracle.quantize_fp8_rows(kv)
    expected = oracle.dequantize_fp8_rows(codes, scales, rope)
    fp8_host, deq_host = fp8.cpu(), dequantised.cpu()
    for b in range(batch):
        got = rows_of(fp8_host, table, b, tokens)
        assert torch.equal(got[:, :512], codes[b])
        assert torch.equal(got[:, 512:528].contiguous().view(torch.float32), scales[b])
        assert torch.equal(got[:, 528:].contiguous().view(torch.bfloat16), rope[b])
        got_rows = deq_host[table[b].long()].reshape(pages * page, 576)[:tokens]
        assert torch.equal(got_rows, expected[b])
    # e4m3 keeps three mantissa bits: relative error of a group's values <= 2^-4 of the group maximum
    error = (expected[..., :512].float() - kv[..., :512].float()).reshape(batch, tokens, 4, 128).abs().amax(-1)
    bound = kv[..., :512].float().reshape(batch, tokens, 4, 128).abs().amax(-1) * 2 ** -4 + 1e-6
    assert bool((error <= bound).all())


def test_decode_over_the_fp8_cache(gpu):
    from dscuda_b200 import mla
    g = torch.Generator().manual_seed(21)
    batch, heads, tokens = 3, 128, 500
    kv = torch.randn(batch, tokens, 576, generator=g).bfloat16()
    query = torch.randn(batch, 1, heads, 576, generator=g).bfloat16()
    lengths = torch.tensor([500, 77, 260], dtype=torch.int32)
    pages = (tokens + 63) // 64
    table = torch.randperm(batch * pages, generator=g).to(torch.int32).reshape(batch, pages)
    fp8 = torch.zeros(batch * pages, 64, 656, dtype=torch.uint8, device=gpu)
    mla.cache_append_fp8(fp8, kv[..., :512].contiguous().to(gpu), kv[..., 512:].contiguous().to(gpu), table.to(gpu), token_counts=lengths.to(gpu))
    cache = mla.cache_dequantize_fp8(fp8)
    scale = 192 ** -0.5
    out, lse = mla.mla_decode(query.to(gpu), cache, table.to(gpu), lengths.to(gpu), scale, splits=4)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    # the oracle on the values the FP8 rows stand for
    stand_in = oracle.dequantize_fp8_rows(*oracle.quantize_fp8_rows(kv))
    packed, _ = oracle.pack_cache(stand_in, 64)
    logical = torch.arange(batch * pages, dtype=torch.int32).reshape(batch, pages)
    ref_out, ref_lse = oracle.paged_decode(query, packed, logical, lengths, scale)
    assert max_err_ratio(out.float().cpu(), ref_out) <= 1e-2
    assert float((lse.cpu() - ref_lse).abs().max()) <= 1e-3
    # and against the unquantised cache: the price of the format (loose: e4m3 values)
    packed_exact, _ = oracle.pack_cache(kv, 64)
    exact_out, _ = oracle.paged_decode(query, packed_exact, logical, lengths, scale)
    assert max_err_ratio(out.float().cpu(), exact_out) <= 0.15
