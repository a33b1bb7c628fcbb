"""Paged-cache append on the GPU against the oracle's pack_cache (reference/python/mla.py:11-23
with a page permutation).  Byte work: every comparison is bit-exact."""

import pytest
import torch

from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu

PAGE = 64
SCALE = 576 ** -0.5


def draw_kv(seed, batch, tokens):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(batch, tokens, 576, generator=g) * 0.25).bfloat16()


def permutation(seed, count):
    return torch.randperm(count, generator=torch.Generator().manual_seed(seed))


@pytest.mark.parametrize("batch,tokens", [(1, 1), (2, 23), (3, 64), (2, 65), (4, 300)])
def test_whole_prefix_equals_pack_cache(gpu, batch, tokens):
    from dscuda_b200 import mla
    kv = draw_kv(10 + tokens, batch, tokens)
    pages = (tokens + PAGE - 1) // PAGE
    perm = permutation(tokens, batch * pages)
    expected, table = oracle.pack_cache(kv, PAGE, perm)
    cache = torch.zeros_like(expected, device=gpu)
    latent = kv[..., :512].contiguous().to(gpu)
    rope = kv[..., 512:].contiguous().to(gpu)
    mla.cache_append(cache, latent, rope, table.to(gpu))
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    assert torch.equal(cache.cpu(), expected)


def test_ragged_incremental_append_and_decode(gpu):
    from dscuda_b200 import mla
    batch, capacity, heads = 3, 200, 5
    kv = draw_kv(77, batch, capacity)
    pages = (capacity + PAGE - 1) // PAGE
    perm = permutation(5, batch * pages)
    full, table = oracle.pack_cache(kv, PAGE, perm)
    prefix = torch.tensor([130, 63, 1], dtype=torch.int32)
    extra = torch.tensor([3, 1, 2], dtype=torch.int32)          # ragged: T = 3 rows, fewer taken for b = 1, 2
    # the cache holds only the prefix of every sequence; the other slots carry a marker
    cache = torch.full_like(full, 7.0)
    flat_table = table.to(torch.int64)
    for b in range(batch):
        for position in range(int(prefix[b])):
            cache[flat_table[b, position // PAGE], position % PAGE] = full[flat_table[b, position // PAGE], position % PAGE]
    expected = cache.clone()
    new_rows = torch.zeros(batch, 3, 576, dtype=torch.bfloat16)
    for b in range(batch):
        for t in range(int(extra[b])):
            position = int(prefix[b]) + t
            new_rows[b, t] = kv[b, position]
            expected[flat_table[b, position // PAGE], position % PAGE, 0] = kv[b, position]
    device_cache = cache.to(gpu)
    mla.cache_append(device_cache, new_rows[..., :512].contiguous().to(gpu), new_rows[..., 512:].contiguous().to(gpu), table.to(gpu),
                     prefix.to(gpu), extra.to(gpu))
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    assert torch.equal(device_cache.cpu(), expected)            # appended rows written, every other byte untouched

    # decode over the appended cache equals the oracle's decode over the same tokens
    lengths = prefix + extra
    g = torch.Generator().manual_seed(9)
    query = (torch.randn(batch, 1, heads, 576, generator=g) * 0.25).bfloat16()
    out, lse = mla.mla_decode(query.to(gpu), device_cache, table.to(gpu), lengths.to(gpu), SCALE, splits=4)
    ref_out, ref_lse = oracle.paged_decode(query.float(), expected.float(), table, lengths, SCALE)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    assert float((out.float().cpu() - ref_out).abs().max()) <= 1e-2 * float(ref_out.abs().max())
    assert float((lse.cpu() - ref_lse).abs().max()) <= 1e-3


def test_indices_outside_the_cache_are_skipped_and_reported(gpu):
    from dscuda_b200 import mla
    kv = draw_kv(3, 2, 4)
    cache = torch.zeros(4, PAGE, 1, 576, dtype=torch.bfloat16, device=gpu)
    table = torch.tensor([[0, 1], [9, 2]], dtype=torch.int32, device=gpu)      # page 9 does not exist
    latent, rope = kv[..., :512].contiguous().to(gpu), kv[..., 512:].contiguous().to(gpu)
    mla.cache_append(cache, latent, rope, table)
    assert mla.device_status(reset=True) == 3
    assert torch.equal(cache[0, :4, 0].cpu(), kv[0])                           # the valid sequence was written
    assert float(cache[1:].abs().max()) == 0.0                                 # nothing else was touched
    start = torch.tensor([126, 0], dtype=torch.int32, device=gpu)              # positions 128, 129 are past two pages
    table_ok = torch.tensor([[0, 1], [2, 3]], dtype=torch.int32, device=gpu)
    mla.cache_append(cache, latent, rope, table_ok, start)
    assert mla.device_status(reset=True) == 3
    assert mla.device_status() == 0
    assert torch.equal(cache[1, 62:64, 0].cpu(), kv[0, :2])
