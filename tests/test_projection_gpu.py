"""The projection GEMMs (latent -> per-head K/V, W_UK absorbed into the query, W_UV applied to the latent
output) on the GPU, through the C ABI, against an fp32 matmul of the same bf16 inputs on the CPU, and the
identity they exist for: attention over up-projected keys/values equals absorbed attention over the latent.
Tolerance: the result is bf16-rounded from fp32 sums, so max|err| <= 2^-7 max|ref| (one bf16 ulp at the top)."""

import pytest
import torch

from conftest import max_err_ratio
from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu


def draw(generator, *shape, std=1.0):
    return (torch.randn(*shape, generator=generator) * std).bfloat16()


@pytest.mark.parametrize("rows,heads", [(1, 1), (70, 3), (257, 16), (1000, 128)])
def test_projections_match_fp32_matmul(gpu, rows, heads):
    from dscuda_b200 import mla
    g = torch.Generator().manual_seed(rows + heads)
    latent, w_uk, w_uv = draw(g, rows, 512), draw(g, heads * 128, 512, std=0.05), draw(g, heads * 128, 512, std=0.05)
    q_nope, o_latent = draw(g, rows, heads, 128), draw(g, rows, heads, 512)
    k_nope, v = mla.up_project(latent.to(gpu), w_uk.to(gpu), w_uv.to(gpu), heads)
    q_latent = mla.absorb_query(q_nope.to(gpu), w_uk.to(gpu))
    out = mla.unabsorb_output(o_latent.to(gpu), w_uv.to(gpu))
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    ref_k = (latent.float() @ w_uk.float().T).reshape(rows, heads, 128)
    ref_v = (latent.float() @ w_uv.float().T).reshape(rows, heads, 128)
    ref_q = torch.einsum("rhk,hkn->rhn", q_nope.float(), w_uk.float().reshape(heads, 128, 512))
    ref_o = torch.einsum("rhk,hnk->rhn", o_latent.float(), w_uv.float().reshape(heads, 128, 512))
    for got, ref in ((k_nope, ref_k), (v, ref_v), (q_latent, ref_q), (out, ref_o)):
        assert got.shape == ref.shape
        assert max_err_ratio(got.float().cpu(), ref) <= 2 ** -7


def test_absorbed_decode_equals_attention_over_up_projected_cache(gpu):
    """One query token per sequence: softmax(q_nope.k_nope + q_pe.k_pe) v computed with per-head keys and
    values equals W_UV applied to the absorbed decode over the latent cache with W_UK folded into the query."""
    from dscuda_b200 import mla
    g = torch.Generator().manual_seed(5)
    batch, heads, length = 2, 16, 300
    latent, k_pe = draw(g, batch, length, 512), draw(g, batch, length, 64)
    w_uk, w_uv = draw(g, heads * 128, 512, std=0.04), draw(g, heads * 128, 512, std=0.04)
    q_nope, q_pe = draw(g, batch, 1, heads, 128), draw(g, batch, 1, heads, 64)
    scale = 192 ** -0.5
    # absorbed route on the GPU
    q_latent = mla.absorb_query(q_nope.to(gpu), w_uk.to(gpu))
    query = torch.cat((q_latent, q_pe.to(gpu)), -1).contiguous()
    cache, table = oracle.pack_cache(torch.cat((latent, k_pe), -1), 64)
    lengths = torch.full((batch,), length, dtype=torch.int32)
    o_latent, _ = mla.mla_decode(query, cache.to(gpu), table.to(gpu), lengths.to(gpu), scale, splits=4)
    out = mla.unabsorb_output(o_latent, w_uv.to(gpu))
    torch.cuda.synchronize()
    # per-head route in fp32 on the CPU
    k_nope = (latent.float() @ w_uk.float().T).reshape(batch, length, heads, 128)
    v = (latent.float() @ w_uv.float().T).reshape(batch, length, heads, 128)
    score = (torch.einsum("bqhc,bkhc->bhqk", q_nope.float(), k_nope) + torch.einsum("bqhr,bkr->bhqk", q_pe.float(), k_pe.float())) * scale
    ref = torch.einsum("bhqk,bkhd->bqhd", score.softmax(-1), v)
    assert max_err_ratio(out.float().cpu(), ref) <= 2e-2        # two bf16 roundings (q_latent, o_latent) on the absorbed route
