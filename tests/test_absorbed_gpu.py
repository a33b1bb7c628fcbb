"""Absorbed-latent forward and paged decode on the GPU, through the C ABI,
against the reference-generated fixtures and the CPU oracle."""

import ctypes

import pytest
import torch

from conftest import load_golden, max_err_ratio
from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["b1_t1_h1", "b2_t17_h3", "b1_t65_h4"])
def test_forward_matches_reference_fixture(gpu, name):
    from dscuda_b200 import mla
    g = load_golden(f"absorbed_{name}")
    inputs = [g[k].to(gpu) for k in ("query", "query_rope", "latent", "key_rope")]
    out, lse = mla.mla_forward(*inputs, g["scale"])
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    # reference tolerances (benchmarks/mla.py:103-105)
    torch.testing.assert_close(out.cpu().float(), g["out"].float(), atol=8e-3, rtol=8e-3)
    torch.testing.assert_close(lse.cpu(), g["lse"], atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("b,t,h", [(1, 128, 8), (2, 257, 4), (1, 512, 8), (1, 70, 128), (1, 200, 3)])
def test_forward_matches_oracle(gpu, b, t, h):
    from dscuda_b200 import mla
    generator = torch.Generator().manual_seed(t * 7 + h)
    shapes = ((b, t, h, 512), (b, t, h, 64), (b, t, 512), (b, t, 64))
    inputs = [(torch.randn(s, generator=generator) * .25).bfloat16() for s in shapes]
    scale = ctypes.c_float(576 ** -.5).value
    out, lse = mla.mla_forward(*[x.to(gpu) for x in inputs], scale)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    ref_out, ref_lse = oracle.absorbed_forward(*inputs, scale, oracle.causal_mask(t))
    torch.testing.assert_close(out.cpu().float(), ref_out.bfloat16().float(), atol=8e-3, rtol=8e-3)
    torch.testing.assert_close(lse.cpu(), ref_lse, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("name", ["b2_t23_h3", "b2_t65_h64", "b3_t129_h16"])
@pytest.mark.parametrize("splits", [1, 8])
def test_decode_matches_reference_fixture(gpu, name, splits):
    from dscuda_b200 import mla
    g = load_golden(f"decode_{name}")
    out, lse = mla.mla_decode(g["query"].to(gpu), g["cache"].to(gpu), g["table"].to(gpu), g["lengths"].to(gpu),
                              g["scale"], splits=splits)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    torch.testing.assert_close(out.cpu().float(), g["out"].float(), atol=8e-3, rtol=8e-3)
    torch.testing.assert_close(lse.cpu(), g["lse"], atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("batch,heads,low,high,splits", [(3, 128, 1, 700, 4), (5, 16, 60, 2000, 8), (2, 200, 500, 1500, 3), (2, 128, 6000, 9000, 17),
                                                        (1, 128, 12000, 12001, 40)])
def test_decode_permuted_pages_and_garbage_tail(gpu, batch, heads, low, high, splits):
    """Random page permutation; the unused tail of every last page and all unused
    pages are filled with NaN, which must not reach the output."""
    from dscuda_b200 import mla
    query, cache, table, lengths = oracle.decode_inputs(seed=batch * 31 + heads, batch=batch, heads=heads, low=low, high=high)
    ref_out, ref_lse = oracle.paged_decode(query, cache, table, lengths, 192 ** -.5)
    poisoned = cache.clone()
    for b in range(batch):
        n = int(lengths[b])
        last_page = int(table[b, (n - 1) // 64])
        if n % 64:
            poisoned[last_page, n % 64:] = float("nan")
    out, lse = mla.mla_decode(query.to(gpu), poisoned.to(gpu), table.to(gpu), lengths.to(gpu), 192 ** -.5, splits=splits)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    assert max_err_ratio(out.cpu().float(), ref_out) <= 1e-2
    assert float((lse.cpu() - ref_lse).abs().max()) <= 1e-3


def test_decode_rejects_bad_arguments(gpu):
    from dscuda_b200 import mla
    g = load_golden("decode_b2_t23_h3")
    with pytest.raises(RuntimeError, match="C=512 and RoPE=64"):
        lib = mla.library("mla")
        status = lib.dscuda_mla_decode(None, None, None, None, None, None, None, 2, 3, 256, 64, 64, 1, 8, 0.1, None)
        mla.checked(lib, "mla", status)
    bad_pages = g["cache"].reshape(-1, 32, 1, 576).contiguous()
    with pytest.raises(RuntimeError, match="multiple of 64"):
        mla.mla_decode(g["query"].to(gpu), bad_pages.to(gpu), g["table"].to(gpu), g["lengths"].to(gpu), g["scale"])


@pytest.mark.parametrize("name", ["b1_t1_h1", "b2_t17_h3", "b1_t65_h4"])
def test_backward_matches_reference_fixture(gpu, name):
    """Gradients against both things the reference compares with: its closed-form
    mla_backward and autograd through its forward (benchmarks/mla.py:109-125)."""
    from dscuda_b200 import mla
    g = load_golden(f"absorbed_{name}")
    inputs = [g[k].to(gpu) for k in ("query", "query_rope", "latent", "key_rope")]
    grads = mla.mla_backward(g["dout"].to(gpu), g["out"].to(gpu), g["lse"].to(gpu), *inputs, g["scale"])
    torch.cuda.synchronize()
    for got, key in zip(grads, ("dquery", "dquery_rope", "dlatent", "dkey_rope")):
        torch.testing.assert_close(got.cpu().float(), g[key].float(), atol=1e-2, rtol=1e-2)
        torch.testing.assert_close(got.cpu().float(), g["ag_" + key].float(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("b,t,h", [(1, 128, 8), (2, 257, 4), (1, 512, 8), (2, 40, 16), (2, 300, 5), (1, 70, 128), (1, 1000, 16), (3, 129, 1),
                                   (1, 5, 3)])
def test_backward_matches_oracle(gpu, b, t, h):
    from conftest import rel_l2
    from dscuda_b200 import mla
    generator = torch.Generator().manual_seed(t * 3 + h)
    shapes = ((b, t, h, 512), (b, t, h, 64), (b, t, 512), (b, t, 64))
    inputs = [(torch.randn(s, generator=generator) * .25).bfloat16() for s in shapes]
    dout = (torch.randn(b, t, h, 512, generator=generator) * .2).bfloat16()
    scale = ctypes.c_float(576 ** -.5).value
    device_inputs = [x.to(gpu) for x in inputs]
    out, lse = mla.mla_forward(*device_inputs, scale)
    grads = mla.mla_backward(dout.to(gpu), out, lse, *device_inputs, scale)
    torch.cuda.synchronize()
    reference = oracle.absorbed_backward(dout, out.cpu(), lse.cpu(), *inputs, scale, oracle.causal_mask(t))
    for name, got, ref in zip(("dquery", "dquery_rope", "dlatent", "dkey_rope"), grads, reference):
        assert rel_l2(got.cpu().float(), ref) <= 1e-2, name
        torch.testing.assert_close(got.cpu().float(), ref.bfloat16().float(), atol=1e-2, rtol=1e-2)


def test_decode_empty_and_overlong_lengths(gpu):
    """Length 0: NaN output and -inf LSE, as the softmax of an empty row gives in the reference
    (reference/python/mla.py:36-38), whatever an earlier call left in the workspace.  A length above
    the capacity of the block-table row is read as that capacity."""
    from dscuda_b200 import mla
    query, cache, table, lengths = oracle.decode_inputs(seed=77, batch=4, heads=16, low=100, high=100)     # 2 pages each
    scale = 192 ** -.5
    workspace = mla.decode_workspace(4, 16, 4, 512, gpu)
    ref_out, ref_lse = oracle.paged_decode(query, cache, table, torch.tensor([100, 128, 100, 128], dtype=torch.int32), scale)
    mla.mla_decode(query.to(gpu), cache.to(gpu), table.to(gpu), lengths.to(gpu), scale, splits=4, workspace=workspace)   # fills the workspace
    odd = torch.tensor([100, 0, 100, 5000], dtype=torch.int32)
    out, lse = mla.mla_decode(query.to(gpu), cache.to(gpu), table.to(gpu), odd.to(gpu), scale, splits=4, workspace=workspace)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    out, lse = out.cpu().float(), lse.cpu()
    assert bool(torch.isnan(out[1]).all()) and bool((lse[1] == float("-inf")).all())
    for b in (0, 2, 3):
        assert max_err_ratio(out[b], ref_out[b]) <= 1e-2
        assert float((lse[b] - ref_lse[b]).abs().max()) <= 1e-3


def test_checked_decode_reports_page_numbers_outside_the_cache(gpu):
    from dscuda_b200 import mla
    query, cache, table, lengths = oracle.decode_inputs(seed=78, batch=3, heads=128, low=200, high=600)
    scale = 192 ** -.5
    args = (query.to(gpu), cache.to(gpu))
    out, lse = mla.mla_decode(*args, table.to(gpu), lengths.to(gpu), scale, splits=4, checked_pages=True)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    ref_out, ref_lse = oracle.paged_decode(query, cache, table, lengths, scale)
    assert max_err_ratio(out.cpu().float(), ref_out) <= 1e-2
    assert float((lse.cpu() - ref_lse).abs().max()) <= 1e-3
    bad = table.clone()
    bad[1, 0] = cache.shape[0] + 1000
    bad[2, 1] = -7
    out, lse = mla.mla_decode(*args, bad.to(gpu), lengths.to(gpu), scale, splits=4, checked_pages=True)
    torch.cuda.synchronize()
    assert mla.device_status(reset=True) == 3
    assert mla.device_status() == 0
    # the sequence with a clean table row is unaffected; the others are finite (page 0 was read instead)
    assert max_err_ratio(out.cpu().float()[0], ref_out[0]) <= 1e-2
    assert bool(torch.isfinite(out.float()).all())
