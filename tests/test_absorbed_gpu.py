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


@pytest.mark.parametrize("batch,heads,low,high,splits", [(3, 128, 1, 700, 4), (5, 16, 60, 2000, 8), (2, 200, 500, 1500, 3)])
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


@pytest.mark.parametrize("b,t,h", [(1, 128, 8), (2, 257, 4), (1, 512, 8), (2, 40, 16)])
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
