"""The CPU oracle against fixtures produced by the reference's own
reference/python/mla.py (tests/golden/make_golden.py).  CPU only."""

import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import mla_oracle as oracle


@pytest.mark.parametrize("name,t", [("b1_t1_h1", 1), ("b2_t17_h3", 17), ("b1_t65_h4", 65)])
def test_absorbed_forward_backward_match_reference(name, t):
    g = load_golden(f"absorbed_{name}")
    inputs = (g["query"], g["query_rope"], g["latent"], g["key_rope"])
    mask = oracle.causal_mask(t)
    out, lse = oracle.absorbed_forward(*inputs, g["scale"], mask)
    # the reference rounds O to bf16 (mla.py:39); rounding the restatement the same way must give the same bits
    assert torch.equal(out.bfloat16(), g["out"])
    torch.testing.assert_close(lse, g["lse"], atol=0, rtol=0)
    grads = oracle.absorbed_backward(g["dout"], g["out"], g["lse"], *inputs, g["scale"], mask)
    for got, key in zip(grads, ("dquery", "dquery_rope", "dlatent", "dkey_rope")):
        assert torch.equal(got.bfloat16(), g[key]), key
        # autograd through the reference forward (benchmarks/mla.py:109-110) agrees within the
        # reference's own backward tolerance (benchmarks/mla.py:125)
        torch.testing.assert_close(got.bfloat16(), g["ag_" + key], atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("name", ["b2_t23_h3", "b2_t65_h64", "b3_t129_h16"])
def test_paged_decode_matches_reference(name):
    g = load_golden(f"decode_{name}")
    out, lse = oracle.paged_decode(g["query"], g["cache"], g["table"], g["lengths"], g["scale"])
    assert torch.equal(out.bfloat16(), g["out"])
    torch.testing.assert_close(lse, g["lse"], atol=1e-6, rtol=1e-6)


def test_paged_decode_is_invariant_under_page_permutation():
    g = load_golden("decode_b3_t129_h16")
    generator = torch.Generator().manual_seed(5)
    pages = g["table"].numel()
    permutation = torch.randperm(pages, generator=generator)
    cache, table = oracle.pack_cache(g["kv"], 64, permutation)
    out, lse = oracle.paged_decode(g["query"], cache, table, g["lengths"], g["scale"])
    assert torch.equal(out.bfloat16(), g["out"])
    assert not torch.equal(table, g["table"])


@pytest.mark.parametrize("name", ["b2_s37_h3", "b1_s130_h2"])
def test_prefill_restatement_matches_reference_embedding(name):
    """Non-absorbed contract: the restatement against what the reference's own
    functions give through the head-fold / zero-pad embedding."""
    g = load_golden(f"prefill_embed_{name}")
    inputs = (g["q_nope"], g["q_pe"], g["k_nope"], g["k_pe"], g["v"])
    out, lse = oracle.prefill_forward(*inputs, g["scale"])
    torch.testing.assert_close(lse, g["lse"], atol=2e-6, rtol=2e-6)
    assert (out.bfloat16().float() - g["out"].float()).abs().max() <= 2 ** -7 * g["out"].float().abs().max()
    assert rel_l2(out, g["out"].float()) < 3e-3
    dq, dk_nope, dk_pe, dv = oracle.prefill_backward(g["dout"], g["out"], g["lse"], *inputs, g["scale"])
    assert rel_l2(dq, g["dq"].float()) < 3e-3
    assert rel_l2(dk_nope, g["dk_nope"].float()) < 3e-3
    assert rel_l2(dv, g["dv"].float()) < 3e-3
    dk_pe_reference = g["dk_pe_heads"].float().sum(2, keepdim=True)
    assert rel_l2(dk_pe, dk_pe_reference) < 3e-3


def test_prefill_backward_matches_autograd_fp64():
    g = torch.Generator().manual_seed(7)
    b, s, h = 2, 19, 3
    tensors = [torch.randn(b, s, hh, d, generator=g, dtype=torch.float64, requires_grad=True)
               for hh, d in ((h, 128), (h, 64), (h, 128), (1, 64), (h, 128))]
    dout = torch.randn(b, s, h, 128, generator=g, dtype=torch.float64)
    scale = 192 ** -0.5
    out, lse = oracle.prefill_forward(*tensors, scale)
    expected = torch.autograd.grad(out, tensors, dout)
    dq, dk_nope, dk_pe, dv = oracle.prefill_backward(dout, out.detach(), lse.detach(), *(t.detach() for t in tensors), scale)
    torch.testing.assert_close(dq, torch.cat(expected[:2], -1), atol=1e-12, rtol=1e-10)
    torch.testing.assert_close(dk_nope, expected[2], atol=1e-12, rtol=1e-10)
    torch.testing.assert_close(dk_pe, expected[3], atol=1e-12, rtol=1e-10)
    torch.testing.assert_close(dv, expected[4], atol=1e-12, rtol=1e-10)


def test_prefill_packed_equals_per_sequence_dense():
    seqlens = [5, 130, 1, 64]
    q_nope, q_pe, k_nope, k_pe, v, dout, cu = oracle.prefill_inputs(9, 0, 0, 2, dtype=torch.float32, seqlens=seqlens)
    scale = 192 ** -0.5
    out, lse = oracle.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, scale, cu)
    grads = oracle.prefill_backward(dout, out, lse, q_nope, q_pe, k_nope, k_pe, v, scale, cu)
    start = 0
    for n in seqlens:
        sl = slice(start, start + n)
        o, l = oracle.prefill_forward(*(t[None, sl] for t in (q_nope, q_pe, k_nope, k_pe, v)), scale)
        torch.testing.assert_close(out[sl], o[0])
        torch.testing.assert_close(lse[:, sl], l[0])
        g = oracle.prefill_backward(dout[None, sl], o, l, *(t[None, sl] for t in (q_nope, q_pe, k_nope, k_pe, v)), scale)
        for packed, dense in zip(grads, g):
            torch.testing.assert_close(packed[sl], dense[0])
        start += n


def test_absorbed_restatement_equals_prefill_restatement_in_degenerate_case():
    """k_nope[h] = v[h] = latent for every head turns the non-absorbed contract
    into the absorbed one (with C = 128)."""
    g = torch.Generator().manual_seed(3)
    b, s, h = 1, 23, 2
    latent = torch.randn(b, s, 128, generator=g, dtype=torch.float64)
    k_pe = torch.randn(b, s, 1, 64, generator=g, dtype=torch.float64)
    q_nope = torch.randn(b, s, h, 128, generator=g, dtype=torch.float64)
    q_pe = torch.randn(b, s, h, 64, generator=g, dtype=torch.float64)
    per_head = latent[:, :, None].expand(b, s, h, 128).contiguous()
    scale = 0.07
    o1, l1 = oracle.prefill_forward(q_nope, q_pe, per_head, k_pe, per_head, scale)
    o2, l2 = oracle.absorbed_forward(q_nope, q_pe, latent, k_pe[:, :, 0], scale, oracle.causal_mask(s))
    torch.testing.assert_close(o1, o2)
    torch.testing.assert_close(l1, l2)


def test_seeded_config_generators_are_stable():
    lengths = oracle.varlen_lengths()
    assert len(lengths) == 16 and all(512 <= n <= 32768 for n in lengths)
    assert lengths == oracle.varlen_lengths()
    q, cache, table, lens = oracle.decode_inputs(batch=4, heads=8, low=10, high=300)
    assert q.shape == (4, 1, 8, 576) and cache.shape[1:] == (64, 1, 576)
    used = torch.cat([table[i, : (int(lens[i]) + 63) // 64] for i in range(4)])
    assert used.unique().numel() == used.numel() == cache.shape[0]


@pytest.mark.parametrize("rows,keys", [((0, 50), (0, 50)), ((37, 90), (0, 31)), ((60, 90), (41, 77))])
def test_block_helpers_equal_the_dense_restatement(rows, keys):
    """`prefill_row_block` / `prefill_key_block` (used to check sequences of tens of thousands of tokens)
    are slices of the dense restatement."""
    q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(11, 2, 90, 3, dtype=torch.float32, dout_std=0.1)
    inputs = (q_nope, q_pe, k_nope, k_pe, v)
    scale = 192 ** -0.5
    out, lse = oracle.prefill_forward(*inputs, scale)
    dq, dk_nope, dk_pe, dv = oracle.prefill_backward(dout, out, lse, *inputs, scale)
    r0, r1 = rows
    b_out, b_lse, b_dq = oracle.prefill_row_block(*inputs, scale, rows, dout)
    torch.testing.assert_close(b_out, out[:, r0:r1], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(b_lse, lse[:, :, r0:r1], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(b_dq, dq[:, r0:r1], atol=1e-5, rtol=1e-5)
    k0, k1 = keys
    b_dk, b_dkpe, b_dv = oracle.prefill_key_block(dout, out, lse, *inputs, scale, keys)
    torch.testing.assert_close(b_dk, dk_nope[:, k0:k1], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(b_dkpe, dk_pe[:, k0:k1], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(b_dv, dv[:, k0:k1], atol=1e-5, rtol=1e-5)
