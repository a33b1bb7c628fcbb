"""Parity at the sizes the benchmark quotes, through the C ABI, against the CPU oracle.

* training step length (S=8192): every gradient of whole heads;
* the decode benchmark itself (batch 64, lengths 1589..32273, 17 718 permuted pages, splits 8): every sequence;
* the packed long-context lengths (up to 26 465 tokens): the last query rows and the first key rows
  of the two longest sequences, through the oracle's block helpers.

Bars: O max|err| <= 1e-2 max|ref|, LSE within 1e-3, gradient relative L2 <= 1e-2.
"""

import pytest
import torch

from conftest import max_err_ratio, rel_l2
from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu

SCALE = 192 ** -0.5


def test_training_length_all_gradients(gpu):
    """B=1, S=8192, two heads drawn like the training configuration (seed 2, dO ~ N(0, 0.1), rotary
    embedding applied): O, LSE, dQ, dK_nope, dV of both heads and the head-summed dK_pe."""
    from dscuda_b200 import mla
    seq, heads = 8192, 2
    q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(2, 1, seq, heads, dout_std=0.1)
    device = [t.to(gpu) for t in (q_nope, q_pe, k_nope, k_pe, v)]
    out, lse = mla.prefill_forward(*device, SCALE)
    grads = mla.prefill_backward(dout.to(gpu), out, lse, *device, SCALE)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    out, lse = out.cpu(), lse.cpu()
    dq, dk_nope, dk_pe, dv = (g.cpu().float() for g in grads)
    dk_pe_reference = torch.zeros(1, seq, 1, 64)
    for h in range(heads):          # one head at a time: the S x S fp32 matrices of a head are 268 MB each
        one = [t[:, :, h:h + 1].contiguous() for t in (q_nope, q_pe, k_nope)] + [k_pe, v[:, :, h:h + 1].contiguous()]
        ref_out, ref_lse = oracle.prefill_forward(*one, SCALE)
        assert max_err_ratio(out[:, :, h:h + 1].float(), ref_out) <= 1e-2
        assert float((lse[:, h:h + 1] - ref_lse).abs().max()) <= 1e-3
        ref = oracle.prefill_backward(dout[:, :, h:h + 1].contiguous(), out[:, :, h:h + 1].contiguous(), lse[:, h:h + 1].contiguous(),
                                      *one, SCALE)
        assert rel_l2(dq[:, :, h:h + 1], ref[0]) <= 1e-2, f"dq head {h}"
        assert rel_l2(dk_nope[:, :, h:h + 1], ref[1]) <= 1e-2, f"dk_nope head {h}"
        assert rel_l2(dv[:, :, h:h + 1], ref[3]) <= 1e-2, f"dv head {h}"
        dk_pe_reference += ref[2]
    assert rel_l2(dk_pe, dk_pe_reference) <= 1e-2, "dk_pe"


def test_decode_benchmark_problem_every_sequence(gpu):
    """The decode benchmark's own inputs (seed 3) at its own `splits`: every one of the 64 sequences,
    whatever CTA-pair range boundaries cut it, against the oracle."""
    from dscuda_b200 import mla
    query, cache, table, lengths = oracle.decode_inputs(seed=3, batch=64, heads=128)
    assert int(lengths.sum()) == 1131680 and cache.shape[0] == 17718
    out, lse = mla.mla_decode(query.to(gpu), cache.to(gpu), table.to(gpu), lengths.to(gpu), SCALE, splits=8)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    out, lse = out.cpu().float(), lse.cpu()
    for first in range(0, 64, 8):
        group = slice(first, first + 8)
        ref_out, ref_lse = oracle.paged_decode(query[group], cache, table[group], lengths[group], SCALE)
        for b in range(8):
            assert max_err_ratio(out[first + b], ref_out[b]) <= 1e-2, f"sequence {first + b} ({int(lengths[first + b])} tokens)"
        assert float((lse[group] - ref_lse).abs().max()) <= 1e-3, f"sequences {first}..{first + 7}"


def test_long_context_longest_sequences(gpu):
    """The 16 packed lengths of the long-context configuration (seed 4, 121 320 tokens), two heads:
    for the two longest sequences (26 465 and 25 869 tokens) the last 256 query rows (O, LSE, dQ) and
    the first 128 key rows (dK_nope, dK_pe, dV) against the oracle's block helpers."""
    from dscuda_b200 import mla
    lengths = oracle.varlen_lengths()
    heads = 2
    q_nope, q_pe, k_nope, k_pe, v, dout, cu = oracle.prefill_inputs(4, 0, 0, heads, dout_std=0.1, seqlens=lengths)
    device = [t.to(gpu) for t in (q_nope, q_pe, k_nope, k_pe, v)]
    out, lse = mla.prefill_forward(*device, SCALE, cu.to(gpu), max(lengths))
    grads = mla.prefill_backward(dout.to(gpu), out, lse, *device, SCALE, cu.to(gpu), max(lengths))
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    out, lse = out.cpu(), lse.cpu()
    dq, dk_nope, dk_pe, dv = (g.cpu().float() for g in grads)
    starts = [int(x) for x in cu]
    for index in sorted(range(len(lengths)), key=lambda i: -lengths[i])[:2]:
        a, b = starts[index], starts[index + 1]
        n = b - a
        assert n >= 25000
        dense = [t[a:b][None] for t in (q_nope, q_pe, k_nope, k_pe, v)]
        ref_out, ref_lse, ref_dq = oracle.prefill_row_block(*dense, SCALE, (n - 256, n), dout[a:b][None])
        assert max_err_ratio(out[b - 256:b].float(), ref_out[0]) <= 1e-2
        assert float((lse[:, b - 256:b] - ref_lse[0]).abs().max()) <= 1e-3
        assert rel_l2(dq[b - 256:b], ref_dq[0]) <= 1e-2, "dq"
        ref_dk, ref_dkpe, ref_dv = oracle.prefill_key_block(dout[a:b][None], out[a:b][None], lse[:, a:b][None], *dense, SCALE, (0, 128))
        assert rel_l2(dk_nope[a:a + 128], ref_dk[0]) <= 1e-2, "dk_nope"
        assert rel_l2(dk_pe[a:a + 128], ref_dkpe[0]) <= 1e-2, "dk_pe"
        assert rel_l2(dv[a:a + 128], ref_dv[0]) <= 1e-2, "dv"
