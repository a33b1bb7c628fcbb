"""Rotary embedding on the GPU against the oracle's rope() evaluated in fp32 on the same
bf16 inputs.  The kernel does the same unfused fp32 arithmetic on double-precision angles, so
the outputs agree bit for bit except where the device's and the host's cos/sin differ in the
last place of their double result; the test allows one bf16 ulp on at most 1e-4 of the elements."""

import pytest
import torch

from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu


def reference(x, positions):
    return oracle.rope(x.float(), positions).bfloat16()


def check(out, ref):
    diff = (out.float() - ref.float()).abs()
    assert float((diff > 0).float().mean()) <= 1e-4
    assert bool((diff <= ref.float().abs() * 2 ** -7 + 1e-30).all())


def draw(seed, *shape):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)).bfloat16()


@pytest.mark.parametrize("b,s,h", [(1, 1, 1), (2, 300, 3), (1, 2048, 16)])
def test_dense_positions(gpu, b, s, h):
    from dscuda_b200 import mla
    q_pe, k_pe = draw(1, b, s, h, 64), draw(2, b, s, 1, 64)
    q, k = q_pe.to(gpu), k_pe.to(gpu)
    mla.rope_apply(q, k)
    torch.cuda.synchronize()
    positions = torch.arange(s)
    check(q.cpu(), torch.stack([reference(q_pe[i], positions) for i in range(b)]))
    check(k.cpu(), torch.stack([reference(k_pe[i], positions) for i in range(b)]))


def test_explicit_positions_and_single_tensors(gpu):
    from dscuda_b200 import mla
    rows, h = 777, 5
    positions = torch.randint(0, 32768, (rows,), generator=torch.Generator().manual_seed(3), dtype=torch.int32)
    q_pe, k_pe = draw(4, rows, h, 64), draw(5, rows, 1, 64)
    q, k = q_pe.to(gpu), k_pe.to(gpu)
    mla.rope_apply(q, None, positions.to(gpu))
    mla.rope_apply(None, k, positions.to(gpu))
    torch.cuda.synchronize()
    check(q.cpu(), reference(q_pe, positions))
    check(k.cpu(), reference(k_pe, positions))
    with pytest.raises(ValueError):
        mla.rope_apply(q_pe.to(gpu))            # packed layout without positions


def test_rotated_inputs_feed_the_attention_kernel(gpu):
    """prefill_inputs() rotates on the host; rotating raw draws on the device gives the same attention output."""
    from dscuda_b200 import mla
    b, s, h = 1, 257, 2
    g = torch.Generator().manual_seed(11)
    raw = [torch.randn(b, s, *tail, generator=g).bfloat16() for tail in ((h, 128), (h, 64), (h, 128), (1, 64), (h, 128))]
    host = [t.clone() for t in raw]
    positions = torch.arange(s)
    host[1] = reference(raw[1][0], positions)[None]
    host[3] = reference(raw[3][0], positions)[None]
    device = [t.to(gpu) for t in raw]
    mla.rope_apply(device[1], device[3])
    out, lse = mla.prefill_forward(*device, 192 ** -0.5)
    ref_out, ref_lse = oracle.prefill_forward(*host, 192 ** -0.5)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    assert float((out.float().cpu() - ref_out).abs().max()) <= 1e-2 * float(ref_out.abs().max())
    assert float((lse.cpu() - ref_lse).abs().max()) <= 1e-3
