"""Causal D=128 grouped-query forward on the GPU against the PyTorch expression
the reference checks it with (benchmarks/flash_attention.py:68-75)."""

import pytest
import torch

from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu


# the reference's test shapes (benchmarks/flash_attention.py:42-47) plus ragged / longer ones
@pytest.mark.parametrize("b,t,hq,hkv", [(1, 64, 2, 2), (2, 64, 4, 2), (1, 128, 4, 1), (1, 256, 8, 8),
                                        (1, 100, 4, 2), (2, 640, 8, 2), (1, 1024, 2, 1)])
def test_forward_matches_pytorch_expression(gpu, b, t, hq, hkv):
    from dscuda_b200 import mla
    generator = torch.Generator().manual_seed(t + hq)
    query = (torch.randn(b, t, hq, 128, generator=generator) * .5).bfloat16()
    key = (torch.randn(b, t, hkv, 128, generator=generator) * .5).bfloat16()
    value = (torch.randn(b, t, hkv, 128, generator=generator) * .5).bfloat16()
    scale = 128 ** -.5
    out, lse = mla.flash_forward(query.to(gpu), key.to(gpu), value.to(gpu), scale)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    ref_out, ref_lse = oracle.flash_forward(query, key, value, scale)
    # reference tolerances (benchmarks/flash_attention.py:112-113)
    torch.testing.assert_close(out.cpu().float(), ref_out.bfloat16().float(), atol=1e-2, rtol=1e-2)
    torch.testing.assert_close(lse.cpu(), ref_lse, atol=1e-4, rtol=1e-5)


def test_rejects_bad_arguments(gpu):
    from dscuda_b200 import mla
    q = torch.zeros(1, 64, 3, 128, device=gpu, dtype=torch.bfloat16)
    kv = torch.zeros(1, 64, 2, 128, device=gpu, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="divisible"):
        mla.flash_forward(q, kv, kv, 0.1)
    q64 = torch.zeros(1, 64, 2, 64, device=gpu, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="head_size 128"):
        mla.flash_forward(q64, q64, q64, 0.1)
