"""Non-absorbed causal prefill forward on the GPU, through the C ABI, against the
CPU oracle and the reference-generated fixtures."""

import pytest
import torch

from conftest import load_golden, max_err_ratio
from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu

SCALE = 192 ** -0.5


def run_forward(gpu, tensors, scale, cu=None, max_seqlen=None):
    from dscuda_b200 import mla
    device = [t.to(gpu) for t in tensors]
    cu_device = None if cu is None else cu.to(gpu)
    out, lse = mla.prefill_forward(*device, scale, cu_device, max_seqlen)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    return out.cpu(), lse.cpu()


def check_forward(out, lse, ref_out, ref_lse):
    # forward bar: max|err| <= 1e-2 * max|ref|, LSE within 1e-3
    assert max_err_ratio(out.float(), ref_out) <= 1e-2
    assert float((lse - ref_lse).abs().max()) <= 1e-3


@pytest.mark.parametrize("b,s,h", [(1, 1, 1), (2, 17, 3), (1, 65, 4), (1, 128, 1), (1, 129, 2), (2, 256, 2),
                                   (1, 300, 3), (1, 520, 2), (1, 1024, 1)])
def test_dense_matches_oracle(gpu, b, s, h):
    q_nope, q_pe, k_nope, k_pe, v, _ = oracle.prefill_inputs(100 + s, b, s, h)
    out, lse = run_forward(gpu, (q_nope, q_pe, k_nope, k_pe, v), SCALE)
    ref_out, ref_lse = oracle.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, SCALE)
    check_forward(out, lse, ref_out, ref_lse)


@pytest.mark.parametrize("name", ["b2_s37_h3", "b1_s130_h2"])
def test_matches_reference_embedding_fixture(gpu, name):
    g = load_golden(f"prefill_embed_{name}")
    tensors = (g["q_nope"], g["q_pe"], g["k_nope"], g["k_pe"], g["v"])
    out, lse = run_forward(gpu, tensors, g["scale"])
    # reference tolerances for forward outputs (benchmarks/mla.py:103-105)
    torch.testing.assert_close(out.float(), g["out"].float(), atol=8e-3, rtol=8e-3)
    torch.testing.assert_close(lse, g["lse"], atol=1e-4, rtol=1e-4)


def test_config1_shape(gpu):
    """B=1, S=256, H=16, seed 0 (the CPU-runnable configuration)."""
    q_nope, q_pe, k_nope, k_pe, v, _ = oracle.prefill_inputs(0, 1, 256, 16)
    out, lse = run_forward(gpu, (q_nope, q_pe, k_nope, k_pe, v), SCALE)
    ref_out, ref_lse = oracle.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, SCALE)
    check_forward(out, lse, ref_out, ref_lse)


@pytest.mark.parametrize("seqlens", [[5, 130, 1, 64], [256, 257, 255], [700]])
def test_packed_matches_oracle(gpu, seqlens):
    q_nope, q_pe, k_nope, k_pe, v, _, cu = oracle.prefill_inputs(41, 0, 0, 2, seqlens=seqlens)
    out, lse = run_forward(gpu, (q_nope, q_pe, k_nope, k_pe, v), SCALE, cu, max(seqlens))
    ref_out, ref_lse = oracle.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, SCALE, cu)
    check_forward(out, lse, ref_out, ref_lse)


def test_is_deterministic(gpu):
    q_nope, q_pe, k_nope, k_pe, v, _ = oracle.prefill_inputs(77, 1, 384, 2)
    first = run_forward(gpu, (q_nope, q_pe, k_nope, k_pe, v), SCALE)
    second = run_forward(gpu, (q_nope, q_pe, k_nope, k_pe, v), SCALE)
    assert torch.equal(first[0], second[0]) and torch.equal(first[1], second[1])


def test_full_size_config2_spot_check(gpu):
    """B=4, S=4096, H=128 (the prefill-forward configuration), generated on the
    device to keep host time bounded; a few (batch, head) pairs are checked
    against the oracle, and every output row through the property that a
    softmax-weighted mean of V lies inside V's range."""
    from dscuda_b200 import mla
    b, s, h = 4, 4096, 128
    generator = torch.Generator(device=gpu).manual_seed(1)

    def draw(*shape):
        return torch.randn(*shape, device=gpu, generator=generator, dtype=torch.float32).bfloat16()

    q_nope, q_pe, k_nope, k_pe, v = draw(b, s, h, 128), draw(b, s, h, 64), draw(b, s, h, 128), draw(b, s, 1, 64), draw(b, s, h, 128)
    out, lse = mla.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, SCALE)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    assert bool(torch.isfinite(out.float()).all()) and bool(torch.isfinite(lse).all())
    assert float(out.float().abs().max()) <= float(v.float().abs().max()) * 1.01
    for bi, hi in ((0, 0), (3, 127), (1, 64)):
        tensors = [t[bi:bi + 1, :, hi:hi + 1].cpu().contiguous() for t in (q_nope, q_pe, k_nope)] + \
                  [k_pe[bi:bi + 1].cpu().contiguous(), v[bi:bi + 1, :, hi:hi + 1].cpu().contiguous()]
        ref_out, ref_lse = oracle.prefill_forward(*tensors, SCALE)
        check_forward(out[bi:bi + 1, :, hi:hi + 1].cpu(), lse[bi:bi + 1, hi:hi + 1].cpu(), ref_out, ref_lse)
