"""Non-absorbed causal MLA backward on the GPU, through the C ABI, against the CPU
oracle (closed form, fp32 on the same bf16 inputs) and the reference-generated
fixtures.  Bar: relative L2 error <= 1e-2 per gradient."""

import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu

SCALE = 192 ** -0.5
NAMES = ("dq", "dk_nope", "dk_pe", "dv")


def run_backward(gpu, tensors, dout, scale, cu=None, max_seqlen=None):
    from dscuda_b200 import mla
    device = [t.to(gpu) for t in tensors]
    cu_device = None if cu is None else cu.to(gpu)
    out, lse = mla.prefill_forward(*device, scale, cu_device, max_seqlen)
    grads = mla.prefill_backward(dout.to(gpu), out, lse, *device, scale, cu_device, max_seqlen)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    return out.cpu(), lse.cpu(), tuple(g.cpu() for g in grads)


def check_grads(grads, reference, bar=1e-2):
    for name, got, ref in zip(NAMES, grads, reference):
        assert got.shape == ref.shape, name
        assert bool(torch.isfinite(got.float()).all()), name
        error = rel_l2(got.float(), ref)
        assert error <= bar, f"{name}: rel-L2 {error:.3e}"


@pytest.mark.parametrize("b,s,h", [(1, 1, 1), (2, 17, 3), (1, 64, 1), (1, 65, 4), (1, 128, 2), (1, 129, 2), (2, 256, 2),
                                   (1, 300, 3), (1, 520, 2), (1, 1100, 1)])
def test_dense_matches_oracle(gpu, b, s, h):
    q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(200 + s, b, s, h, dout_std=0.1)
    tensors = (q_nope, q_pe, k_nope, k_pe, v)
    out, lse, grads = run_backward(gpu, tensors, dout, SCALE)
    reference = oracle.prefill_backward(dout, out, lse, *tensors, SCALE)
    if s == 1:
        # one key: dS is exactly zero, so dq and dk vanish; compare absolutely
        assert float(grads[0].float().abs().max()) <= 1e-3 and float(grads[1].float().abs().max()) <= 1e-3
        assert rel_l2(grads[3].float(), reference[3]) <= 1e-2
        return
    check_grads(grads, reference)


@pytest.mark.parametrize("name", ["b2_s37_h3", "b1_s130_h2"])
def test_matches_reference_embedding_fixture(gpu, name):
    g = load_golden(f"prefill_embed_{name}")
    tensors = (g["q_nope"], g["q_pe"], g["k_nope"], g["k_pe"], g["v"])
    _, _, grads = run_backward(gpu, tensors, g["dout"], g["scale"])
    reference = (g["dq"].float(), g["dk_nope"].float(), g["dk_pe_heads"].float().sum(2, keepdim=True), g["dv"].float())
    check_grads(grads, reference)


def test_config1_shape(gpu):
    q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(0, 1, 256, 16)
    tensors = (q_nope, q_pe, k_nope, k_pe, v)
    out, lse, grads = run_backward(gpu, tensors, dout, SCALE)
    check_grads(grads, oracle.prefill_backward(dout, out, lse, *tensors, SCALE))


@pytest.mark.parametrize("seqlens", [[5, 130, 1, 64], [256, 257, 255], [700]])
def test_packed_matches_oracle(gpu, seqlens):
    q_nope, q_pe, k_nope, k_pe, v, dout, cu = oracle.prefill_inputs(43, 0, 0, 2, dout_std=0.1, seqlens=seqlens)
    tensors = (q_nope, q_pe, k_nope, k_pe, v)
    out, lse, grads = run_backward(gpu, tensors, dout, SCALE, cu, max(seqlens))
    check_grads(grads, oracle.prefill_backward(dout, out, lse, *tensors, SCALE, cu))


def test_gradients_are_overwritten_not_accumulated(gpu):
    """Two calls on the same buffers give bit-identical results, dk_pe (a sum over heads in a fixed order) included."""
    from dscuda_b200 import mla
    q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(5, 1, 200, 3, dout_std=0.1)
    device = [t.to(gpu) for t in (q_nope, q_pe, k_nope, k_pe, v)]
    out, lse = mla.prefill_forward(*device, SCALE)
    workspace = mla.prefill_backward_workspace(1, 200, 200, 3, gpu)
    grads = mla.prefill_backward(dout.to(gpu), out, lse, *device, SCALE, workspace=workspace)
    first = [g.clone() for g in grads]
    mla.prefill_backward(dout.to(gpu), out, lse, *device, SCALE, workspace=workspace, grads=grads)
    torch.cuda.synchronize()
    for name, a, b in zip(NAMES, first, grads):
        assert torch.equal(a, b), name
    # the fp32 head-sum of dk_pe sits at the start of the workspace
    acc = workspace[: 200 * 64 * 4].view(torch.float32).reshape(200, 64)
    torch.testing.assert_close(acc.bfloat16(), grads[2].reshape(200, 64))


def test_linearity_in_dout_at_training_size(gpu):
    """S=8192 (the training configuration's length) on a few heads: gradients are
    linear in dO, and one (batch, head) slice is checked against the oracle."""
    from dscuda_b200 import mla
    b, s, h = 1, 8192, 2
    generator = torch.Generator(device=gpu).manual_seed(2)

    def draw(*shape, std=1.0):
        return (torch.randn(*shape, device=gpu, generator=generator, dtype=torch.float32) * std).bfloat16()

    q_nope, q_pe, k_nope, k_pe, v = draw(b, s, h, 128), draw(b, s, h, 64), draw(b, s, h, 128), draw(b, s, 1, 64), draw(b, s, h, 128)
    dout = draw(b, s, h, 128, std=0.1)
    out, lse = mla.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, SCALE)
    g1 = [g.clone() for g in mla.prefill_backward(dout, out, lse, q_nope, q_pe, k_nope, k_pe, v, SCALE)]
    g2 = mla.prefill_backward((dout.float() * 2).bfloat16(), out, lse, q_nope, q_pe, k_nope, k_pe, v, SCALE)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    for name, a, c in zip(NAMES, g1, g2):
        assert rel_l2(c.float().cpu(), 2 * a.float().cpu()) <= 1e-2, name
    # oracle check of head 0 on the first 2048 tokens is not a slice of the full problem for dk/dv
    # (later queries contribute), so check dq only there, and everything on a full single head at S=2048
    tensors = [t[:, :2048, :1].cpu().contiguous() for t in (q_nope, q_pe, k_nope)] + [k_pe[:, :2048].cpu().contiguous(),
                                                                                    v[:, :2048, :1].cpu().contiguous()]
    ref = oracle.prefill_backward(dout[:, :2048, :1].cpu().contiguous(), out[:, :2048, :1].cpu().contiguous(),
                                  lse[:, :1, :2048].cpu().contiguous(), *tensors, SCALE)
    assert rel_l2(g1[0][:, :2048, :1].float().cpu(), ref[0]) <= 1e-2


def test_long_context_packed_lengths(gpu):
    """The 16 packed sequence lengths of the long-context configuration (log-uniform
    in [512, 32768], seed 4; 121 320 tokens) on 2 heads: finite outputs, each short
    sequence checked against the oracle, and the dk_pe head-sum equal to the sum of
    two single-head runs (what a head-sharded multi-GPU run adds up)."""
    from dscuda_b200 import mla
    lengths = oracle.varlen_lengths()
    total = sum(lengths)
    heads = 2
    generator = torch.Generator(device=gpu).manual_seed(4)

    def draw(*shape, std=1.0):
        return (torch.randn(*shape, device=gpu, generator=generator, dtype=torch.float32) * std).bfloat16()

    q_nope, q_pe, k_nope, k_pe, v = draw(total, heads, 128), draw(total, heads, 64), draw(total, heads, 128), draw(total, 1, 64), draw(total, heads, 128)
    dout = draw(total, heads, 128, std=0.1)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=gpu)
    out, lse = mla.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, SCALE, cu, max(lengths))
    grads = mla.prefill_backward(dout, out, lse, q_nope, q_pe, k_nope, k_pe, v, SCALE, cu, max(lengths))
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    for tensor in (out, lse, *grads):
        assert bool(torch.isfinite(tensor.float()).all())
    # the three shortest sequences against the oracle (each is an independent causal problem)
    starts = [0] + list(torch.tensor(lengths).cumsum(0))
    for index in sorted(range(len(lengths)), key=lambda i: lengths[i])[:3]:
        a, b = int(starts[index]), int(starts[index + 1])
        cpu = [t[a:b][None].cpu().contiguous() for t in (q_nope, q_pe, k_nope, k_pe, v)]
        ref_out, ref_lse = oracle.prefill_forward(*cpu, SCALE)
        assert float((out[a:b].float().cpu() - ref_out[0]).abs().max()) <= 1e-2 * float(ref_out.abs().max())
        assert float((lse[:, a:b].cpu() - ref_lse[0]).abs().max()) <= 1e-3
        reference = oracle.prefill_backward(dout[a:b][None].cpu(), out[a:b][None].cpu(), lse[:, a:b][None].cpu(), *cpu, SCALE)
        check_grads([g[a:b][None].cpu() for g in grads], reference)
    # head sharding: one head at a time gives the same per-head gradients and dk_pe partial sums that add up
    partial_sum = torch.zeros(total, 64, device=gpu)
    for h in range(heads):
        sl = [t[:, h:h + 1].contiguous() for t in (q_nope, q_pe, k_nope)] + [k_pe, v[:, h:h + 1].contiguous()]
        o1, l1 = mla.prefill_forward(*sl, SCALE, cu, max(lengths))
        workspace = mla.prefill_backward_workspace(len(lengths), max(lengths), total, 1, gpu)
        g1 = mla.prefill_backward(dout[:, h:h + 1].contiguous(), o1, l1, *sl, SCALE, cu, max(lengths), workspace=workspace)
        torch.cuda.synchronize()
        assert torch.equal(o1, out[:, h:h + 1]) and torch.equal(g1[0], grads[0][:, h:h + 1]) and torch.equal(g1[3], grads[3][:, h:h + 1])
        partial_sum += workspace[: total * 64 * 4].view(torch.float32).reshape(total, 64)
    assert rel_l2(partial_sum.cpu(), grads[2].float().reshape(total, 64).cpu()) <= 5e-3


@pytest.mark.parametrize("limit_heads", [0, 1, 2])
def test_dense_backward_paths_agree(gpu, limit_heads):
    """Dense batches: dQ from the stored dS^T (all heads in one group, or group after group when the
    scratch limit holds fewer heads) and dQ from the recomputing kernel (limit 0) give the same
    gradients as the oracle, and the launch count follows the grouping."""
    from dscuda_b200 import mla
    b, s, h = 2, 333, 3
    q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(11, b, s, h, dout_std=0.1)
    tensors = (q_nope, q_pe, k_nope, k_pe, v)
    device = [t.to(gpu) for t in tensors]
    out, lse = mla.prefill_forward(*device, SCALE)
    tiles = (s + 127) // 128
    per_head = b * (tiles * tiles + tiles) * 16384
    previous = mla.prefill_backward_scratch_limit(limit_heads * per_head)
    try:
        expected_launches = 4 if limit_heads == 0 else 2 + 2 * ((h + limit_heads - 1) // limit_heads)
        assert mla.prefill_backward_launches(b, s, b * s, h) == expected_launches
        grads = mla.prefill_backward(dout.to(gpu), out, lse, *device, SCALE)
        torch.cuda.synchronize()
        assert mla.device_status() == 0
    finally:
        mla.prefill_backward_scratch_limit(previous)
    assert mla.prefill_backward_scratch_limit() == previous
    check_grads(tuple(g.cpu() for g in grads), oracle.prefill_backward(dout, out.cpu(), lse.cpu(), *tensors, SCALE))


@pytest.mark.parametrize("limit", [None, 0, 1 << 20])
def test_packed_backward_routes_agree(gpu, limit):
    """Packed batches: dQ streamed from the stored dS^T (default limit: one group; 1 MiB: one head per group, the
    workspace sized by the bound that needs no lengths) and the recomputing kernel (limit 0) against the oracle."""
    from dscuda_b200 import mla
    seqlens = [70, 1, 333, 128, 200]
    heads = 3
    total = sum(seqlens)
    q_nope, q_pe, k_nope, k_pe, v, dout, cu = oracle.prefill_inputs(17, 0, 0, heads, dout_std=0.1, seqlens=seqlens)
    tensors = (q_nope, q_pe, k_nope, k_pe, v)
    previous = mla.prefill_backward_scratch_limit(-1 if limit is None else limit)
    try:
        launches = mla.prefill_backward_launches(len(seqlens), max(seqlens), total, heads, packed=True)
        assert launches == {None: 4, 0: 4, 1 << 20: 8}[limit]
        out, lse, grads = run_backward(gpu, tensors, dout, SCALE, cu, max(seqlens))
    finally:
        mla.prefill_backward_scratch_limit(previous)
    check_grads(grads, oracle.prefill_backward(dout, out, lse, *tensors, SCALE, cu))
