"""Every entry point only launches on the caller's stream, so a call can be captured in a CUDA
graph and replayed on new data in the same buffers - the way the reference's timing harness runs
its operators (benchmarks/common.py:68-76)."""

import pytest
import torch

from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu

SCALE = 192 ** -0.5


def capture(fn):
    fn()                                     # first call outside the capture (attribute set-up, entry-point lookup)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph


def test_prefill_forward_and_backward_replay(gpu):
    from dscuda_b200 import mla
    b, s, h = 1, 200, 2
    first = [t.to(gpu) for t in oracle.prefill_inputs(41, b, s, h, dout_std=0.1)]
    second = [t.to(gpu) for t in oracle.prefill_inputs(42, b, s, h, dout_std=0.1)]
    x = [t.clone() for t in first]
    out, lse = torch.empty_like(x[4]), torch.empty(b, h, s, device=gpu)
    workspace = mla.prefill_backward_workspace(b, s, b * s, h, gpu)
    grads = (torch.empty(b, s, h, 192, device=gpu, dtype=torch.bfloat16), torch.empty_like(x[2]), torch.empty_like(x[3]), torch.empty_like(x[4]))

    def step():
        mla.prefill_forward(*x[:5], SCALE, output=out, lse=lse)
        mla.prefill_backward(x[5], out, lse, *x[:5], SCALE, workspace=workspace, grads=grads)

    graph = capture(step)
    for buffer, value in zip(x, second):
        buffer.copy_(value)
    graph.replay()
    torch.cuda.synchronize()
    replayed = [t.clone() for t in (out, lse, *grads)]
    step()                                   # the same data, launched directly
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    for a, b_ in zip(replayed, (out, lse, *grads)):
        assert torch.equal(a, b_)
    ref_out, ref_lse = oracle.prefill_forward(*[t.cpu() for t in second[:5]], SCALE)
    assert float((replayed[0].float().cpu() - ref_out).abs().max()) <= 1e-2 * float(ref_out.abs().max())


def test_decode_append_and_rope_replay(gpu):
    from dscuda_b200 import mla
    query, cache, table, lengths = (t.to(gpu) for t in oracle.decode_inputs(seed=5, batch=3, heads=4, low=60, high=200))
    workspace = mla.decode_workspace(3, 4, 4, 512, gpu)
    out = torch.empty(3, 1, 4, 512, device=gpu, dtype=torch.bfloat16)
    lse = torch.empty(3, 4, 1, device=gpu)
    new_latent = torch.randn(3, 1, 512, device=gpu).bfloat16()
    new_rope = torch.randn(3, 1, 64, device=gpu).bfloat16()
    positions = (lengths - 1).contiguous()                      # overwrite the last cached token of every sequence
    rope_rows = positions.clone()

    def step():
        mla.rope_apply(None, new_rope.view(3, 1, 64), rope_rows)
        mla.cache_append(cache, new_latent, new_rope, table, positions)
        mla.mla_decode(query, cache, table, lengths, 576 ** -0.5, 4, workspace, out, lse)

    graph = capture(step)
    new_latent.copy_(torch.randn(3, 1, 512, device=gpu).bfloat16())
    new_rope.copy_(torch.randn(3, 1, 64, device=gpu).bfloat16())
    kept_rope = new_rope.clone()
    graph.replay()
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    expected_rope = oracle.rope(kept_rope.float().cpu().view(3, 1, 64), positions.cpu()).bfloat16()
    assert float((new_rope.float().cpu().view(3, 1, 64) - expected_rope.float()).abs().max()) <= 2 ** -7 * float(expected_rope.float().abs().max())
    ref_out, ref_lse = oracle.paged_decode(query.float().cpu(), cache.float().cpu(), table.cpu(), lengths.cpu(), 576 ** -0.5)
    assert float((out.float().cpu() - ref_out).abs().max()) <= 1e-2 * float(ref_out.abs().max())
    assert float((lse.cpu() - ref_lse).abs().max()) <= 1e-3
    for b in range(3):                                           # the appended row is what the decode saw
        page = int(table[b, int(positions[b]) // 64])
        row = cache[page, int(positions[b]) % 64, 0]
        assert torch.equal(row[:512], new_latent[b, 0]) and torch.equal(row[512:], new_rope[b, 0])
