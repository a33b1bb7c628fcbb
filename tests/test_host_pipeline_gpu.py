"""Host staging pipeline: steps fed from pinned host memory through two device buffer sets
give the same outputs as steps run on tensors that already live on the device."""

import pytest
import torch

from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu

SCALE = 192 ** -0.5
KEYS = ("q_nope", "q_pe", "k_nope", "k_pe", "v")


def host_step(seed, b, s, h):
    q_nope, q_pe, k_nope, k_pe, v, _ = oracle.prefill_inputs(seed, b, s, h)
    return {k: t.contiguous().pin_memory() for k, t in zip(KEYS, (q_nope, q_pe, k_nope, k_pe, v))}


def test_pipelined_steps_match_direct_calls(gpu):
    from dscuda_b200 import mla
    from dscuda_b200.host_pipeline import HostPipeline

    steps = [host_step(300 + i, 1, 200, 2) for i in range(5)]      # more steps than buffer sets
    direct = []
    for step in steps:
        out, lse = mla.prefill_forward(*(step[k].to(gpu) for k in KEYS), SCALE)
        direct.append((out.cpu(), lse.cpu()))

    pipe = HostPipeline({k: steps[0][k].to(gpu) for k in KEYS}, gpu)
    assert pipe.bytes_per_step == sum(t.numel() * t.element_size() for t in steps[0].values())
    results = []
    pipe.stage(steps[0])
    for i in range(len(steps)):
        if i + 1 < len(steps):
            pipe.stage(steps[i + 1])
        x = pipe.acquire()
        out, lse = mla.prefill_forward(*(x[k] for k in KEYS), SCALE)
        pipe.release()
        results.append((out, lse))
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    for (out, lse), (ref_out, ref_lse) in zip(results, direct):
        assert torch.equal(out.cpu(), ref_out)
        assert torch.equal(lse.cpu(), ref_lse)


def test_misuse_is_reported(gpu):
    from dscuda_b200.host_pipeline import HostPipeline

    step = host_step(7, 1, 16, 1)
    pipe = HostPipeline({k: step[k].to(gpu) for k in KEYS}, gpu)
    with pytest.raises(RuntimeError):
        pipe.acquire()                       # nothing staged
    pipe.stage(step)
    pipe.stage(step)
    with pytest.raises(RuntimeError):
        pipe.stage(step)                     # both sets in use
    pipe.acquire()
    with pytest.raises(RuntimeError):
        pipe.acquire()                       # previous step not released
    pipe.release()
    with pytest.raises(RuntimeError):
        pipe.release()
    unpinned = {k: t.clone() for k, t in step.items()}
    with pytest.raises(ValueError):
        pipe.stage(unpinned)
    torch.cuda.synchronize()
