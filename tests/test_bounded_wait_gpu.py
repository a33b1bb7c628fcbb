"""The bounded in-kernel wait giving up, exercised without any fault: a test-only kernel
(tests/csrc/bounded_wait_probe.cu, built as build/libdscuda_test_probes.so) calls the product's
own `mbar_wait_limit` with a limit of about a millisecond on a barrier that nobody arrives on.
The launch must end by itself with status 1 and its tensor memory released, a launch made while
the status is set must leave at once, and after a reset both the probe and the real kernels run
normally in the same context."""

import ctypes
import pathlib

import pytest
import torch

from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu

ROOT = pathlib.Path(__file__).resolve().parents[1]


def probe_library():
    path = ROOT / "build" / "libdscuda_test_probes.so"
    assert path.exists(), f"{path} is missing: run `python -m dscuda_b200.build`"
    lib = ctypes.CDLL(str(path))
    lib.dscuda_test_bounded_wait.argtypes = [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
    lib.dscuda_test_bounded_wait.restype = ctypes.c_int
    return lib


def run_probe(lib, limit_cycles, arrive, reset_first):
    out = (ctypes.c_int * 4)()
    assert lib.dscuda_test_bounded_wait(limit_cycles, arrive, reset_first, out) == 0, "CUDA error in the probe"
    return dict(gave_up=out[0], left_at_entry=out[1], tmem_released=out[2], status=out[3])


def test_wait_runs_out_cleanly_and_the_context_stays_usable(gpu):
    from dscuda_b200 import mla
    lib = probe_library()
    # an arrival completes the wait: status stays 0
    assert run_probe(lib, 2_000_000, arrive=1, reset_first=1) == dict(gave_up=0, left_at_entry=0, tmem_released=32, status=0)
    # nobody arrives: the wait gives up after ~1 ms, the CTA releases its tensor memory, status 1
    assert run_probe(lib, 2_000_000, arrive=0, reset_first=0) == dict(gave_up=1, left_at_entry=0, tmem_released=32, status=1)
    # while the status is set, a launch leaves at entry and touches nothing
    assert run_probe(lib, 2_000_000, arrive=1, reset_first=0) == dict(gave_up=0, left_at_entry=1, tmem_released=0, status=1)
    # reset: back to normal
    assert run_probe(lib, 2_000_000, arrive=1, reset_first=1) == dict(gave_up=0, left_at_entry=0, tmem_released=32, status=0)
    # the real kernels still work in this context (tensor memory was not leaked)
    scale = 192 ** -0.5
    q_nope, q_pe, k_nope, k_pe, v, _ = oracle.prefill_inputs(1, 1, 200, 2)
    out, lse = mla.prefill_forward(*[t.to(gpu) for t in (q_nope, q_pe, k_nope, k_pe, v)], scale)
    torch.cuda.synchronize()
    ref_out, ref_lse = oracle.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, scale)
    assert float((out.float().cpu() - ref_out).abs().max()) <= 1e-2 * float(ref_out.abs().max())
    assert float((lse.cpu() - ref_lse).abs().max()) <= 1e-3
    assert mla.device_status() == 0
