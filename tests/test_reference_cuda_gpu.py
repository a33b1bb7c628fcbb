"""This repository's kernels against the reference's own CUDA kernels on the same GPU.

`oracle/build_reference_cuda.py` compiles the reference's MLA kernels for sm_100a from its checkout into
`oracle/_ref/libdscuda_mla_reference.so` (test infrastructure, never loaded by the product).  Both libraries
export the same bridge symbols (`benchmarks/bindings/mla_bridge.cu:12-63` of the reference), so the same
arguments go to both, on the shapes of the reference's own benchmark lists (`benchmarks/mla.py:34-45`),
with its input scales (0.25, dO 0.2), its decode lengths and its tolerances (`:103-105,122-125`).
Skipped where the library was not built (no reference checkout at build time)."""

import ctypes
import pathlib

import pytest
import torch

from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu

ROOT = pathlib.Path(__file__).resolve().parents[1]
REFERENCE_LIBRARY = ROOT / "oracle" / "_ref" / "libdscuda_mla_reference.so"
FLASH_REFERENCE_LIBRARY = ROOT / "oracle" / "_ref" / "libdscuda_flash_attention_reference.so"
P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


@pytest.fixture(scope="module")
def reference():
    if not REFERENCE_LIBRARY.exists():
        pytest.skip("the reference's CUDA kernels were not built (python oracle/build_reference_cuda.py)")
    lib = ctypes.CDLL(str(REFERENCE_LIBRARY))
    lib.dscuda_mla_forward.argtypes = [P] * 6 + [I] * 5 + [F, P]
    lib.dscuda_mla_backward.argtypes = [P] * 11 + [I] * 5 + [F, P]
    lib.dscuda_mla_decode.argtypes = [P] * 7 + [I] * 7 + [F, P]
    lib.dscuda_mla_workspace_elements.argtypes = [I] * 4
    lib.dscuda_mla_workspace_elements.restype = ctypes.c_size_t
    lib.dscuda_mla_last_error.restype = ctypes.c_char_p
    return lib


def ok(lib, status):
    assert status == 0, lib.dscuda_mla_last_error().decode()


def stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("b,t,h", [(1, 128, 8), (2, 257, 4), (1, 512, 8), (2, 17, 3), (1, 65, 4)])
def test_forward_and_backward_equal_the_reference_kernels(gpu, reference, b, t, h):
    from dscuda_b200 import mla
    g = torch.Generator().manual_seed(t)
    q, qr, kv, kr = (((torch.randn(shape, generator=g) * 0.25).bfloat16()).to(gpu) for shape in ((b, t, h, 512), (b, t, h, 64), (b, t, 512), (b, t, 64)))
    dout = (torch.randn(b, t, h, 512, generator=g) * 0.2).bfloat16().to(gpu)
    scale = ctypes.c_float(576 ** -0.5).value
    ref_out = torch.empty(b, t, h, 512, device=gpu, dtype=torch.bfloat16)
    ref_lse = torch.empty(b, h, t, device=gpu)
    ok(reference, reference.dscuda_mla_forward(ref_out.data_ptr(), ref_lse.data_ptr(), q.data_ptr(), qr.data_ptr(), kv.data_ptr(), kr.data_ptr(),
                                               b, t, h, 512, 64, scale, stream()))
    out, lse = mla.mla_forward(q, qr, kv, kr, scale)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), ref_out.float(), atol=8e-3, rtol=8e-3)
    torch.testing.assert_close(lse, ref_lse, atol=1e-4, rtol=1e-4)
    # both backwards from the same saved forward (the reference's)
    ref_grads = [torch.empty_like(x) for x in (q, qr, kv, kr)]
    ok(reference, reference.dscuda_mla_backward(*[x.data_ptr() for x in ref_grads], dout.data_ptr(), ref_out.data_ptr(), ref_lse.data_ptr(),
                                                q.data_ptr(), qr.data_ptr(), kv.data_ptr(), kr.data_ptr(), b, t, h, 512, 64, scale, stream()))
    grads = mla.mla_backward(dout, ref_out, ref_lse, q, qr, kv, kr, scale)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    for name, got, ref in zip(("dq_latent", "dq_rope", "dkv_latent", "dk_rope"), grads, ref_grads):
        torch.testing.assert_close(got.float(), ref.float(), atol=1e-2, rtol=1e-2, msg=lambda m, name=name: f"{name}: {m}")


@pytest.mark.parametrize("b,t,h", [(2, 1024, 16), (1, 256, 16), (4, 4096, 32), (3, 129, 128), (2, 65, 64)])
def test_decode_equals_the_reference_kernels(gpu, reference, b, t, h):
    from dscuda_b200 import mla
    g = torch.Generator().manual_seed(t + h)
    query = (torch.randn(b, 1, h, 576, generator=g) * 0.25).bfloat16()
    kv = (torch.randn(b, t, 576, generator=g) * 0.25).bfloat16()
    lengths = [max(1, t - i * t // (2 * b)) for i in range(b)]          # benchmarks/mla.py:58-60 of the reference
    lengths = [1] + lengths[1:-1] + [t] if b > 1 else lengths
    cache, table = oracle.pack_cache(kv, 64)
    splits = 8
    scale = ctypes.c_float(576 ** -0.5).value
    query, cache, table = query.to(gpu), cache.to(gpu), table.to(gpu)
    length_tensor = torch.tensor(lengths, dtype=torch.int32, device=gpu)
    workspace = torch.empty(reference.dscuda_mla_workspace_elements(b, h, splits, 512), device=gpu)
    ref_out = torch.empty(b, 1, h, 512, device=gpu, dtype=torch.bfloat16)
    ref_lse = torch.empty(b, h, 1, device=gpu)
    ok(reference, reference.dscuda_mla_decode(ref_out.data_ptr(), ref_lse.data_ptr(), query.data_ptr(), cache.data_ptr(), table.data_ptr(),
                                              length_tensor.data_ptr(), workspace.data_ptr(), b, h, 512, 64, 64, table.shape[1], splits, scale, stream()))
    out, lse = mla.mla_decode(query, cache, table, length_tensor, scale, splits=splits)
    torch.cuda.synchronize()
    assert mla.device_status() == 0
    torch.testing.assert_close(out.float(), ref_out.float(), atol=8e-3, rtol=8e-3)
    torch.testing.assert_close(lse.reshape(-1), ref_lse.reshape(-1), atol=1e-4, rtol=1e-4)


def test_speed_beside_the_reference_kernels(gpu, reference):
    """Both libraries timed with CUDA events on the reference's benchmark shapes (`benchmarks/mla.py:34-45`: its largest
    prefill shape, decode shapes of its `h100` suite).  The figures go to gpurun_out/reference_cuda_timing.json where
    that directory exists; the assertion only says that nothing here is slower than the code it replaces."""
    import json
    from dscuda_b200 import mla
    g = torch.Generator(device=gpu).manual_seed(11)

    def draw(*shape):
        return (torch.randn(*shape, device=gpu, generator=g) * 0.25).bfloat16()

    def microseconds(call, steps=5, warmup=2):
        for _ in range(warmup):
            call()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            call()
        stop.record()
        stop.synchronize()
        return start.elapsed_time(stop) * 1e3 / steps

    scale = ctypes.c_float(576 ** -0.5).value
    rows = {}
    b, t, h = 1, 512, 8
    q, qr, kv, kr, dout = draw(b, t, h, 512), draw(b, t, h, 64), draw(b, t, 512), draw(b, t, 64), draw(b, t, h, 512)
    out, lse = mla.mla_forward(q, qr, kv, kr, scale)
    ref_out, ref_lse = torch.empty_like(out), torch.empty_like(lse)
    ref_grads = [torch.empty_like(x) for x in (q, qr, kv, kr)]
    rows[f"forward B={b} T={t} H={h}"] = (
        microseconds(lambda: mla.mla_forward(q, qr, kv, kr, scale)),
        microseconds(lambda: reference.dscuda_mla_forward(ref_out.data_ptr(), ref_lse.data_ptr(), q.data_ptr(), qr.data_ptr(), kv.data_ptr(),
                                                          kr.data_ptr(), b, t, h, 512, 64, scale, stream())))
    rows[f"backward B={b} T={t} H={h}"] = (
        microseconds(lambda: mla.mla_backward(dout, out, lse, q, qr, kv, kr, scale)),
        microseconds(lambda: reference.dscuda_mla_backward(*[x.data_ptr() for x in ref_grads], dout.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                                           q.data_ptr(), qr.data_ptr(), kv.data_ptr(), kr.data_ptr(), b, t, h, 512, 64, scale, stream())))
    for b, t, h in ((4, 4096, 128), (8, 8192, 128)):
        query = draw(b, 1, h, 576)
        pages = t // 64
        cache = draw(b * pages, 64, 1, 576)
        table = torch.arange(b * pages, dtype=torch.int32, device=gpu).reshape(b, pages)
        lengths = torch.tensor([max(1, t - i * t // (2 * b)) for i in range(b)], dtype=torch.int32, device=gpu)
        workspace = torch.empty(reference.dscuda_mla_workspace_elements(b, h, 8, 512), device=gpu)
        d_out = torch.empty(b, 1, h, 512, device=gpu, dtype=torch.bfloat16)
        d_lse = torch.empty(b, h, 1, device=gpu)
        r_out, r_lse = torch.empty_like(d_out), torch.empty_like(d_lse)
        rows[f"decode B={b} KV={t} H={h}"] = (
            microseconds(lambda: mla.mla_decode(query, cache, table, lengths, scale, splits=8, workspace=workspace, output=d_out, lse=d_lse)),
            microseconds(lambda: reference.dscuda_mla_decode(r_out.data_ptr(), r_lse.data_ptr(), query.data_ptr(), cache.data_ptr(), table.data_ptr(),
                                                             lengths.data_ptr(), workspace.data_ptr(), b, h, 512, 64, 64, pages, 8, scale, stream())))
        torch.testing.assert_close(d_out.float(), r_out.float(), atol=8e-3, rtol=8e-3)
    if FLASH_REFERENCE_LIBRARY.exists():        # the largest shape of the reference's flash-attention list
        flash = ctypes.CDLL(str(FLASH_REFERENCE_LIBRARY))
        flash.dscuda_flash_forward.argtypes = [P] * 5 + [I] * 5 + [F, P]
        b, t, hq, hkv = 4, 2048, 8, 1
        fq, fk, fv = draw(b, t, hq, 128), draw(b, t, hkv, 128), draw(b, t, hkv, 128)
        f_out, f_lse = torch.empty_like(fq), torch.empty(b, hq, t, device=gpu)
        rows[f"flash forward B={b} T={t} Hq={hq} Hkv={hkv}"] = (
            microseconds(lambda: mla.flash_forward(fq, fk, fv, 128 ** -0.5)),
            microseconds(lambda: flash.dscuda_flash_forward(f_out.data_ptr(), f_lse.data_ptr(), fq.data_ptr(), fk.data_ptr(), fv.data_ptr(),
                                                            b, t, hq, hkv, 128, 128 ** -0.5, stream())))
    report = {name: {"this_us": mine, "reference_us": theirs, "speedup": theirs / mine} for name, (mine, theirs) in rows.items()}
    for name, row in report.items():
        print(f"{name}: this {row['this_us']:.1f} us, reference kernels {row['reference_us']:.1f} us, x{row['speedup']:.1f}")
    log = ROOT / "gpurun_out"
    if log.is_dir():
        (log / "reference_cuda_timing.json").write_text(json.dumps(report, indent=1))
    assert all(row["speedup"] >= 1.0 for row in report.values()), report


@pytest.mark.parametrize("b,t,hq,hkv", [(1, 64, 2, 2), (2, 64, 4, 2), (1, 128, 4, 1), (1, 256, 8, 8), (1, 512, 8, 2), (4, 2048, 8, 1)])
def test_flash_forward_equals_the_reference_kernel(gpu, b, t, hq, hkv):
    """D = 128 grouped-query forward on the shapes of `benchmarks/flash_attention.py:42-56` of the reference (input
    scale 0.5, tolerances of its own check), both libraries timed on the largest one."""
    from dscuda_b200 import mla
    if not FLASH_REFERENCE_LIBRARY.exists():
        pytest.skip("the reference's CUDA kernels were not built (python oracle/build_reference_cuda.py)")
    lib = ctypes.CDLL(str(FLASH_REFERENCE_LIBRARY))
    lib.dscuda_flash_forward.argtypes = [P] * 5 + [I] * 5 + [F, P]
    lib.dscuda_flash_last_error.restype = ctypes.c_char_p
    g = torch.Generator().manual_seed(t + hq)
    q = (torch.randn(b, t, hq, 128, generator=g) * 0.5).bfloat16().to(gpu)
    k = (torch.randn(b, t, hkv, 128, generator=g) * 0.5).bfloat16().to(gpu)
    v = (torch.randn(b, t, hkv, 128, generator=g) * 0.5).bfloat16().to(gpu)
    scale = 128 ** -0.5
    ref_out = torch.empty_like(q)
    ref_lse = torch.empty(b, hq, t, device=gpu)
    status = lib.dscuda_flash_forward(ref_out.data_ptr(), ref_lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), b, t, hq, hkv, 128, scale, stream())
    assert status == 0, lib.dscuda_flash_last_error().decode()
    out, lse = mla.flash_forward(q, k, v, scale)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), ref_out.float(), atol=1e-2, rtol=1e-2)
    torch.testing.assert_close(lse, ref_lse, atol=1e-4, rtol=1e-4)
