"""Seeded random shapes around the tile boundaries (64, 128, 256, 384 rows), dense and packed, for the
non-absorbed forward + backward, and random paged decode problems, all against the oracle with the
bars of the other tests (O max|err| <= 1e-2 max|ref|, LSE <= 1e-3, gradient rel-L2 <= 1e-2)."""

import random

import pytest
import torch

from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu

SCALE = 192 ** -0.5
EDGES = [2, 17, 63, 64, 65, 127, 128, 129, 191, 255, 256, 257, 383, 384, 385]


def rel_l2(got, ref):
    return float((got.float().cpu() - ref).norm() / ref.norm())


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_prefill_random_shapes(gpu, seed):
    from dscuda_b200 import mla
    rng = random.Random(seed)
    for case in range(12):
        heads = rng.choice([1, 2, 3, 5])
        if rng.random() < 0.5:
            lengths = [rng.choice(EDGES + [rng.randint(2, 600)]) for _ in range(rng.randint(1, 4))]
            q_nope, q_pe, k_nope, k_pe, v, dout, cu = oracle.prefill_inputs(1000 * seed + case, 0, 0, heads, dout_std=0.1, seqlens=lengths)
            layout = (cu.to(gpu), max(lengths))
            ref_layout = (cu,)
        else:
            batch, seq = rng.randint(1, 3), rng.choice(EDGES + [rng.randint(2, 700)])
            q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(1000 * seed + case, batch, seq, heads, dout_std=0.1)
            layout, ref_layout = (), ()
        device = [t.to(gpu) for t in (q_nope, q_pe, k_nope, k_pe, v)]
        out, lse = mla.prefill_forward(*device, SCALE, *layout)
        grads = mla.prefill_backward(dout.to(gpu), out, lse, *device, SCALE, *layout)
        torch.cuda.synchronize()
        assert mla.device_status() == 0
        ref_out, ref_lse = oracle.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, SCALE, *ref_layout)
        ref_grads = oracle.prefill_backward(dout, out.cpu(), lse.cpu(), q_nope, q_pe, k_nope, k_pe, v, SCALE, *ref_layout)
        assert float((out.float().cpu() - ref_out).abs().max()) <= 1e-2 * float(ref_out.abs().max())
        assert float((lse.cpu() - ref_lse).abs().max()) <= 1e-3
        for got, ref in zip(grads, ref_grads):
            assert rel_l2(got, ref) <= 1e-2


@pytest.mark.parametrize("seed", [0, 1])
def test_decode_random_shapes(gpu, seed):
    from dscuda_b200 import mla
    rng = random.Random(100 + seed)
    for case in range(10):
        batch, heads, splits = rng.randint(1, 5), rng.choice([1, 3, 16, 64, 128]), rng.choice([1, 2, 4, 8])
        query, cache, table, lengths = oracle.decode_inputs(seed=3000 + 10 * seed + case, batch=batch, heads=heads, low=1,
                                                            high=rng.choice([64, 65, 130, 700, 2000]))
        out, lse = mla.mla_decode(query.to(gpu), cache.to(gpu), table.to(gpu), lengths.to(gpu), SCALE, splits=splits)
        torch.cuda.synchronize()
        assert mla.device_status() == 0
        ref_out, ref_lse = oracle.paged_decode(query, cache, table, lengths, SCALE)
        assert float((out.float().cpu() - ref_out).abs().max()) <= 1e-2 * float(ref_out.abs().max())
        assert float((lse.cpu() - ref_lse).abs().max()) <= 1e-3


@pytest.mark.parametrize("seed", [0, 1])
def test_absorbed_random_shapes(gpu, seed):
    """Absorbed causal forward and backward on random (batch, tokens, heads): head counts that do not divide the
    128-row tiles (so a row tile starts and ends inside a token), token counts around the key-tile boundaries,
    several batch entries (the rows past a batch entry's last token belong to the next one)."""
    import ctypes
    from dscuda_b200 import mla
    rng = random.Random(200 + seed)
    scale = ctypes.c_float(576 ** -.5).value
    for case in range(8):
        b, h = rng.randint(1, 3), rng.choice([1, 3, 5, 7, 8, 16, 24, 128])
        t = rng.choice([1, 2, 17, 63, 64, 65, 127, 128, 129, 255, 257, rng.randint(2, 400)])
        if h == 128:
            t = min(t, 130)
        g = torch.Generator().manual_seed(5000 + 100 * seed + case)
        inputs = [(torch.randn(shape, generator=g) * .25).bfloat16() for shape in ((b, t, h, 512), (b, t, h, 64), (b, t, 512), (b, t, 64))]
        dout = (torch.randn(b, t, h, 512, generator=g) * .2).bfloat16()
        device = [x.to(gpu) for x in inputs]
        out, lse = mla.mla_forward(*device, scale)
        grads = mla.mla_backward(dout.to(gpu), out, lse, *device, scale)
        torch.cuda.synchronize()
        assert mla.device_status() == 0
        mask = oracle.causal_mask(t)
        ref_out, ref_lse = oracle.absorbed_forward(*inputs, scale, mask)
        torch.testing.assert_close(out.cpu().float(), ref_out.bfloat16().float(), atol=8e-3, rtol=8e-3, msg=lambda m: f"b={b} t={t} h={h}: {m}")
        torch.testing.assert_close(lse.cpu(), ref_lse, atol=1e-4, rtol=1e-4)
        ref_grads = oracle.absorbed_backward(dout, out.cpu(), lse.cpu(), *inputs, scale, mask)
        for got, ref in zip(grads, ref_grads):
            if float(ref.abs().max()) < 1e-6:       # one key: dS is exactly zero and so are the score-path gradients
                assert float(got.float().abs().max()) <= 1e-3, (b, t, h)
            else:
                assert rel_l2(got, ref) <= 1e-2, (b, t, h)


@pytest.mark.parametrize("seed", [0, 1])
def test_backward_random_scratch_limits(gpu, seed):
    """The non-absorbed backward under random scratch limits: anything from no scratch (the recomputing kernel) over
    one head per group to everything at once, dense and packed; the gradients do not depend on the grouping."""
    from dscuda_b200 import mla
    rng = random.Random(300 + seed)
    for case in range(6):
        heads = rng.choice([2, 3, 5])
        packed = rng.random() < 0.5
        if packed:
            lengths = [rng.choice(EDGES + [rng.randint(2, 500)]) for _ in range(rng.randint(2, 4))]
            q_nope, q_pe, k_nope, k_pe, v, dout, cu = oracle.prefill_inputs(7000 + 10 * seed + case, 0, 0, heads, dout_std=0.1, seqlens=lengths)
            layout, ref_layout = (cu.to(gpu), max(lengths)), (cu,)
        else:
            batch, seq = rng.randint(1, 2), rng.choice(EDGES + [rng.randint(2, 500)])
            q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(7000 + 10 * seed + case, batch, seq, heads, dout_std=0.1)
            layout, ref_layout = (), ()
        device = [t.to(gpu) for t in (q_nope, q_pe, k_nope, k_pe, v)]
        out, lse = mla.prefill_forward(*device, SCALE, *layout)
        reference = oracle.prefill_backward(dout, out.cpu(), lse.cpu(), q_nope, q_pe, k_nope, k_pe, v, SCALE, *ref_layout)
        # bytes of dS^T scratch one head needs by the library's bound (include/mla.h): below it the recomputing kernel runs
        count, longest = (len(lengths), max(lengths)) if packed else (batch, seq)
        total = sum(lengths) if packed else batch * seq
        key_tiles = (longest + 127) // 128
        per_head = min(count * (key_tiles * key_tiles + key_tiles), longest * total // 16384 + 1 + 3 * total // 128 + 1 + 2 * count) * 16384
        results = []
        limits = (0, rng.choice([1 << 16, 1 << 19, 1 << 21, per_head, 2 * per_head]), 1 << 34)
        for limit in limits:
            previous = mla.prefill_backward_scratch_limit(limit)
            try:
                grads = mla.prefill_backward(dout.to(gpu), out, lse, *device, SCALE, *layout)
                torch.cuda.synchronize()
            finally:
                mla.prefill_backward_scratch_limit(previous)
            assert mla.device_status() == 0
            for got, ref in zip(grads, reference):
                assert rel_l2(got, ref) <= 1e-2, (limit, packed)
            results.append(grads)
        # dK, dk_pe and dV come from the same kernel on the same tiles whatever the route: identical bits; dQ too
        # whenever both routes stream it from the scratch (group after group or all heads at once)
        for route in results[:2]:
            for index in (1, 2, 3):
                assert torch.equal(route[index], results[2][index])
        if limits[1] >= per_head:
            assert torch.equal(results[1][0], results[2][0])
