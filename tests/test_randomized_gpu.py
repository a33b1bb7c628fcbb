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
