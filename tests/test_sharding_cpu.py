"""Head / sequence sharding logic on two gloo ranks (CPU).  The CPU oracle stands
in for the kernels: each rank computes its own heads, the shards are gathered
and the dK_pe partial sums added, and the result must equal the unsharded
computation."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dscuda_b200 import sharding
from oracle import mla_oracle as oracle


def test_head_range_is_a_balanced_partition():
    for heads, world in ((128, 8), (128, 3), (5, 4), (2, 4)):
        ranges = [sharding.head_range(heads, world, r) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == heads
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        sizes = [b - a for a, b in ranges]
        assert max(sizes) - min(sizes) <= 1


def test_decode_partition_balances_pages():
    _, _, _, lengths = oracle.decode_inputs(seed=3, batch=64, heads=1, low=1024, high=32768)
    groups = sharding.decode_partition(lengths.tolist(), 8)
    assert sorted(i for g in groups for i in g) == list(range(64))
    pages = [sum((int(lengths[i]) + 63) // 64 for i in g) for g in groups]
    assert max(pages) - min(pages) <= max((int(n) + 63) // 64 for n in lengths)
    assert max(pages) <= 1.05 * sum(pages) / 8


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        b, s, h = 1, 70, 5
        q_nope, q_pe, k_nope, k_pe, v, dout = oracle.prefill_inputs(13, b, s, h, dtype=torch.float32, dout_std=0.1)
        scale = 192 ** -.5
        start, stop = sharding.head_range(h, world, rank)
        mine = [t[:, :, start:stop].contiguous() for t in (q_nope, q_pe, k_nope)] + [k_pe, v[:, :, start:stop].contiguous()]
        out, lse = oracle.prefill_forward(*mine, scale)
        dq, dk_nope, dk_pe, dv = oracle.prefill_backward(dout[:, :, start:stop].contiguous(), out, lse, *mine, scale)
        full_out = sharding.gather_heads(out, h, 2)
        full_lse = sharding.gather_heads(lse, h, 1)
        full_dq = sharding.gather_heads(dq, h, 2)
        full_dv = sharding.gather_heads(dv, h, 2)
        total_dk_pe = sharding.sum_dk_pe_partials(dk_pe.float().contiguous())
        ref_out, ref_lse = oracle.prefill_forward(q_nope, q_pe, k_nope, k_pe, v, scale)
        ref = oracle.prefill_backward(dout, ref_out, ref_lse, q_nope, q_pe, k_nope, k_pe, v, scale)
        torch.testing.assert_close(full_out, ref_out)
        torch.testing.assert_close(full_lse, ref_lse)
        torch.testing.assert_close(full_dq, ref[0], atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(full_dv, ref[3], atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(total_dk_pe, ref[2], atol=1e-4, rtol=1e-4)
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_head_sharded_forward_backward_on_two_gloo_ranks():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}


def test_decode_splits_keep_the_ranges_equal():
    """`mla.decode_splits`: enough partial slots that the longest sequence may spread over ranges of total / 74 tiles,
    never fewer than the reference harness's 8, never more than 64."""
    from dscuda_b200 import mla
    assert mla.decode_splits([1024] * 64) == 8                       # many short sequences: the minimum
    lengths = [32768] * 8                                            # 8 x 256 tiles: 28 per range, a sequence spans 10 ranges
    assert mla.decode_splits(lengths) == 1 + -(-256 // -(-8 * 256 // 74))
    assert mla.decode_splits([32768]) == 64                          # one sequence over all 74 ranges: capped
    assert mla.decode_splits([5], heads=16) == 8
