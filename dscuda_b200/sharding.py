"""Host-side sharding of the MLA path over the GPUs of one node.

Attention is independent per (batch, head), so the data path needs no
collective: each rank runs the kernels on its own heads (prefill / training) or
its own sequences (decode).  What is left for the host:

* which heads / sequences a rank owns (`head_range`, `decode_partition`);
* the verification gather of per-rank outputs (`gather_heads`);
* the one reduction the math has: dK_pe sums over heads, so head-sharded ranks
  hold partial sums that must be added (`sum_dk_pe_partials`).

Everything here works on any `torch.distributed` backend (NCCL on GPUs, gloo on
CPU for the tests).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def head_range(heads: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced [start, stop) of the heads rank `rank` owns."""
    if not 0 <= rank < world:
        raise ValueError("rank outside the world")
    base, extra = divmod(heads, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def decode_partition(lengths, world: int, page: int = 64) -> list[list[int]]:
    """Sequences per rank, balanced by cache pages (longest first onto the
    lightest rank), so that every cached token is read by exactly one GPU."""
    pages = [(int(n) + page - 1) // page for n in lengths]
    order = sorted(range(len(pages)), key=lambda i: -pages[i])
    loads = [0] * world
    owned: list[list[int]] = [[] for _ in range(world)]
    for index in order:
        target = min(range(world), key=lambda r: (loads[r], r))
        owned[target].append(index)
        loads[target] += pages[index]
    return [sorted(group) for group in owned]


def gather_heads(local: torch.Tensor, heads: int, dim: int, group=None) -> torch.Tensor:
    """All-gather head shards (sizes from `head_range`) along `dim`; every rank gets the full tensor."""
    world = dist.get_world_size(group)
    sizes = [head_range(heads, world, r) for r in range(world)]
    widest = max(stop - start for start, stop in sizes)
    shape = list(local.shape)
    shape[dim] = widest
    padded = local.new_zeros(shape)
    padded.narrow(dim, 0, local.shape[dim]).copy_(local)
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded.contiguous(), group=group)
    return torch.cat([piece.narrow(dim, 0, stop - start) for piece, (start, stop) in zip(pieces, sizes)], dim)


def sum_dk_pe_partials(partial: torch.Tensor, group=None) -> torch.Tensor:
    """Adds the per-rank fp32 dK_pe partial sums (in place) and returns the total."""
    if partial.dtype != torch.float32:
        raise ValueError("dK_pe partial sums are added in fp32")
    dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial
