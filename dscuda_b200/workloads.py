"""The five benchmark configurations of the MLA path and their seeded synthetic inputs.

    C1  B=1, S=256,  H=16   forward + backward (the reference's CPU-sized case)
    C2  B=4, S=4096, H=128  forward only
    C3  B=2, S=8192, H=128  forward + backward (the headline training step)
    C4  paged decode, batch 64, H=128, lengths uniform in [1024, 32768], 64-token pages
    C5  16 packed sequences, lengths log-uniform in [512, 32768], forward + backward

Nothing here comes from a dataset: the shapes are DeepSeek-V3-sized dimensions and the
values are seeded normal draws.  The work counts are the algorithmic ones every reported
TFLOP/s and GB/s figure uses: 640 FLOP per causal (query, key) pair and head forward,
1664 backward; decode bytes are every cached token read once plus Q, O, LSE and the tables.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

SCALE = 192 ** -0.5
FWD_FLOP_PER_PAIR = 2 * (192 + 128)
BWD_FLOP_PER_PAIR = 2 * (192 + 128 + 128 + 192 + 192)

CONFIGS: Dict[str, dict] = {
    "C1": dict(kind="dense", batch=1, seq=256, heads=16, seed=0, dout_std=1.0, backward=True),
    "C2": dict(kind="dense", batch=4, seq=4096, heads=128, seed=1, dout_std=1.0, backward=False),
    "C3": dict(kind="dense", batch=2, seq=8192, heads=128, seed=2, dout_std=0.1, backward=True),
    "C4": dict(kind="decode", batch=64, heads=128, seed=3, low=1024, high=32768, page=64, splits=8),
    "C5": dict(kind="packed", sequences=16, heads=16, seed=4, low=512, high=32768, dout_std=0.1, backward=True),
}


def causal_pairs(length: int) -> int:
    return length * (length + 1) // 2


def dense_flops(config: dict) -> int:
    pairs = causal_pairs(config["seq"]) * config["batch"] * config["heads"]
    return pairs * (FWD_FLOP_PER_PAIR + (BWD_FLOP_PER_PAIR if config["backward"] else 0))


def packed_flops(lengths: List[int], heads: int, backward: bool = True) -> int:
    pairs = sum(causal_pairs(n) for n in lengths) * heads
    return pairs * (FWD_FLOP_PER_PAIR + (BWD_FLOP_PER_PAIR if backward else 0))


def decode_bytes(lengths: torch.Tensor, table: torch.Tensor, batch: int, heads: int) -> int:
    """Cache rows read once (shared by all heads), Q in, O and LSE out, table and lengths."""
    return int(lengths.sum()) * 576 * 2 + batch * heads * (576 + 512) * 2 + batch * heads * 4 + table.numel() * 4 + lengths.numel() * 4


def decode_flops(lengths: torch.Tensor, heads: int) -> int:
    return 2 * (576 + 512) * heads * int(lengths.sum())


def dense_inputs(config: dict, device: torch.device, shard: int = 0, rotate=None) -> Dict[str, torch.Tensor]:
    """Seeded N(0,1) bf16 tensors drawn on the device.  Rotary embedding is input preparation (the
    kernels take q_pe / k_pe as they are): `rotate(q_pe, k_pe, positions)`, when given, applies it in place
    with position = index along the sequence (`dscuda_b200.mla.rope_apply` has that signature).  `shard`
    selects the per-head tensors of one head shard of a larger job (a different stream of draws per
    shard); `k_pe`, the rotary key every head shares, is the same for every shard."""
    shared = torch.Generator(device=device).manual_seed(config["seed"])
    g = torch.Generator(device=device).manual_seed(config["seed"] + 7919 * shard) if shard else shared
    b, s, h = config["batch"], config["seq"], config["heads"]

    def draw(*shape, std=1.0, generator=g):
        return (torch.randn(*shape, device=device, generator=generator, dtype=torch.float32) * std).bfloat16()

    k_pe = draw(b, s, 1, 64, generator=shared)
    tensors = dict(q_nope=draw(b, s, h, 128), q_pe=draw(b, s, h, 64), k_nope=draw(b, s, h, 128), k_pe=k_pe, v=draw(b, s, h, 128))
    if config["backward"]:
        tensors["dout"] = draw(b, s, h, 128, std=config["dout_std"])
    if rotate is not None:
        rotate(tensors["q_pe"], tensors["k_pe"], None)
    return tensors


def varlen_lengths(seed: int = 4, count: int = 16, low: int = 512, high: int = 32768) -> List[int]:
    """Sequence lengths log-uniform in [low, high] from a CPU generator (the same on every machine)."""
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(count, generator=g, dtype=torch.float64)
    return [int(round(math.exp(math.log(low) + float(x) * (math.log(high) - math.log(low))))) for x in u]


def packed_inputs(lengths: List[int], heads: int, seed: int, device: torch.device, dout_std: float = 0.1, shard: int = 0, rotate=None):
    """Packed [total, H, *] tensors plus int32 cu_seqlens on the device (`shard` and `rotate` as in
    dense_inputs; positions restart at 0 in every sequence)."""
    total = sum(lengths)
    shared = torch.Generator(device=device).manual_seed(seed)
    g = torch.Generator(device=device).manual_seed(seed + 7919 * shard) if shard else shared

    def draw(*shape, std=1.0, generator=g):
        return (torch.randn(*shape, device=device, generator=generator, dtype=torch.float32) * std).bfloat16()

    k_pe = draw(total, 1, 64, generator=shared)
    tensors = dict(q_nope=draw(total, heads, 128), q_pe=draw(total, heads, 64), k_nope=draw(total, heads, 128), k_pe=k_pe,
                   v=draw(total, heads, 128))
    tensors["dout"] = draw(total, heads, 128, std=dout_std)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=device)
    if rotate is not None:
        positions = torch.cat([torch.arange(n, dtype=torch.int32) for n in lengths]).to(device)
        rotate(tensors["q_pe"], tensors["k_pe"], positions)
    return tensors, cu


def decode_inputs(seed: int = 3, batch: int = 64, heads: int = 128, low: int = 1024, high: int = 32768, page: int = 64,
                  lengths: Optional[torch.Tensor] = None):
    """Packed query [B,1,H,576], paged cache [pages,64,1,576] ~ N(0,1) bf16, lengths uniform in
    [low, high], page table cut from one random permutation of all pages (CPU generator)."""
    g = torch.Generator().manual_seed(seed)
    if lengths is None:
        lengths = torch.randint(low, high + 1, (batch,), generator=g)
    lengths = torch.as_tensor(lengths, dtype=torch.int64)
    pages_each = (lengths + page - 1) // page
    total_pages = int(pages_each.sum())
    max_pages = int(pages_each.max())
    cache = torch.randn(total_pages, page, 1, 576, generator=g, dtype=torch.float32).bfloat16()
    query = torch.randn(batch, 1, heads, 576, generator=g, dtype=torch.float32).bfloat16()
    order = torch.randperm(total_pages, generator=g).to(torch.int32)
    table = torch.zeros(batch, max_pages, dtype=torch.int32)
    start = 0
    for b in range(batch):
        n = int(pages_each[b])
        table[b, :n] = order[start:start + n]
        start += n
    return query, cache, table, lengths.to(torch.int32)
