"""CPU oracle for the MLA path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain CPU torch, the arithmetic of the reference's
`reference/python/mla.py` and of the PyTorch expression in
`benchmarks/flash_attention.py`.  It exists so that the CUDA kernels can be
checked; nothing in the product path may import it.  Only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark use it.

Parity pin: the reference stores no golden vectors, so this restatement is
pinned against outputs of the reference's own `mla_forward`/`mla_backward`
(imported from the reference checkout by `tests/golden/make_golden.py`), which
are committed as fixtures under `tests/golden/`.

Two families of functions:

* the absorbed contract of the reference itself (head-shared latent is both K
  and V): `absorbed_forward`, `absorbed_backward`, `paged_decode`;
* the non-absorbed contract (per-head k_nope / v, one shared k_pe head) that
  the reference has no function for: `prefill_forward`, `prefill_backward`.
  They follow the same steps as `reference/python/mla.py:26-57` with the
  latent replaced by per-head tensors.

All functions keep fp64 inputs in fp64 and compute everything else in fp32
(`reference/python/mla.py:6-8`).  They return UN-ROUNDED results; the caller
rounds to bf16 where the reference does (`mla.py:39,56-57`).
"""

from __future__ import annotations

import math

import torch


def _compute(tensor: torch.Tensor) -> torch.Tensor:
    # reference/python/mla.py:6-8 -- 4- and 8-byte floats stay, bf16 widens.
    return tensor if tensor.element_size() >= 4 else tensor.float()


def causal_mask(t: int) -> torch.Tensor:
    # benchmarks/mla.py:62-63
    return torch.ones(t, t, dtype=torch.bool).tril()


# --------------------------------------------------------------------------
# Absorbed contract (reference/python/mla.py)
# --------------------------------------------------------------------------

def _absorbed_scores(query, query_rope, latent, key_rope, scale, mask):
    # reference/python/mla.py:26-29
    score = (torch.einsum("bqhc,bkc->bhqk", query, latent)
             + torch.einsum("bqhr,bkr->bhqk", query_rope, key_rope)) * scale
    return score.masked_fill(~mask, float("-inf"))


def absorbed_forward(query, query_rope, latent, key_rope, scale, mask):
    """reference/python/mla.py:32-39 without the final bf16 cast.

    query [B,Q,H,C], query_rope [B,Q,H,R], latent [B,K,C], key_rope [B,K,R];
    mask broadcastable to [B,H,Q,K].  Returns (output [B,Q,H,C], lse [B,H,Q]).
    """
    query, query_rope, latent, key_rope = map(
        _compute, (query, query_rope, latent, key_rope))
    score = _absorbed_scores(query, query_rope, latent, key_rope, scale, mask)
    lse = score.logsumexp(dim=-1)
    probability = (score - lse.unsqueeze(-1)).exp()
    output = torch.einsum("bhqk,bkc->bqhc", probability, latent)
    return output.contiguous(), lse.contiguous()


def absorbed_backward(dout, output, lse, query, query_rope, latent, key_rope,
                      scale, mask):
    """reference/python/mla.py:42-57 without the final bf16 cast."""
    dout, output, query, query_rope, latent, key_rope = map(
        _compute, (dout, output, query, query_rope, latent, key_rope))
    score = _absorbed_scores(query, query_rope, latent, key_rope, scale, mask)
    probability = (score - lse.unsqueeze(-1)).exp()
    dprobability = torch.einsum("bqhc,bkc->bhqk", dout, latent)
    delta = (dout * output).sum(dim=-1).transpose(1, 2).unsqueeze(-1)
    dscore = probability * (dprobability - delta) * scale
    dquery = torch.einsum("bhqk,bkc->bqhc", dscore, latent)
    dquery_rope = torch.einsum("bhqk,bkr->bqhr", dscore, key_rope)
    dlatent = (torch.einsum("bhqk,bqhc->bkc", dscore, query)
               + torch.einsum("bhqk,bqhc->bkc", probability, dout))
    dkey_rope = torch.einsum("bhqk,bqhr->bkr", dscore, query_rope)
    return tuple(t.contiguous()
                 for t in (dquery, dquery_rope, dlatent, dkey_rope))


def pack_cache(kv, page_size=64, permutation=None):
    """reference/python/mla.py:11-23, plus an optional page permutation.

    kv [B,N,W] -> (cache [B*pages,page,1,W], table [B,pages] int32).  With
    `permutation` (a permutation of range(B*pages)) logical page i is stored
    at physical page permutation[i] and the table says so.
    """
    batch, tokens, width = kv.shape
    pages = (tokens + page_size - 1) // page_size
    padded = torch.nn.functional.pad(kv, (0, 0, 0, pages * page_size - tokens))
    logical = padded.reshape(batch * pages, page_size, 1, width)
    table = torch.arange(batch * pages, dtype=torch.int32).reshape(batch, pages)
    if permutation is None:
        return logical.contiguous(), table
    permutation = torch.as_tensor(permutation, dtype=torch.int64)
    physical = torch.empty_like(logical)
    physical[permutation] = logical
    return physical.contiguous(), permutation.to(torch.int32).reshape(batch, pages)


def paged_decode(query, paged_cache, block_table, lengths, scale, rank=512):
    """One query token per sequence against a paged cache.

    The reference checks decode against `mla_forward` with a length mask
    (`benchmarks/mla.py:62-67`); this gathers the pages through the table
    (`kernels/attention/mla/sm89.cu:443-446`) and does the same.

    query [B,1,H,rank+rope], paged_cache [blocks,page,1,rank+rope],
    block_table [B,pages] int32, lengths [B] int32.
    Returns (output [B,1,H,rank], lse [B,H,1]).
    """
    batch = query.shape[0]
    page = paged_cache.shape[1]
    pages = block_table.shape[1]
    gathered = paged_cache[block_table.long().reshape(-1)]          # [B*pages,page,1,W]
    kv = gathered.reshape(batch, pages * page, -1)
    positions = torch.arange(pages * page)[None]
    mask = (positions < torch.as_tensor(lengths).long()[:, None])[:, None, None]
    return absorbed_forward(query[..., :rank], query[..., rank:],
                            kv[..., :rank], kv[..., rank:], scale, mask)


def quantize_fp8_rows(kv):
    """FP8 cache rows of tokens `kv` [..., 576] bf16 (no counterpart in the reference, which is unquantised):
    per 128-column group of the 512 latent values scale = max|x| / 448 (1 for a zero group), value / scale
    rounded to e4m3; returns (codes uint8 [..., 512], scales fp32 [..., 4], rope bf16 [..., 64])."""
    latent = kv[..., :512].float().reshape(*kv.shape[:-1], 4, 128)
    amax = latent.abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    codes = (latent / scale).to(torch.float8_e4m3fn).view(torch.uint8).reshape(*kv.shape[:-1], 512)
    return codes, scale.squeeze(-1).contiguous(), kv[..., 512:].contiguous()


def dequantize_fp8_rows(codes, scales, rope):
    """The bf16 rows [..., 576] an FP8 cache row stands for: e4m3 * scale rounded to bf16, rotary values unchanged."""
    latent = codes.view(torch.float8_e4m3fn).float().reshape(*codes.shape[:-1], 4, 128) * scales.unsqueeze(-1)
    return torch.cat((latent.reshape(*codes.shape[:-1], 512).bfloat16(), rope), -1)


# --------------------------------------------------------------------------
# Non-absorbed contract (per-head k_nope / v, shared k_pe)
# --------------------------------------------------------------------------

def _prefill_scores(q_nope, q_pe, k_nope, k_pe, scale, mask):
    # reference/python/mla.py:26-29 with latent[b,k,c] -> k_nope[b,k,h,c]
    score = (torch.einsum("bqhc,bkhc->bhqk", q_nope, k_nope)
             + torch.einsum("bqhr,bkr->bhqk", q_pe, k_pe[:, :, 0])) * scale
    return score.masked_fill(~mask, float("-inf"))


def _prefill_forward_dense(q_nope, q_pe, k_nope, k_pe, v, scale):
    mask = causal_mask(q_nope.shape[1])
    score = _prefill_scores(q_nope, q_pe, k_nope, k_pe, scale, mask)
    lse = score.logsumexp(dim=-1)                                   # mla.py:36
    probability = (score - lse.unsqueeze(-1)).exp()                 # mla.py:37
    output = torch.einsum("bhqk,bkhd->bqhd", probability, v)        # mla.py:38
    return output, lse


def _prefill_backward_dense(dout, output, lse, q_nope, q_pe, k_nope, k_pe, v, scale):
    mask = causal_mask(q_nope.shape[1])
    score = _prefill_scores(q_nope, q_pe, k_nope, k_pe, scale, mask)
    probability = (score - lse.unsqueeze(-1)).exp()                 # mla.py:46
    dprobability = torch.einsum("bqhd,bkhd->bhqk", dout, v)         # mla.py:47
    delta = (dout * output).sum(dim=-1).transpose(1, 2).unsqueeze(-1)  # mla.py:48
    dscore = probability * (dprobability - delta) * scale           # mla.py:49
    dq_nope = torch.einsum("bhqk,bkhc->bqhc", dscore, k_nope)       # mla.py:50
    dq_pe = torch.einsum("bhqk,bkr->bqhr", dscore, k_pe[:, :, 0])   # mla.py:51
    dk_nope = torch.einsum("bhqk,bqhc->bkhc", dscore, q_nope)       # mla.py:53, no head sum
    dv = torch.einsum("bhqk,bqhd->bkhd", probability, dout)         # mla.py:54, no head sum
    dk_pe = torch.einsum("bhqk,bqhr->bkr", dscore, q_pe)[:, :, None]  # mla.py:55, head sum kept
    return torch.cat((dq_nope, dq_pe), -1), dk_nope, dk_pe, dv


def _segments(total, cu_seqlens):
    if cu_seqlens is None:
        return None
    cu = [int(x) for x in cu_seqlens]
    assert cu[0] == 0 and cu[-1] == total
    return list(zip(cu[:-1], cu[1:]))


def prefill_forward(q_nope, q_pe, k_nope, k_pe, v, scale, cu_seqlens=None):
    """Causal non-absorbed MLA forward.

    Dense: q_nope [B,S,H,128], q_pe [B,S,H,64], k_nope [B,S,H,128],
    k_pe [B,S,1,64], v [B,S,H,128] -> (O [B,S,H,128], LSE [B,H,S]).
    Packed (cu_seqlens given): the leading [B,S] becomes [total]; causal
    within each sequence; LSE is [H,total].
    """
    q_nope, q_pe, k_nope, k_pe, v = map(_compute, (q_nope, q_pe, k_nope, k_pe, v))
    if cu_seqlens is None:
        output, lse = _prefill_forward_dense(q_nope, q_pe, k_nope, k_pe, v, scale)
        return output.contiguous(), lse.contiguous()
    outputs, lses = [], []
    for a, b in _segments(q_nope.shape[0], cu_seqlens):
        o, l = _prefill_forward_dense(*(t[None, a:b] for t in (q_nope, q_pe, k_nope, k_pe, v)), scale)
        outputs.append(o[0])
        lses.append(l[0])
    return torch.cat(outputs, 0).contiguous(), torch.cat(lses, 1).contiguous()


def prefill_backward(dout, output, lse, q_nope, q_pe, k_nope, k_pe, v, scale,
                     cu_seqlens=None):
    """Closed-form backward of `prefill_forward`.

    Returns (dQ [...,H,192] = nope||pe, dK_nope [...,H,128],
    dK_pe [...,1,64] summed over heads, dV [...,H,128]).
    """
    dout, output, q_nope, q_pe, k_nope, k_pe, v = map(
        _compute, (dout, output, q_nope, q_pe, k_nope, k_pe, v))
    if cu_seqlens is None:
        return tuple(t.contiguous() for t in _prefill_backward_dense(
            dout, output, lse, q_nope, q_pe, k_nope, k_pe, v, scale))
    parts = []
    for a, b in _segments(q_nope.shape[0], cu_seqlens):
        parts.append(_prefill_backward_dense(
            dout[None, a:b], output[None, a:b], lse[None, :, a:b],
            *(t[None, a:b] for t in (q_nope, q_pe, k_nope, k_pe, v)), scale))
    return tuple(torch.cat([p[i][0] for p in parts], 0).contiguous() for i in range(4))


def prefill_row_block(q_nope, q_pe, k_nope, k_pe, v, scale, rows, dout=None):
    """The query rows `rows = (r0, r1)` of a dense causal problem without the full
    S x S matrices: only the (r1-r0) x r1 score block is formed.  Same steps as
    `_prefill_forward_dense` / `_prefill_backward_dense` (reference/python/mla.py:26-51)
    restricted to those rows, so sequences of tens of thousands of tokens can be
    checked on the CPU.

    Tensors are dense [B,S,H,*].  Returns (O [B,r1-r0,H,128], LSE [B,H,r1-r0]) and,
    when `dout` [B,S,H,128] is given, also dQ [B,r1-r0,H,192].
    """
    q_nope, q_pe, k_nope, k_pe, v = map(_compute, (q_nope, q_pe, k_nope, k_pe, v))
    r0, r1 = rows
    queries = torch.arange(r0, r1)[:, None]
    mask = torch.arange(r1)[None, :] <= queries                                  # key k visible to query q iff k <= q
    score = _prefill_scores(q_nope[:, r0:r1], q_pe[:, r0:r1], k_nope[:, :r1], k_pe[:, :r1], scale, mask)
    lse = score.logsumexp(dim=-1)
    probability = (score - lse.unsqueeze(-1)).exp()
    output = torch.einsum("bhqk,bkhd->bqhd", probability, v[:, :r1])
    if dout is None:
        return output.contiguous(), lse.contiguous()
    dout = _compute(dout)[:, r0:r1]
    dprobability = torch.einsum("bqhd,bkhd->bhqk", dout, v[:, :r1])
    delta = (dout * output).sum(dim=-1).transpose(1, 2).unsqueeze(-1)
    dscore = probability * (dprobability - delta) * scale
    dq = torch.cat((torch.einsum("bhqk,bkhc->bqhc", dscore, k_nope[:, :r1]),
                    torch.einsum("bhqk,bkr->bqhr", dscore, k_pe[:, :r1, 0])), -1)
    return output.contiguous(), lse.contiguous(), dq.contiguous()


def prefill_key_block(dout, output, lse, q_nope, q_pe, k_nope, k_pe, v, scale, keys):
    """The key rows `keys = (k0, k1)` of the closed-form backward without the full
    S x S matrices: only the (S-k0) x (k1-k0) block (queries k0..S-1) is formed.
    Same steps as `_prefill_backward_dense` (reference/python/mla.py:46-55).

    Dense [B,S,H,*] tensors, `output` / `lse` [B,H,S] from the forward.  Returns
    (dK_nope [B,k1-k0,H,128], dK_pe [B,k1-k0,1,64] summed over heads, dV [B,k1-k0,H,128]).
    """
    dout, output, q_nope, q_pe, k_nope, k_pe, v = map(_compute, (dout, output, q_nope, q_pe, k_nope, k_pe, v))
    k0, k1 = keys
    total = q_nope.shape[1]
    mask = torch.arange(k0, k1)[None, :] <= torch.arange(k0, total)[:, None]
    score = _prefill_scores(q_nope[:, k0:], q_pe[:, k0:], k_nope[:, k0:k1], k_pe[:, k0:k1], scale, mask)
    probability = (score - lse[:, :, k0:].unsqueeze(-1)).exp()
    dprobability = torch.einsum("bqhd,bkhd->bhqk", dout[:, k0:], v[:, k0:k1])
    delta = (dout[:, k0:] * output[:, k0:]).sum(dim=-1).transpose(1, 2).unsqueeze(-1)
    dscore = probability * (dprobability - delta) * scale
    dk_nope = torch.einsum("bhqk,bqhc->bkhc", dscore, q_nope[:, k0:])
    dv = torch.einsum("bhqk,bqhd->bkhd", probability, dout[:, k0:])
    dk_pe = torch.einsum("bhqk,bqhr->bkr", dscore, q_pe[:, k0:])[:, :, None]
    return dk_nope.contiguous(), dk_pe.contiguous(), dv.contiguous()


# --------------------------------------------------------------------------
# FlashAttention D=128 GQA forward (benchmarks/flash_attention.py:68-75)
# --------------------------------------------------------------------------

def flash_forward(query, key, value, scale):
    """query [B,T,Hq,D], key/value [B,T,Hkv,D] -> (O [B,T,Hq,D], LSE [B,Hq,T])."""
    query, key, value = map(_compute, (query, key, value))
    group = query.shape[2] // key.shape[2]
    if group > 1:
        key = key.repeat_interleave(group, dim=2)
        value = value.repeat_interleave(group, dim=2)
    q, k, v = (x.transpose(1, 2) for x in (query, key, value))
    mask = causal_mask(query.shape[1])
    scores = (q @ k.transpose(-1, -2) * scale).masked_fill(~mask, -torch.inf)
    return (scores.softmax(-1) @ v).transpose(1, 2).contiguous(), scores.logsumexp(-1)


# --------------------------------------------------------------------------
# Seeded synthetic inputs for the five benchmark configurations
# --------------------------------------------------------------------------

def rope(x, positions, theta=10000.0):
    """Rotate-half RoPE: pairs (i, i+R/2), angle pos * theta^(-2i/R).

    x [..., S, H, R] with `positions` [S] (or broadcastable to the S axis).
    """
    r = x.shape[-1]
    half = r // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / r)
    angle = positions.to(torch.float64)[:, None] * inv[None]           # [S, half]
    cos = angle.cos()[:, None, :].to(x.dtype)
    sin = angle.sin()[:, None, :].to(x.dtype)
    a, b = x[..., :half], x[..., half:]
    return torch.cat((a * cos - b * sin, a * sin + b * cos), -1)


def prefill_inputs(seed, batch, seq, heads, dtype=torch.bfloat16, dout_std=1.0,
                   seqlens=None):
    """q_nope, q_pe, k_nope, k_pe, v, dO ~ N(0,1) (dO ~ N(0,dout_std)) from a
    CPU generator; RoPE (theta 10000, positions from 0 within each sequence) is
    applied to q_pe / k_pe here, so kernels see post-RoPE tensors.

    Dense: leading dims [batch, seq].  Packed: `seqlens` given -> leading dim
    [sum(seqlens)] and cu_seqlens is returned as the last item.
    """
    g = torch.Generator().manual_seed(seed)
    lead = (batch, seq) if seqlens is None else (int(sum(seqlens)),)

    def draw(*tail):
        return torch.randn(*lead, *tail, generator=g, dtype=torch.float32)

    q_nope, q_pe, k_nope, k_pe, v = draw(heads, 128), draw(heads, 64), draw(heads, 128), draw(1, 64), draw(heads, 128)
    dout = draw(heads, 128) * dout_std
    if seqlens is None:
        positions = torch.arange(seq)
        q_pe, k_pe = rope(q_pe, positions), rope(k_pe, positions)
        cu = None
    else:
        positions = torch.cat([torch.arange(int(n)) for n in seqlens])
        q_pe, k_pe = rope(q_pe, positions), rope(k_pe, positions)
        cu = torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0)), dtype=torch.int32)
    tensors = tuple(t.to(dtype).contiguous() for t in (q_nope, q_pe, k_nope, k_pe, v, dout))
    return tensors + ((cu,) if seqlens is not None else ())


def varlen_lengths(seed=4, count=16, low=512, high=32768):
    """Sequence lengths log-uniform in [low, high] from a CPU generator."""
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(count, generator=g, dtype=torch.float64)
    return [int(round(math.exp(math.log(low) + float(x) * (math.log(high) - math.log(low))))) for x in u]


def decode_inputs(seed=3, batch=64, heads=128, low=1024, high=32768, page=64,
                  lengths=None):
    """Packed query [B,1,H,576], paged cache [pages,64,1,576] ~ N(0,1) bf16,
    lengths uniform in [low, high], randomly permuted page table."""
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
