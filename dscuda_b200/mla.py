"""Host side of the MLA path: torch tensors in, C-ABI calls out.

The functions mirror what the reference's `benchmarks/mla.py:79-117` does by
hand (raw `data_ptr()`s, the current stream, caller-owned outputs and
workspace).  They allocate outputs with torch, launch on the current stream and
return without synchronising.  Inputs must be contiguous CUDA tensors; bf16
unless stated.  No CPU fallback exists.
"""

from __future__ import annotations

import torch

from .library import checked, library  # noqa: F401 (re-exported for callers)


def prefill_backward_launches(batch, max_seq, total, heads, packed=False) -> int:
    """Kernels one `dscuda_mla_prefill_backward` call launches: the delta pre-pass, the dk_pe sum, and
    the two main kernels (dense batches: once per group of heads that fits the scratch limit)."""
    return library("mla").dscuda_mla_prefill_backward_launches(batch, max_seq, total, heads, int(packed))


def prefill_backward_scratch_limit(limit_bytes=-1) -> int:
    """Sets the workspace the dense backward may spend on dS^T (`dscuda_mla_prefill_backward_scratch_limit`);
    returns the previous limit.  0 selects the recomputing dQ kernel, a negative value only reads."""
    return library("mla").dscuda_mla_prefill_backward_scratch_limit(limit_bytes)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor):
    return None if tensor is None else tensor.data_ptr()


def _require(*tensors):
    for tensor in tensors:
        if tensor is None:
            continue
        if not tensor.is_cuda:
            raise RuntimeError("dscuda_b200 runs on CUDA tensors only; there is no CPU path")
        if not tensor.is_contiguous():
            raise ValueError("tensors must be contiguous")


def mla_forward(query, query_rope, latent, key_rope, scale):
    """Absorbed causal forward (`dscuda_mla_forward`).
    query [B,T,H,512], query_rope [B,T,H,64], latent [B,T,512], key_rope [B,T,64]
    -> (output [B,T,H,512] bf16, lse [B,H,T] fp32)."""
    _require(query, query_rope, latent, key_rope)
    b, t, h, c = query.shape
    r = query_rope.shape[-1]
    output = torch.empty_like(query)
    lse = torch.empty(b, h, t, device=query.device, dtype=torch.float32)
    lib = library("mla")
    checked(lib, "mla", lib.dscuda_mla_forward(
        _ptr(output), _ptr(lse), _ptr(query), _ptr(query_rope), _ptr(latent), _ptr(key_rope),
        b, t, h, c, r, scale, _stream()))
    return output, lse


def mla_backward(dout, output, lse, query, query_rope, latent, key_rope, scale):
    """Absorbed backward (`dscuda_mla_backward`) -> (dquery, dquery_rope, dlatent, dkey_rope)."""
    _require(dout, output, lse, query, query_rope, latent, key_rope)
    b, t, h, c = query.shape
    r = query_rope.shape[-1]
    grads = tuple(torch.empty_like(x) for x in (query, query_rope, latent, key_rope))
    lib = library("mla")
    checked(lib, "mla", lib.dscuda_mla_backward(
        *map(_ptr, grads), _ptr(dout), _ptr(output), _ptr(lse), _ptr(query), _ptr(query_rope), _ptr(latent), _ptr(key_rope),
        b, t, h, c, r, scale, _stream()))
    return grads


def decode_workspace(batch, heads, splits, rank=512, device="cuda"):
    lib = library("mla")
    return torch.empty(lib.dscuda_mla_workspace_elements(batch, heads, splits, rank), device=device, dtype=torch.float32)


def decode_splits(lengths, heads=128, minimum=8, clusters=74, maximum=64) -> int:
    """Partial slots per (sequence, head) that let the decode kernel cut the batch's 128-key tiles into equal ranges,
    one per pair of SMs.  The kernel never makes a range shorter than longest sequence / (splits - 1) tiles (a sequence
    may not spread over more ranges than it has slots), so a small batch of long sequences needs more slots than the
    reference harness's 8 to keep every SM pair busy.  `lengths`: cached tokens per sequence (a list or a CPU tensor)."""
    tiles = [(int(n) + 127) // 128 for n in lengths]
    head_tiles = (heads + 127) // 128
    per_range = max(1, -(-sum(tiles) * head_tiles // clusters))
    return max(minimum, min(maximum, 1 + -(-max(tiles, default=1) // per_range)))


def mla_decode(query, paged_cache, block_table, lengths, scale, splits=8, workspace=None, output=None, lse=None, checked_pages=False):
    """Paged decode (`dscuda_mla_decode`; `dscuda_mla_decode_checked` with `checked_pages`, which also
    passes the number of cache pages so that a page number outside the cache is replaced and reported).
    query [B,1,H,576], paged_cache [blocks,page,1,576], block_table [B,pages] int32,
    lengths [B] int32 -> (output [B,1,H,512] bf16, lse [B,H,1] fp32)."""
    _require(query, paged_cache, block_table, lengths, workspace)
    b, _, h, width = query.shape
    rank, rope = 512, width - 512
    page_size = paged_cache.shape[1]
    if workspace is None:
        workspace = decode_workspace(b, h, splits, rank, query.device)
    if output is None:
        output = torch.empty(b, 1, h, rank, device=query.device, dtype=torch.bfloat16)
    if lse is None:
        lse = torch.empty(b, h, 1, device=query.device, dtype=torch.float32)
    lib = library("mla")
    if checked_pages:
        checked(lib, "mla", lib.dscuda_mla_decode_checked(
            _ptr(output), _ptr(lse), _ptr(query), _ptr(paged_cache), _ptr(block_table), _ptr(lengths), _ptr(workspace),
            b, h, rank, rope, page_size, block_table.shape[1], paged_cache.shape[0], splits, scale, _stream()))
    else:
        checked(lib, "mla", lib.dscuda_mla_decode(
            _ptr(output), _ptr(lse), _ptr(query), _ptr(paged_cache), _ptr(block_table), _ptr(lengths), _ptr(workspace),
            b, h, rank, rope, page_size, block_table.shape[1], splits, scale, _stream()))
    return output, lse


def cache_append(paged_cache, kv_latent, key_rope, block_table, start_positions=None, token_counts=None):
    """Writes new tokens into the paged cache in place (`dscuda_mla_cache_append`).
    paged_cache [blocks,page,1,576], kv_latent [B,T,512], key_rope [B,T,64] bf16, block_table [B,pages] int32;
    start_positions / token_counts [B] int32 or None (0 / all T rows).  Token t of sequence b lands at
    position start_positions[b] + t."""
    _require(paged_cache, kv_latent, key_rope, block_table, start_positions, token_counts)
    b, t, rank = kv_latent.shape
    lib = library("mla")
    checked(lib, "mla", lib.dscuda_mla_cache_append(
        _ptr(paged_cache), _ptr(kv_latent), _ptr(key_rope), _ptr(block_table), _ptr(start_positions), _ptr(token_counts),
        b, t, rank, key_rope.shape[-1], paged_cache.shape[1], block_table.shape[1], paged_cache.shape[0], _stream()))
    return paged_cache


FP8_CACHE_ROW_BYTES = 656       # 512 e4m3 + four fp32 group scales + 64 bf16 rotary values


def cache_append_fp8(paged_fp8_cache, kv_latent, key_rope, block_table, start_positions=None, token_counts=None):
    """`cache_append` into the FP8 cache (`dscuda_mla_cache_append_fp8`): paged_fp8_cache [blocks, page, 656] uint8."""
    _require(paged_fp8_cache, kv_latent, key_rope, block_table, start_positions, token_counts)
    if paged_fp8_cache.dtype != torch.uint8 or paged_fp8_cache.shape[-1] != FP8_CACHE_ROW_BYTES:
        raise ValueError("the FP8 cache is a uint8 tensor [blocks, page, 656]")
    b, t, rank = kv_latent.shape
    lib = library("mla")
    checked(lib, "mla", lib.dscuda_mla_cache_append_fp8(
        _ptr(paged_fp8_cache), _ptr(kv_latent), _ptr(key_rope), _ptr(block_table), _ptr(start_positions), _ptr(token_counts),
        b, t, rank, key_rope.shape[-1], paged_fp8_cache.shape[1], block_table.shape[1], paged_fp8_cache.shape[0], _stream()))
    return paged_fp8_cache


def cache_dequantize_fp8(paged_fp8_cache, paged_cache=None, first_row=0, rows=None):
    """FP8 cache rows -> the bf16 cache layout the decode reads (`dscuda_mla_cache_dequantize_fp8`).
    Rows are physical (page * page_size + slot); by default the whole cache."""
    _require(paged_fp8_cache, paged_cache)
    blocks, page, _ = paged_fp8_cache.shape
    if paged_cache is None:
        paged_cache = torch.empty(blocks, page, 1, 576, device=paged_fp8_cache.device, dtype=torch.bfloat16)
    if rows is None:
        rows = blocks * page - first_row
    lib = library("mla")
    checked(lib, "mla", lib.dscuda_mla_cache_dequantize_fp8(_ptr(paged_cache), _ptr(paged_fp8_cache), first_row, rows, _stream()))
    return paged_cache


def rope_apply(q_pe=None, k_pe=None, positions=None, theta=10000.0):
    """Rotary embedding in place (`dscuda_mla_rope_apply`) of q_pe [..., H, 64] and/or k_pe [..., 1, 64] (bf16).
    `positions` int32 [rows] on the device, or None for dense [B, S, ...] tensors (position = index along S)."""
    _require(q_pe, k_pe, positions)
    anchor = q_pe if q_pe is not None else k_pe
    if anchor is None:
        raise ValueError("nothing to rotate")
    heads = q_pe.shape[-2] if q_pe is not None else 1
    rows = anchor.numel() // (anchor.shape[-2] * anchor.shape[-1])
    if positions is None and anchor.dim() != 4:
        raise ValueError("packed tensors need explicit positions")
    sequence = anchor.shape[1] if positions is None else 0
    lib = library("mla")
    checked(lib, "mla", lib.dscuda_mla_rope_apply(_ptr(q_pe), _ptr(k_pe), _ptr(positions), rows, heads, sequence, anchor.shape[-1], theta,
                                                   _stream()))
    return q_pe, k_pe


def up_project(kv_latent, w_uk, w_uv, heads):
    """Per-head keys and values from the latent (`dscuda_mla_up_project`): kv_latent [..., 512],
    w_uk / w_uv [H*128, 512] -> (k_nope [..., H, 128], v [..., H, 128])."""
    _require(kv_latent, w_uk, w_uv)
    rows = kv_latent.numel() // kv_latent.shape[-1]
    lead = kv_latent.shape[:-1]
    k_nope = torch.empty(*lead, heads, 128, device=kv_latent.device, dtype=torch.bfloat16)
    v = torch.empty_like(k_nope)
    lib = library("mla")
    checked(lib, "mla", lib.dscuda_mla_up_project(_ptr(k_nope), _ptr(v), _ptr(kv_latent), _ptr(w_uk), _ptr(w_uv), rows, heads, _stream()))
    return k_nope, v


def absorb_query(q_nope, w_uk):
    """W_UK folded into the query (`dscuda_mla_absorb_query`): q_nope [..., H, 128], w_uk [H*128, 512] -> q_latent [..., H, 512]."""
    _require(q_nope, w_uk)
    heads = q_nope.shape[-2]
    rows = q_nope.numel() // (heads * q_nope.shape[-1])
    q_latent = torch.empty(*q_nope.shape[:-1], 512, device=q_nope.device, dtype=torch.bfloat16)
    lib = library("mla")
    checked(lib, "mla", lib.dscuda_mla_absorb_query(_ptr(q_latent), _ptr(q_nope), _ptr(w_uk), rows, heads, _stream()))
    return q_latent


def unabsorb_output(output_latent, w_uv):
    """W_UV applied to the latent output (`dscuda_mla_unabsorb_output`): o_latent [..., H, 512], w_uv [H*128, 512] -> out [..., H, 128]."""
    _require(output_latent, w_uv)
    heads = output_latent.shape[-2]
    rows = output_latent.numel() // (heads * output_latent.shape[-1])
    out = torch.empty(*output_latent.shape[:-1], 128, device=output_latent.device, dtype=torch.bfloat16)
    lib = library("mla")
    checked(lib, "mla", lib.dscuda_mla_unabsorb_output(_ptr(out), _ptr(output_latent), _ptr(w_uv), rows, heads, _stream()))
    return out


def _prefill_dims(q_nope, cu_seqlens, max_seqlen):
    if cu_seqlens is None:
        b, s, h, _ = q_nope.shape
        return b, s, b * s, h
    total, h, _ = q_nope.shape
    if max_seqlen is None:
        raise ValueError("packed layout needs max_seqlen (an upper bound on the longest sequence)")
    return cu_seqlens.numel() - 1, int(max_seqlen), total, h


def prefill_forward(q_nope, q_pe, k_nope, k_pe, v, scale, cu_seqlens=None, max_seqlen=None, output=None, lse=None):
    """Non-absorbed causal forward (`dscuda_mla_prefill_forward`).
    Dense [B,S,H,*] or packed [total,H,*] with int32 cu_seqlens on the device.
    -> (output like v, lse [B,H,S] or [H,total])."""
    _require(q_nope, q_pe, k_nope, k_pe, v, cu_seqlens)
    batch, max_seq, total, heads = _prefill_dims(q_nope, cu_seqlens, max_seqlen)
    if output is None:
        output = torch.empty_like(v)
    if lse is None:
        shape = (batch, heads, max_seq) if cu_seqlens is None else (heads, total)
        lse = torch.empty(shape, device=v.device, dtype=torch.float32)
    lib = library("mla")
    checked(lib, "mla", lib.dscuda_mla_prefill_forward(
        _ptr(output), _ptr(lse), _ptr(q_nope), _ptr(q_pe), _ptr(k_nope), _ptr(k_pe), _ptr(v), _ptr(cu_seqlens),
        batch, max_seq, total, heads, q_nope.shape[-1], q_pe.shape[-1], v.shape[-1], scale, _stream()))
    return output, lse


def prefill_backward_workspace(batch, max_seq, total, heads, device="cuda"):
    lib = library("mla")
    return torch.empty(lib.dscuda_mla_prefill_backward_workspace_bytes(batch, max_seq, total, heads),
                       device=device, dtype=torch.uint8)


def prefill_backward(dout, output, lse, q_nope, q_pe, k_nope, k_pe, v, scale, cu_seqlens=None, max_seqlen=None,
                     workspace=None, grads=None):
    """Non-absorbed backward (`dscuda_mla_prefill_backward`)
    -> (dq [...,H,192], dk_nope [...,H,128], dk_pe [...,1,64], dv [...,H,128])."""
    _require(dout, output, lse, q_nope, q_pe, k_nope, k_pe, v, cu_seqlens, workspace)
    batch, max_seq, total, heads = _prefill_dims(q_nope, cu_seqlens, max_seqlen)
    if workspace is None:
        workspace = prefill_backward_workspace(batch, max_seq, total, heads, v.device)
    if grads is None:
        lead = q_nope.shape[:-1]
        dq = torch.empty(*lead, 192, device=v.device, dtype=torch.bfloat16)
        grads = (dq, torch.empty_like(k_nope), torch.empty_like(k_pe), torch.empty_like(v))
    lib = library("mla")
    checked(lib, "mla", lib.dscuda_mla_prefill_backward(
        *map(_ptr, grads), _ptr(dout), _ptr(output), _ptr(lse), _ptr(q_nope), _ptr(q_pe), _ptr(k_nope), _ptr(k_pe), _ptr(v),
        _ptr(cu_seqlens), _ptr(workspace), batch, max_seq, total, heads,
        q_nope.shape[-1], q_pe.shape[-1], v.shape[-1], scale, _stream()))
    return grads


def flash_forward(query, key, value, scale):
    """Causal D=128 GQA forward (`dscuda_flash_forward`).
    query [B,T,Hq,128], key/value [B,T,Hkv,128] -> (output, lse [B,Hq,T])."""
    _require(query, key, value)
    b, t, hq, d = query.shape
    output = torch.empty_like(query)
    lse = torch.empty(b, hq, t, device=query.device, dtype=torch.float32)
    lib = library("flash_attention")
    checked(lib, "flash", lib.dscuda_flash_forward(
        _ptr(output), _ptr(lse), _ptr(query), _ptr(key), _ptr(value), b, t, hq, key.shape[2], d, scale, _stream()))
    return output, lse


def device_status(reset=False) -> int:
    """0 when no kernel of this library has hit a bounded-wait timeout."""
    mla = library("mla").dscuda_mla_device_status(int(reset))
    flash = library("flash_attention").dscuda_flash_device_status(int(reset))
    return mla or flash
