"""Checks of kernel outputs against the CPU oracle at sizes where the full problem is too large
for the CPU.  TEST INFRASTRUCTURE ONLY, like the rest of `oracle/`: the benchmark (`bench.py`) and
the harness (`dscuda_b200.suite`) call these after running the kernels, the way the reference's
harness compares with its PyTorch expressions before and after timing
(benchmarks/common.py:84-85,109-110).  Nothing here computes a result that is returned to a user.

Bars (BASELINE acceptance): forward output max|err| <= 1e-2 max|ref|, LSE within 1e-3, gradient
relative L2 <= 1e-2.  Every function returns {check name: bool}.
"""
from __future__ import annotations

import torch

from . import mla_oracle as oracle

OUT_BAR, LSE_BAR, GRAD_BAR = 1e-2, 1e-3, 1e-2


def _rel(got, ref):
    return float((got.double() - ref.double()).norm() / ref.double().norm().clamp_min(1e-30))


def _out_ok(got, ref):
    return float((got.double() - ref.double()).abs().max()) <= OUT_BAR * float(ref.abs().max())


def dense_slices(tensors, out, lse, grads, scale, batch_index=0, head=0, rows=256, keys=128, keys_all_heads=32):
    """Dense [B,S,H,*] problem (device or host tensors): one (batch, head) on the last `rows` query
    rows (O, LSE, dQ) and the first `keys` keys (dK_nope, dV); dK_pe, which sums over heads, on the
    first `keys_all_heads` keys with every head.  `grads` None: forward only."""
    b = slice(batch_index, batch_index + 1)
    h = slice(head, head + 1)
    seq = tensors["q_nope"].shape[1]

    def one(t):
        return t[b, :, h].float().cpu().contiguous()

    dense = [one(tensors["q_nope"]), one(tensors["q_pe"]), one(tensors["k_nope"]), tensors["k_pe"][b].float().cpu().contiguous(), one(tensors["v"])]
    window = (max(0, seq - rows), seq)
    checks = {}
    if grads is not None:
        ref_out, ref_lse, ref_dq = oracle.prefill_row_block(*dense, scale, window, one(tensors["dout"]))
        checks["dq"] = _rel(grads[0][b, window[0]:window[1], h].float().cpu(), ref_dq) <= GRAD_BAR
    else:
        ref_out, ref_lse = oracle.prefill_row_block(*dense, scale, window)
    checks["out"] = _out_ok(out[b, window[0]:window[1], h].float().cpu(), ref_out)
    checks["lse"] = float((lse[b, h, window[0]:window[1]].cpu() - ref_lse).abs().max()) <= LSE_BAR
    if grads is not None:
        block = (0, min(keys, seq))
        ref_dk, _, ref_dv = oracle.prefill_key_block(one(tensors["dout"]), one(out), lse[b, h].cpu().contiguous(), *dense, scale, block)
        checks["dk_nope"] = _rel(grads[1][b, block[0]:block[1], h].float().cpu(), ref_dk) <= GRAD_BAR
        checks["dv"] = _rel(grads[3][b, block[0]:block[1], h].float().cpu(), ref_dv) <= GRAD_BAR
        block = (0, min(keys_all_heads, seq))
        every = [tensors[k][b].float().cpu().contiguous() for k in ("q_nope", "q_pe", "k_nope", "k_pe", "v")]
        _, ref_dk_pe, _ = oracle.prefill_key_block(tensors["dout"][b].float().cpu(), out[b].float().cpu(), lse[b].cpu().contiguous(), *every, scale,
                                                   block)
        checks["dk_pe"] = _rel(grads[2][b, block[0]:block[1]].float().cpu(), ref_dk_pe) <= GRAD_BAR
    return checks


def dense_full(tensors, out, lse, grads, scale):
    """Small dense problems: everything against the full restatement."""
    cpu = {k: v.cpu() for k, v in tensors.items()}
    inputs = [cpu[k] for k in ("q_nope", "q_pe", "k_nope", "k_pe", "v")]
    ref_out, ref_lse = oracle.prefill_forward(*inputs, scale)
    checks = {"out": _out_ok(out.float().cpu(), ref_out), "lse": float((lse.cpu() - ref_lse).abs().max()) <= LSE_BAR}
    if grads is not None:
        ref = oracle.prefill_backward(cpu["dout"], out.cpu(), lse.cpu(), *inputs, scale)
        for name, got, want in zip(("dq", "dk_nope", "dk_pe", "dv"), grads, ref):
            checks[name] = _rel(got.float().cpu(), want) <= GRAD_BAR
    return checks


def packed_slices(tensors, cu_seqlens, out, lse, grads, scale, sequence, rows=256, keys=128):
    """Packed [total,H,*] problem: sequence number `sequence` as its own dense causal problem, on its
    last `rows` query rows and first `keys` keys, every head of the call."""
    a, b = int(cu_seqlens[sequence]), int(cu_seqlens[sequence + 1])
    n = b - a
    dense = [tensors[k][a:b][None].float().cpu().contiguous() for k in ("q_nope", "q_pe", "k_nope", "k_pe", "v")]
    dout = tensors["dout"][a:b][None].float().cpu()
    window = (max(0, n - rows), n)
    ref_out, ref_lse, ref_dq = oracle.prefill_row_block(*dense, scale, window, dout)
    checks = {"out": _out_ok(out[a + window[0]:b].float().cpu(), ref_out[0]),
              "lse": float((lse[:, a + window[0]:b].cpu() - ref_lse[0]).abs().max()) <= LSE_BAR,
              "dq": _rel(grads[0][a + window[0]:b].float().cpu(), ref_dq[0]) <= GRAD_BAR}
    block = (0, min(keys, n))
    ref_dk, ref_dk_pe, ref_dv = oracle.prefill_key_block(dout, out[a:b][None].float().cpu(), lse[:, a:b][None].cpu().contiguous(), *dense, scale, block)
    checks["dk_nope"] = _rel(grads[1][a:a + block[1]].float().cpu(), ref_dk[0]) <= GRAD_BAR
    checks["dk_pe"] = _rel(grads[2][a:a + block[1]].float().cpu(), ref_dk_pe[0]) <= GRAD_BAR
    checks["dv"] = _rel(grads[3][a:a + block[1]].float().cpu(), ref_dv[0]) <= GRAD_BAR
    return checks


def decode_sequences(query, cache, table, lengths, out, lse, scale, picks):
    """Host inputs of a paged decode call and its device outputs: the sequences `picks`."""
    picks = list(picks)
    ref_out, ref_lse = oracle.paged_decode(query[picks], cache, table[picks], lengths[picks], scale)
    got_out, got_lse = out[picks].float().cpu(), lse[picks].cpu()
    return {"out": _out_ok(got_out, ref_out), "lse": float((got_lse - ref_lse).abs().max()) <= LSE_BAR}
