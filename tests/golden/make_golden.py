"""Generate the golden fixtures in this directory from the reference itself.

Run once where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's `reference/python/mla.py` (never copied into this
repository), runs `mla_forward` / `mla_backward` on small seeded CPU inputs and
stores inputs and outputs as compressed `.npz` files.  bf16 tensors are stored
as their raw 16-bit patterns (`*_bf16` keys, int16).

Fixtures:

* `absorbed_*.npz`  - the reference contract as is (C=512, R=64), shapes taken
  from the reference's own test list (`benchmarks/mla.py:36-39`), input scale
  0.25 and dO scale 0.2 as there (`:51,108`), scale = (C+R)^-0.5 as a C float
  (`:55`).  Holds O, LSE from `mla_forward`, the four gradients from
  `mla_backward`, and the gradients `torch.autograd` gives through
  `mla_forward` (what `benchmarks/mla.py:109-110` calls expected).
* `decode_*.npz`    - `mla_forward` with one query token and the length mask of
  `benchmarks/mla.py:58-66`; cache packed by `pack_cache`.
* `prefill_embed_*.npz` - the non-absorbed contract computed BY THE REFERENCE
  through a head-fold / zero-pad embedding: heads become batch entries,
  query' = [q_nope | 0], latent' = [k_nope | v], so that `mla_forward` yields
  LSE directly and O in the second half of its output, and `mla_backward` with
  dout' = [0 | dO] yields dq_nope, dq_pe, [dk_nope | dv] and per-head dk_pe.
"""

import ctypes
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent


def bits(t):
    return t.contiguous().view(torch.int16).numpy()


def absorbed_case(mla, name, b, t, h, seed):
    g = torch.Generator().manual_seed(seed)
    c, r = 512, 64
    shapes = ((b, t, h, c), (b, t, h, r), (b, t, c), (b, t, r))
    inputs = tuple((torch.randn(s, generator=g) * .25).bfloat16() for s in shapes)
    dout = (torch.randn((b, t, h, c), generator=g) * .2).bfloat16()
    scale = ctypes.c_float((c + r) ** -.5).value
    mask = torch.ones(t, t, dtype=torch.bool).tril()
    oracle = tuple(x.float().detach().requires_grad_() for x in inputs)
    out_ag, lse_ag = mla.mla_forward(*oracle, scale, mask)
    autograd = tuple(x.bfloat16() for x in torch.autograd.grad(out_ag, oracle, dout))
    out, lse = mla.mla_forward(*inputs, scale, mask)
    grads = mla.mla_backward(dout, out, lse, *inputs, scale, mask)
    np.savez_compressed(
        HERE / f"absorbed_{name}.npz", scale=np.float32(scale),
        query_bf16=bits(inputs[0]), query_rope_bf16=bits(inputs[1]),
        latent_bf16=bits(inputs[2]), key_rope_bf16=bits(inputs[3]), dout_bf16=bits(dout),
        out_bf16=bits(out), lse=lse.numpy(),
        dquery_bf16=bits(grads[0]), dquery_rope_bf16=bits(grads[1]),
        dlatent_bf16=bits(grads[2]), dkey_rope_bf16=bits(grads[3]),
        ag_dquery_bf16=bits(autograd[0]), ag_dquery_rope_bf16=bits(autograd[1]),
        ag_dlatent_bf16=bits(autograd[2]), ag_dkey_rope_bf16=bits(autograd[3]))


def decode_case(mla, name, b, t, h, seed):
    g = torch.Generator().manual_seed(seed)
    c, r = 512, 64
    query = (torch.randn((b, 1, h, c + r), generator=g) * .25).bfloat16()
    kv = (torch.randn((b, t, c + r), generator=g) * .25).bfloat16()
    lengths = tuple(max(1, t - i * t // (2 * b)) for i in range(b))
    lengths = (1,) + lengths[1:-1] + (t,)
    scale = ctypes.c_float((c + r) ** -.5).value
    length_tensor = torch.tensor(lengths, dtype=torch.int32)
    mask = (torch.arange(t)[None] < length_tensor[:, None])[:, None, None]
    out, lse = mla.mla_forward(query[..., :c], query[..., c:], kv[..., :c], kv[..., c:], scale, mask)
    cache, table = mla.pack_cache(kv, 64)
    np.savez_compressed(
        HERE / f"decode_{name}.npz", scale=np.float32(scale),
        query_bf16=bits(query), kv_bf16=bits(kv), lengths=length_tensor.numpy(),
        cache_bf16=bits(cache), table=table.numpy(), out_bf16=bits(out), lse=lse.numpy())


def prefill_embed_case(mla, name, b, s, h, seed):
    g = torch.Generator().manual_seed(seed)
    shapes = ((b, s, h, 128), (b, s, h, 64), (b, s, h, 128), (b, s, 1, 64), (b, s, h, 128))
    q_nope, q_pe, k_nope, k_pe, v = ((torch.randn(x, generator=g) * .5).bfloat16() for x in shapes)
    dout = (torch.randn((b, s, h, 128), generator=g) * .2).bfloat16()
    scale = ctypes.c_float(192 ** -.5).value
    mask = torch.ones(s, s, dtype=torch.bool).tril()

    def fold(x):                                    # [B,S,H,D] -> [B*H,S,1,D]
        return x.permute(0, 2, 1, 3).reshape(b * h, s, 1, x.shape[-1])

    zeros = torch.zeros(b * h, s, 1, 128, dtype=torch.bfloat16)
    query = torch.cat((fold(q_nope), zeros), -1)
    query_rope = fold(q_pe)
    latent = torch.cat((fold(k_nope), fold(v)), -1)[:, :, 0]
    key_rope = k_pe[:, :, 0].repeat_interleave(h, dim=0)
    out, lse = mla.mla_forward(query, query_rope, latent, key_rope, scale, mask)
    dout_e = torch.cat((zeros, fold(dout)), -1)
    dquery, dquery_rope, dlatent, dkey_rope = mla.mla_backward(
        dout_e, out, lse, query, query_rope, latent, key_rope, scale, mask)

    def unfold(x):                                  # [B*H,S,D] -> [B,S,H,D]
        return x.reshape(b, h, s, x.shape[-1]).permute(0, 2, 1, 3).contiguous()

    o = unfold(out[:, :, 0, 128:])
    dq = torch.cat((unfold(dquery[:, :, 0, :128]), unfold(dquery_rope[:, :, 0])), -1)
    dk_nope, dv = unfold(dlatent[..., :128]), unfold(dlatent[..., 128:])
    # per-head dk_pe from the reference is already bf16-rounded; the head sum is taken in fp32
    dk_pe_heads = unfold(dkey_rope)
    np.savez_compressed(
        HERE / f"prefill_embed_{name}.npz", scale=np.float32(scale),
        q_nope_bf16=bits(q_nope), q_pe_bf16=bits(q_pe), k_nope_bf16=bits(k_nope),
        k_pe_bf16=bits(k_pe), v_bf16=bits(v), dout_bf16=bits(dout),
        out_bf16=bits(o), lse=lse.reshape(b, h, s).numpy(),
        dq_bf16=bits(dq), dk_nope_bf16=bits(dk_nope), dv_bf16=bits(dv),
        dk_pe_heads_bf16=bits(dk_pe_heads))


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of the reference checkout>")
    reference = pathlib.Path(sys.argv[1])
    sys.path.insert(0, str(reference))
    from reference.python import mla
    torch.manual_seed(0)
    absorbed_case(mla, "b1_t1_h1", 1, 1, 1, seed=11)
    absorbed_case(mla, "b2_t17_h3", 2, 17, 3, seed=12)
    absorbed_case(mla, "b1_t65_h4", 1, 65, 4, seed=13)
    decode_case(mla, "b2_t23_h3", 2, 23, 3, seed=21)
    decode_case(mla, "b2_t65_h64", 2, 65, 64, seed=22)
    decode_case(mla, "b3_t129_h16", 3, 129, 16, seed=23)
    prefill_embed_case(mla, "b2_s37_h3", 2, 37, 3, seed=31)
    prefill_embed_case(mla, "b1_s130_h2", 1, 130, 2, seed=32)
    for path in sorted(HERE.glob("*.npz")):
        print(path.name, path.stat().st_size)


if __name__ == "__main__":
    main()
