"""Generates the committed golden fixtures in this directory.

    python tests/golden/make_golden.py

The reference ships no golden vectors and its Mojo kernels cannot run here, so the fixtures pin
what the reference's own GPU tests treat as truth: torch's CPU fp32 scaled-dot-product attention
on seeded inputs.  The cases reuse the reference tests' seeds, shapes and input scaling
(tests/test_eager_kernels.py:9478-9501: seeds 20260718 / 20260719, fused QKV ``randn * 0.25``,
``grad_output = randn``; :9609-9683 and :9697-9775: BHSD and partial-tail shapes with seeds
``20260816 + S`` / ``20260817 + S``), kept small so each file is a few hundred KB.
Inputs are stored already rounded to the case dtype (as fp32 arrays); outputs are fp32.

The ``ext_*`` fixtures cover what lies beyond the reference's gate: a causal mask over unequal
lengths in both alignments (top-left: torch's rule; bottom-right: fa4_fwd_kernel.mojo:266-273)
and dropout.  Their expected values come from the float64 restatement (oracle/restatement.py),
the dropout mask from the numpy Philox4x32-10 (oracle/philox.py), stored bit-packed, so the
torch-side oracle, the mask generator and the kernels are all pinned against them.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def fused_qkv_case(seed, batch, seqlen, heads, head_dim, dtype):
    width = heads * head_dim
    g = torch.Generator().manual_seed(seed)
    fused = (torch.randn(batch, seqlen, 3 * width, generator=g, dtype=torch.float32) * 0.25).to(dtype)
    dout = torch.randn(batch, heads, seqlen, head_dim, generator=g, dtype=torch.float32).to(dtype)
    q, k, v = (p.view(batch, seqlen, heads, head_dim).transpose(1, 2) for p in fused.split(width, dim=2))
    return fused, q, k, v, dout


def reference_outputs(q, k, v, dout, causal, scale):
    from oracle import sdpa_oracle as O

    out, lse = O.sdpa_forward(q, k, v, causal, scale)
    _, dq, dk, dv = O.sdpa_backward(q, k, v, dout, causal, scale)
    return out, lse, dq, dk, dv


def main():
    cases = {}
    # nanoGPT-style fused-QKV cases (causal, fwd+bwd)
    for name, seed, b, s, h, d, dtype in (
        ("fused_bf16_d64", 20260718, 1, 128, 4, 64, torch.bfloat16),
        ("fused_f16_d128", 20260718, 1, 128, 2, 128, torch.float16),
        ("fused_bf16_d128_b2", 20260719, 2, 256, 1, 128, torch.bfloat16),
    ):
        fused, q, k, v, dout = fused_qkv_case(seed, b, s, h, d, dtype)
        out, lse, dq, dk, dv = reference_outputs(q, k, v, dout, True, d ** -0.5)
        cases[name] = dict(fused=fused.float().numpy(), dout=dout.float().numpy(), out=out.numpy(), lse=lse.numpy(),
                           dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy(),
                           meta=np.array([b, h, h, s, d, 1, {torch.bfloat16: 1, torch.float16: 2}[dtype]]))
    # partial-tail BHSD forward (out + lse), and a GQA / non-causal / fp32 case each
    for name, seed, b, hq, hkv, s, d, causal, dtype in (
        ("tail_bf16_s193", 20260817 + 193, 1, 1, 1, 193, 64, True, torch.bfloat16),
        ("gqa_bf16_s256", 20260816 + 256, 1, 2, 1, 256, 128, True, torch.bfloat16),
        ("noncausal_f16_s130", 20260816 + 130, 1, 1, 1, 130, 128, False, torch.float16),
        ("fp32_s256", 0, 1, 1, 1, 256, 64, True, torch.float32),
    ):
        g = torch.Generator().manual_seed(seed)
        q = (torch.randn(b, hq, s, d, generator=g) * 0.25).to(dtype)
        k = (torch.randn(b, hkv, s, d, generator=g) * 0.25).to(dtype)
        v = (torch.randn(b, hkv, s, d, generator=g) * 0.25).to(dtype)
        dout = torch.randn(b, hq, s, d, generator=g).to(dtype)
        out, lse, dq, dk, dv = reference_outputs(q, k, v, dout, causal, d ** -0.5)
        code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[dtype]
        cases[name] = dict(q=q.float().numpy(), k=k.float().numpy(), v=v.float().numpy(), dout=dout.float().numpy(),
                           out=out.numpy(), lse=lse.numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy(),
                           meta=np.array([b, hq, hkv, s, d, int(causal), code]))
    from oracle import restatement as R
    from oracle.philox import keep_mask

    # name, seed, b, hq, hkv, sq, sk, d, mode, dtype, (p, philox seed, philox offset)
    for name, seed, b, hq, hkv, sq, sk, d, mode, dtype, drop in (
        ("ext_bottom_right_bf16", 20260920, 1, 4, 2, 96, 200, 64, 2, torch.bfloat16, None),
        ("ext_top_left_f16", 20260921, 1, 2, 2, 200, 96, 128, 1, torch.float16, None),
        ("ext_more_queries_than_keys_bf16", 20260922, 1, 2, 1, 160, 72, 64, 2, torch.bfloat16, None),
        ("ext_dropout_bf16", 20260923, 2, 2, 1, 130, 130, 64, 1, torch.bfloat16, (0.25, 0x0123456789ABCDEF, 40)),
    ):
        g = torch.Generator().manual_seed(seed)
        q = (torch.randn(b, hq, sq, d, generator=g) * 0.5).to(dtype)
        k = (torch.randn(b, hkv, sk, d, generator=g) * 0.5).to(dtype)
        v = (torch.randn(b, hkv, sk, d, generator=g) * 0.5).to(dtype)
        dout = torch.randn(b, hq, sq, d, generator=g).to(dtype)
        f64 = lambda t: t.float().numpy().astype(np.float64)
        keep, keep_scale = (None, 1.0) if drop is None else keep_mask(b, hq, sq, sk, *drop)
        out, lse = R.forward(f64(q), f64(k), f64(v), mode, d ** -0.5, keep, keep_scale)
        dq, dk, dv = R.backward(f64(q), f64(k), f64(v), f64(dout), mode, d ** -0.5, keep, keep_scale)
        code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[dtype]
        arrays = dict(q=q.float().numpy(), k=k.float().numpy(), v=v.float().numpy(), dout=dout.float().numpy(),
                      out=out.astype(np.float32), lse=lse.astype(np.float32), dq=dq.astype(np.float32),
                      dk=dk.astype(np.float32), dv=dv.astype(np.float32),
                      meta=np.array([b, hq, hkv, sq, sk, d, mode, code]))
        if drop is not None:
            arrays["keep_bits"] = np.packbits(keep)
            arrays["drop"] = np.array([int(round(drop[0] * 1e6)), drop[1] & 0xFFFFFFFF, drop[1] >> 32, drop[2]],
                                      dtype=np.uint64)
        cases[name] = arrays
    for name, arrays in cases.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **{k: np.asarray(v) for k, v in arrays.items()})
        print(name, {k: tuple(np.asarray(v).shape) for k, v in arrays.items()})


if __name__ == "__main__":
    main()
