"""Shared helpers for the test-suite: golden-fixture loading and the tolerance rule."""

import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DTYPES = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16}

# Tolerances of the parity contract: max-abs 2e-2 on bf16/fp16 out and dQ/dK/dV, 1e-3 on fp32
# out and on logsumexp.
TOL_16BIT = 2e-2
TOL_FP32 = 1e-3
TOL_LSE = 1e-3


def golden_names():
    """The fixtures inside the reference's gate (equal lengths, no dropout)."""
    names = sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))
    return [n for n in names if not n.startswith("ext_")]


def ext_golden_names():
    """The fixtures beyond it: causal masks over unequal lengths, dropout."""
    names = sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "ext_*.npz")))
    return names


def load_ext_golden(name):
    """Returns (meta dict, q, k, v, dout as CPU tensors of the case dtype, expected fp32 dict).
    meta: B, Hq, Hkv, Sq, Sk, D, mode (B200FA_CAUSAL_*), dtype, scale, dropout (None or
    (p, seed, offset)), keep (bool array (B,Hq,Sq,Sk) or None)."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    b, hq, hkv, sq, sk, d, mode, code = (int(x) for x in z["meta"])
    dtype = DTYPES[code]
    meta = dict(B=b, Hq=hq, Hkv=hkv, Sq=sq, Sk=sk, D=d, mode=mode, dtype=dtype, scale=d ** -0.5, dropout=None, keep=None)
    if "drop" in z:
        p6, lo, hi, off = (int(x) for x in z["drop"])
        meta["dropout"] = (p6 / 1e6, lo | (hi << 32), off)
        meta["keep"] = np.unpackbits(z["keep_bits"])[: b * hq * sq * sk].reshape(b, hq, sq, sk).astype(bool)
    q, k, v, dout = (torch.from_numpy(z[n]).to(dtype) for n in ("q", "k", "v", "dout"))
    expected = {n: torch.from_numpy(z[n]) for n in ("out", "lse", "dq", "dk", "dv")}
    return meta, q, k, v, dout, expected


def load_golden(name):
    """Returns (meta dict, q, k, v, dout as CPU tensors of the case dtype, expected fp32 dict)."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    b, hq, hkv, s, d, causal, code = (int(x) for x in z["meta"])
    dtype = DTYPES[code]
    meta = dict(B=b, Hq=hq, Hkv=hkv, S=s, D=d, causal=bool(causal), dtype=dtype, scale=d ** -0.5)
    dout = torch.from_numpy(z["dout"]).to(dtype)
    if "fused" in z:
        fused = torch.from_numpy(z["fused"]).to(dtype)
        width = hq * d
        q, k, v = (p.view(b, s, hq, d).transpose(1, 2) for p in fused.split(width, dim=2))
        meta["fused"] = fused
    else:
        q, k, v = (torch.from_numpy(z[n]).to(dtype) for n in ("q", "k", "v"))
    expected = {n: torch.from_numpy(z[n]) for n in ("out", "lse", "dq", "dk", "dv")}
    return meta, q, k, v, dout, expected


def parity_report(name, got, ref, tol, dtype=None, ref_is_rounded=False):
    """Both bounds of the parity contract for one tensor, as numbers:
    ``max_abs`` - the strict max-abs error; ``over_flat`` - how many elements exceed the flat
    tolerance `tol`; ``over_widened`` - how many exceed `tol` + half a storage ulp of the
    reference value (the bound `assert_within` enforces; a whole ulp when the reference is itself
    a result rounded to the 16-bit storage type); ``n`` - elements compared."""
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    finite = torch.isfinite(ref)
    # entries that are -inf / +inf on both sides (logsumexp of a row that sees no key) agree exactly
    same_inf = (~finite) & (got == ref)
    err = torch.where(finite, (got - ref).abs(), torch.where(same_inf, torch.zeros_like(ref), torch.full_like(ref, float("inf"))))
    half_ulp = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}.get(dtype, 0.0)
    if ref_is_rounded:
        half_ulp *= 2
    bound = tol + half_ulp * torch.where(finite, ref.abs(), torch.zeros_like(ref))
    # elements over the flat tolerance where rounding the result to the storage type cannot
    # account for even half of it (half an ulp of the reference below tol / 2)
    rounding = half_ulp * torch.where(finite, ref.abs(), torch.zeros_like(ref))
    return {"name": name, "max_abs": err.max().item(), "over_flat": int((err > tol).sum()),
            "over_flat_unexplained": int(((err > tol) & (rounding < tol / 2)).sum()),
            "over_widened": int((err > bound).sum()), "n": err.numel(), "tol": tol,
            "max_ref": ref[finite].abs().max().item() if finite.any() else 0.0}


def assert_within(name, got, ref, tol, dtype=None):
    """max-abs `tol`, widened by half a bf16/fp16 ulp of the reference value where the reference
    is large enough that rounding the result to the storage type alone exceeds `tol` (half an
    ulp of bf16 is 2^-9 relative: 0.0156 at magnitude 4, 0.031 at 8)."""
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{name}: shape {tuple(got.shape)} != {tuple(ref.shape)}"
    assert not torch.isnan(got).any(), f"{name}: NaN in result"
    half_ulp = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}.get(dtype, 0.0)
    bound = tol + half_ulp * ref.abs()
    err = (got - ref).abs()
    worst = (err - bound).max().item()
    assert worst <= 0, (f"{name}: max-abs error {err.max().item():.3e} (tolerance {tol}, "
                        f"worst excess {worst:.3e} at |ref| up to {ref.abs().max().item():.2f})")
    return err.max().item()
