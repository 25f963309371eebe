"""Times the split-KV forward (few query rows per KV head over a long key sequence) on one GPU.

    python -m torch_mojo_backend_b200.decode_bench                      # the default list of shapes
    python -m torch_mojo_backend_b200.decode_bench --shape 8,32,8,1,32768,128 --reps 3

One JSON line per shape: the time of one call of ``b200fa_fwd_splitkv``,
CUDA events on the launching stream after three warm-up calls, K and V larger than L2 or an L2 flush
between calls when they are not; ``gbs`` counts the bytes of K and V once, which is what the call
has to read; ``frac`` divides by the measured copy bandwidth when a MEASURED_PEAKS.json lies beside
the package's parent folder, else by 6650 GB/s.  ``prefill_ms`` is the tensor-core prefill kernel
on the same problem.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from . import _lib, raw

DEFAULT_SHAPES = [
    (8, 32, 8, 1, 32768, 128),
    (64, 32, 8, 1, 8192, 128),
    (1, 32, 8, 1, 131072, 128),
    (16, 32, 8, 4, 16384, 128),
    (32, 12, 12, 1, 4096, 64),
    (1, 8, 8, 1, 4096, 128),
]
L2_BYTES = 126 << 20


def hbm_peak() -> tuple[float, str]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def time_calls(fn, reps: int, flush) -> float:
    """Mean milliseconds per call.  Inputs larger than L2: the calls run back to back between two
    events; otherwise L2 is flushed before each call and every call is timed by itself."""
    for _ in range(3):
        fn()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if flush is None:
        torch.cuda.synchronize()
        start.record()
        for _ in range(reps):
            fn()
        stop.record()
        stop.synchronize()
        return start.elapsed_time(stop) / reps
    total = 0.0
    for _ in range(reps):
        flush.zero_()
        start.record()
        fn()
        stop.record()
        stop.synchronize()
        total += start.elapsed_time(stop)
    return total / reps


def run_shape(shape, reps: int, dtype: torch.dtype, causal: int, peak: float, peak_kind: str) -> dict:
    B, Hq, Hkv, Sq, Sk, D = shape
    g = torch.Generator(device="cuda").manual_seed(0)
    q = (torch.randn(B, Hq, Sq, D, device="cuda", generator=g) * 0.5).to(dtype)
    k = (torch.randn(B, Hkv, Sk, D, device="cuda", generator=g) * 0.5).to(dtype)
    v = (torch.randn(B, Hkv, Sk, D, device="cuda", generator=g) * 0.5).to(dtype)
    out = torch.empty_like(q)
    lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device="cuda")
    nbytes = _lib.fwd_splitkv_workspace_bytes(B, Hq, Hkv, Sq, Sk, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    kv_bytes = 2 * B * Hkv * Sk * D * q.element_size()
    flush = None if kv_bytes > 2 * L2_BYTES else torch.empty(2 * L2_BYTES, dtype=torch.uint8, device="cuda")
    ms = time_calls(lambda: raw.flash_fwd_splitkv(q, k, v, causal=causal, out=out, lse=lse, workspace=ws), reps, flush)
    ms_prefill = time_calls(lambda: raw.flash_fwd(q, k, v, causal=causal, out=out, lse=lse), reps, flush)
    gbs = kv_bytes / ms / 1e6
    return {"shape": {"B": B, "Hq": Hq, "Hkv": Hkv, "Sq": Sq, "Sk": Sk, "D": D}, "dtype": str(dtype).split(".")[1],
            "ms": round(ms, 4), "gbs": round(gbs, 1), "peak_gbs": peak, "peak": peak_kind, "frac": round(gbs / peak, 3),
            "prefill_ms": round(ms_prefill, 4), "l2": "inputs larger than L2" if flush is None else "flushed"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", action="append", help="B,Hq,Hkv,Sq,Sk,D (repeatable)")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--mask", type=int, default=2, help="0 none, 1 upper-left causal, 2 lower-right causal")
    args = ap.parse_args()
    shapes = [tuple(int(x) for x in s.split(",")) for s in args.shape] if args.shape else DEFAULT_SHAPES
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    peak, kind = hbm_peak()
    for shape in shapes:
        print(json.dumps(run_shape(shape, args.reps, dtype, args.mask, peak, kind)), flush=True)


if __name__ == "__main__":
    main()
