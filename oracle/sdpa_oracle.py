"""TEST INFRASTRUCTURE ONLY — the parity oracle and the timed CPU baseline.

The oracle is torch's CPU scaled-dot-product attention on float32 upcasts of the SAME
16-bit-rounded inputs the GPU sees, which is exactly what the reference's GPU tests compare its
kernels against (tests/test_eager_kernels.py:9495-9535); the logsumexp comes from the CPU flash
op (``aten::_scaled_dot_product_flash_attention_for_cpu``).  Parity status: see
``oracle/restatement.py`` — not pinned against the reference's own Mojo kernels (they cannot run
here), pinned against the reference tests' expectation and an independent float64 restatement.

This module also owns the seeded synthetic inputs for the five benchmark configurations and
the FLOP convention (forward ``4*B*H*Sq*Sk*D``, halved when causal; backward 2.5x forward —
benchmarks/test_attention.py:46,163).
"""

from __future__ import annotations

import dataclasses
import math
import os
import time

import torch


@dataclasses.dataclass(frozen=True)
class Config:
    name: str
    dtype: torch.dtype
    causal: bool
    B: int
    Hq: int
    Hkv: int
    S: int
    D: int
    scale: float
    backward: bool
    dist: str  # "normal", "half_normal" (0.5*N(0,1)) or "uniform" (U(-1,1))

    def fwd_flops(self) -> float:
        f = 4.0 * self.B * self.Hq * self.S * self.S * self.D
        return f / 2 if self.causal else f

    def bwd_flops(self) -> float:
        return 2.5 * self.fwd_flops()

    def fwd_bytes(self) -> float:
        es = torch.empty((), dtype=self.dtype).element_size()
        qo = 2 * self.B * self.Hq * self.S * self.D * es
        kv = 2 * self.B * self.Hkv * self.S * self.D * es
        return qo + kv + self.B * self.Hq * self.S * 4

    def bwd_bytes(self) -> float:
        es = torch.empty((), dtype=self.dtype).element_size()
        q_like = 4 * self.B * self.Hq * self.S * self.D * es  # q, out, dout read; dq written
        kv_like = 4 * self.B * self.Hkv * self.S * self.D * es  # k, v read; dk, dv written
        return q_like + kv_like + self.B * self.Hq * self.S * 4


CONFIGS = {
    "C1": Config("C1", torch.float32, True, 2, 4, 4, 256, 64, 1 / math.sqrt(64), False, "normal"),
    "C2": Config("C2", torch.bfloat16, True, 8, 12, 12, 1024, 64, 0.125, True, "normal"),
    "C3": Config("C3", torch.bfloat16, True, 4, 32, 8, 4096, 128, 1 / math.sqrt(128), True, "half_normal"),
    "C4": Config("C4", torch.bfloat16, True, 1, 32, 32, 32768, 128, 1 / math.sqrt(128), False, "normal"),
    "C5": Config("C5", torch.float16, False, 64, 16, 16, 2048, 128, 1 / math.sqrt(128), True, "uniform"),
}


def shard(cfg: Config, rank: int, world: int) -> Config:
    """The slice of `cfg` that rank `rank` of `world` owns.

    Units are (batch, kv-head group) pairs: the batch is split first, then KV heads (with the
    query heads that read them); a GQA group is never split.
    """
    if world == 1:
        return cfg
    if cfg.B % world == 0:
        return dataclasses.replace(cfg, B=cfg.B // world)
    if world % cfg.B == 0 and cfg.Hkv % (world // cfg.B) == 0:
        per = world // cfg.B
        return dataclasses.replace(cfg, B=1, Hq=cfg.Hq // per, Hkv=cfg.Hkv // per)
    raise ValueError(f"{cfg.name} does not split over {world} ranks")


def make_inputs(cfg: Config, seed: int = 0, B: int | None = None, Hq: int | None = None,
                Hkv: int | None = None, S: int | None = None):
    """q, k, v, dout as CPU tensors of cfg.dtype, drawn in that order from one seeded generator
    (the draw discipline of benchmarks/test_attention.py:36-47,126-128)."""
    B = cfg.B if B is None else B
    Hq = cfg.Hq if Hq is None else Hq
    Hkv = cfg.Hkv if Hkv is None else Hkv
    S = cfg.S if S is None else S
    g = torch.Generator().manual_seed(seed)

    def draw(shape):
        if cfg.dist == "uniform":
            return torch.rand(shape, generator=g, dtype=torch.float32) * 2 - 1
        x = torch.randn(shape, generator=g, dtype=torch.float32)
        return x * 0.5 if cfg.dist == "half_normal" else x

    q = draw((B, Hq, S, cfg.D)).to(cfg.dtype)
    k = draw((B, Hkv, S, cfg.D)).to(cfg.dtype)
    v = draw((B, Hkv, S, cfg.D)).to(cfg.dtype)
    dout = torch.randn((B, Hq, S, cfg.D), generator=g, dtype=torch.float32).to(cfg.dtype)
    return q, k, v, dout


def _bottom_right_mask(sq: int, sk: int) -> torch.Tensor:
    """Boolean (sq, sk) mask of the bottom-right aligned causal rule ``j <= i + (sk - sq)``
    (torch_mojo_backend/eager_flash_attention/fa4_fwd_kernel.mojo:266-273)."""
    return torch.arange(sk)[None, :] <= torch.arange(sq)[:, None] + (sk - sq)


def sdpa_forward(q, k, v, causal, scale: float):
    """(out fp32, lse fp32) from torch's CPU flash op on fp32 upcasts.  ``causal``: False/0,
    True/1 (torch's is_causal: top-left aligned) or 2 (bottom-right aligned, given to torch as
    an explicit boolean mask; needs every query row to see at least one key, i.e. Sk >= Sq)."""
    q32, k32, v32 = (t.detach().float().contiguous() for t in (q, k, v))
    if int(causal) == 2:
        # the CPU flash op takes an additive mask of the query dtype
        mask = torch.zeros(q.shape[2], k.shape[2]).masked_fill(~_bottom_right_mask(q.shape[2], k.shape[2]), float("-inf"))
        out, lse = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(
            q32, k32, v32, 0.0, False, attn_mask=mask, scale=scale
        )
        return out, lse
    out, lse = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(
        q32, k32, v32, 0.0, bool(causal), scale=scale
    )
    return out, lse


def sdpa_backward(q, k, v, dout, causal, scale: float):
    """(out, dq, dk, dv) in fp32 via autograd through CPU SDPA on fp32 upcasts (``causal`` as in
    sdpa_forward)."""
    q32, k32, v32 = (t.detach().float().contiguous().requires_grad_() for t in (q, k, v))
    gqa = q.shape[1] != k.shape[1]
    if int(causal) == 2:
        out = torch.nn.functional.scaled_dot_product_attention(
            q32, k32, v32, attn_mask=_bottom_right_mask(q.shape[2], k.shape[2]), dropout_p=0.0, scale=scale,
            enable_gqa=gqa)
    else:
        out = torch.nn.functional.scaled_dot_product_attention(
            q32, k32, v32, dropout_p=0.0, is_causal=bool(causal), scale=scale, enable_gqa=gqa)
    out.backward(dout.detach().float())
    return out.detach(), q32.grad, k32.grad, v32.grad


def sdpa_dropout(q, k, v, dout, causal, scale: float, keep: torch.Tensor, keep_scale: float):
    """(out, lse, dq, dk, dv) in fp32 for attention with a GIVEN dropout mask, from plain torch CPU
    ops and autograd: softmax of the masked scaled scores, entries multiplied by
    ``keep * keep_scale`` before they meet V.  ``keep``: bool (B, Hq, Sq, Sk).  torch's own SDPA
    cannot be handed a mask of ours, so this is the torch-side oracle for the dropout path; the
    float64 restatement (oracle/restatement.py) is checked against it."""
    q32, k32, v32 = (t.detach().float().contiguous().requires_grad_() for t in (q, k, v))
    group = q.shape[1] // k.shape[1]
    kk = k32.repeat_interleave(group, dim=1) if group > 1 else k32
    vv = v32.repeat_interleave(group, dim=1) if group > 1 else v32
    s = torch.matmul(q32, kk.transpose(-1, -2)) * scale
    sq, sk = s.shape[-2:]
    mode = int(causal)
    if mode:
        off = 0 if mode == 1 else sk - sq
        s = s.masked_fill(~(torch.arange(sk)[None, :] <= torch.arange(sq)[:, None] + off), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1)
    out = torch.matmul(p * (keep.float() * keep_scale), vv)
    out.backward(dout.detach().float())
    return out.detach(), lse.detach(), q32.grad, k32.grad, v32.grad


def time_cpu(cfg: Config, *, backward: bool, sample_heads: int = 0, reps: int = 1, threads: int | None = None,
             sample_flops: float = 2.0e12, target_seconds: float = 0.0):
    """Time the CPU path on a bounded slice of `cfg` in its real dtype.

    The slice is whole (batch entry, KV-head group) units: `sample_heads` KV-head groups of one
    batch entry when given, otherwise as many units as bring one repetition to about
    `sample_flops` (KV-head groups of one batch entry first, then further batch entries).  It is
    repeated `reps` times, and beyond that until `target_seconds` of CPU work have been spent
    (at most 20 repetitions); the best repetition counts.

    Returns (TFLOP/s, seconds of the best repetition, threads used, description of the sample).
    """
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    group = cfg.Hq // cfg.Hkv
    unit = 4.0 * group * cfg.S * cfg.S * cfg.D * (0.5 if cfg.causal else 1.0) * (3.5 if backward else 1.0)
    if sample_heads > 0:
        hkv, batch = max(1, min(sample_heads, cfg.Hkv)), 1
    else:
        units = max(1, int(round(sample_flops / unit)))
        hkv = min(cfg.Hkv, units)
        batch = max(1, min(cfg.B, units // hkv))
    q, k, v, dout = make_inputs(cfg, B=batch, Hq=hkv * group, Hkv=hkv)
    flops = unit * hkv * batch   # forward, plus 2.5x forward for the backward: the way a training step runs it
    best, spent, done = float("inf"), 0.0, 0
    while done < max(1, reps) or (spent < target_seconds and done < 20):
        t0 = time.perf_counter()
        if backward:
            qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
            o = torch.nn.functional.scaled_dot_product_attention(
                qq, kk, vv, dropout_p=0.0, is_causal=cfg.causal, scale=cfg.scale, enable_gqa=group > 1
            )
            o.backward(dout)
        else:
            torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(q, k, v, 0.0, cfg.causal, scale=cfg.scale)
        dt = time.perf_counter() - t0
        best, spent, done = min(best, dt), spent + dt, done + 1
    sample = (f"B={batch}, Hq={hkv * group}, Hkv={hkv}, S={cfg.S}, D={cfg.D}, {'fwd+bwd' if backward else 'fwd'}, "
              f"best of {done} ({spent:.1f} s of CPU work)")
    return flops / best / 1e12, best, threads, sample
