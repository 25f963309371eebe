"""TEST INFRASTRUCTURE ONLY — numpy float64 restatement of the reference's attention math.

Parity status: the reference's Mojo kernels cannot be built or run in this environment
(they need the ``mojo``/``max`` toolchain), and the reference ships no golden vectors, so this
restatement is NOT pinned against outputs of the reference's own kernels ("parity unpinned"
in that sense).  It is pinned against the expectation the reference's own GPU tests use —
torch's CPU fp32 SDPA on seeded inputs (tests/test_eager_kernels.py:9495-9535) and an explicit
masked ``logsumexp`` (tests/test_eager_kernels.py:9556-9571) — by ``tests/test_oracle.py`` and
the committed fixtures in ``tests/golden``.

Each function follows the arithmetic of the reference kernel it cites, written tile-free in
float64 so it is an independent check of torch's CPU SDPA rather than a copy of it.
"""

from __future__ import annotations

import numpy as np

LOG2E = 1.4426950408889634


def expand_kv_heads(x: np.ndarray, heads_q: int) -> np.ndarray:
    """Query head h reads key/value head h // (Hq // Hkv).

    Follows the head map of torch_mojo_backend/eager_flash_attention/fa4_fwd_kernel.mojo:396-398,428
    and torch_mojo_backend/aten_functions.py:621-637 (``repeat_interleave`` along the head axis).
    """
    group = heads_q // x.shape[1]
    return np.repeat(x, group, axis=1)


def causal_offset(causal, sq: int, sk: int) -> int | None:
    """None when unmasked, else the diagonal offset: query row i sees key column j iff
    ``j <= i + offset``.  ``causal`` is False/0, True/1 (top-left aligned: offset 0, what torch's CPU
    SDPA does for is_causal) or 2 (bottom-right aligned: offset ``sk - sq``, the rule of
    torch_mojo_backend/eager_flash_attention/fa4_fwd_kernel.mojo:266-273, "row i attends col j iff
    j <= i + (slk - slq)").  The two coincide when sq == sk."""
    mode = int(causal)
    if mode == 0:
        return None
    return 0 if mode == 1 else sk - sq


def visible(causal, sq: int, sk: int) -> np.ndarray:
    """Boolean (sq, sk) matrix of the key columns each query row may attend to."""
    off = causal_offset(causal, sq, sk)
    if off is None:
        return np.ones((sq, sk), dtype=bool)
    return np.arange(sk)[None, :] <= np.arange(sq)[:, None] + off


def scores(q: np.ndarray, k: np.ndarray, causal) -> np.ndarray:
    """S = Q K^T with the masked entries set to -inf.

    Follows torch_mojo_backend/eager_flash_attention/fa4_fwd_kernel.mojo:530-543 (the kernel uses
    -1e30 for -inf; both give exp2(...) == 0 in float64 and float32 alike).
    """
    s = np.einsum("bhqd,bhkd->bhqk", q, k)
    sq, sk = s.shape[-2:]
    return np.where(visible(causal, sq, sk), s, -np.inf)


def forward(q, k, v, causal, scale: float, keep=None, keep_scale: float = 1.0):
    """(out, lse) as the forward kernel defines them.

    Follows torch_mojo_backend/eager_flash_attention/fa4_fwd_kernel.mojo:650-861 (row max, exp2 of
    ``s*c - m*c`` with ``c = scale*log2(e)``, row sum), :1014-1022 (O / rowsum) and :1138-1160
    (``LSE = rowmax*c*ln2 + ln(rowsum)``).  A query row that sees no key gets out = 0 and
    lse = -inf.  ``keep`` (bool, (B,Hq,Sq,Sk)) is a dropout mask: the row sum and lse keep every
    probability, only the entries that multiply V are dropped and the kept ones scaled.
    """
    q = np.asarray(q, dtype=np.float64)
    k = expand_kv_heads(np.asarray(k, dtype=np.float64), q.shape[1])
    v = expand_kv_heads(np.asarray(v, dtype=np.float64), q.shape[1])
    c = scale * LOG2E
    s = scores(q, k, causal)
    m = s.max(axis=-1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    p = np.exp2(s * c - m * c)
    l = p.sum(axis=-1, keepdims=True)
    pv = p if keep is None else p * keep * keep_scale
    with np.errstate(divide="ignore", invalid="ignore"):
        out = np.where(l > 0, np.einsum("bhqk,bhkd->bhqd", pv, v) / l, 0.0)
        lse = np.where(l > 0, (m * c) * np.log(2.0) + np.log(l), -np.inf)
    return out, lse[..., 0]


def backward(q, k, v, dout, causal, scale: float, keep=None, keep_scale: float = 1.0):
    """(dq, dk, dv) as the backward kernels define them.

    Follows torch_mojo_backend/eager_flash_attention/fa4_bwd_kernel.mojo:1-44 and :810-980:
    ``dpsum = rowsum(dO*O)`` (preprocess, :1634-1662), ``P = exp2(S*c - lse*log2e)``,
    ``dV = P^T dO``, ``dP = dO V^T``, ``dS = P*(dP - dpsum)``, ``dK = scale * dS^T Q``
    (:1443-1444), ``dQ = scale * dS K`` (:1855).  Gradients of shared key/value heads are summed
    over the query heads of the group.  With a dropout mask ``keep``: ``dV = (P*D)^T dO`` and
    ``dS = P*(D*dP - dpsum)`` with ``D = keep * keep_scale`` (``dpsum`` uses the dropped-out O).
    """
    q = np.asarray(q, dtype=np.float64)
    heads_q = q.shape[1]
    heads_kv = np.asarray(k).shape[1]
    k64 = expand_kv_heads(np.asarray(k, dtype=np.float64), heads_q)
    v64 = expand_kv_heads(np.asarray(v, dtype=np.float64), heads_q)
    dout = np.asarray(dout, dtype=np.float64)
    out, lse = forward(q, k, v, causal, scale, keep, keep_scale)
    c = scale * LOG2E
    s = scores(q, k64, causal)
    lse2 = np.where(np.isfinite(lse), lse * LOG2E, np.inf)     # rows that saw no key: P = 0
    p = np.exp2(s * c - lse2[..., None])
    dmul = 1.0 if keep is None else keep * keep_scale
    dpsum = (dout * out).sum(axis=-1, keepdims=True)
    dv = np.einsum("bhqk,bhqd->bhkd", p * dmul, dout)
    dp = np.einsum("bhqd,bhkd->bhqk", dout, v64) * dmul
    ds = p * (dp - dpsum)
    dk = scale * np.einsum("bhqk,bhqd->bhkd", ds, q)
    dq = scale * np.einsum("bhqk,bhkd->bhqd", ds, k64)
    group = heads_q // heads_kv
    if group > 1:
        b, _, sk, d = dk.shape
        dk = dk.reshape(b, heads_kv, group, sk, d).sum(axis=2)
        dv = dv.reshape(b, heads_kv, group, sk, d).sum(axis=2)
    return dq, dk, dv
