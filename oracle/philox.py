"""TEST INFRASTRUCTURE ONLY — numpy restatement of the dropout mask of the attention kernels.

Philox4x32-10 as published (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as
1, 2, 3", SC'11; the generator behind the Philox (seed, offset) pair that
``aten::_scaled_dot_product_flash_attention`` returns — reference slots:
torch_mojo_backend/eager_kernels/aten_fast.py:7726-7734, host-side reservation:
torch_mojo_backend/mojo_device/torch_mojo_device_module.py:84-99).  The reference has no kernel
that consumes the pair, so the layout of the stream below is this library's own
(``include/b200fa.h``, b200fa_fwd_dropout) and parity for dropout is pinned against this
restatement plus the generator's published known-answer vectors (tests/test_oracle.py).

Stream layout: one call per run of 16 key columns of one query row; key = seed; counter =
(column // 16, row, low word of offset + b*Hq + h, high word of it); byte ``4*w + r`` of the call
(word w, byte r from the low end) belongs to column ``16*(column//16) + 4*w + r``; an element is
kept when its byte >= threshold = round(256 p) (at most 255).
"""

from __future__ import annotations

import numpy as np

M0 = np.uint64(0xD2511F53)
M1 = np.uint64(0xCD9E8D57)
W0 = 0x9E3779B9
W1 = 0xBB67AE85
MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(counter: np.ndarray, key: tuple[int, int]) -> np.ndarray:
    """counter: (..., 4) uint32; key: (k0, k1).  Returns (..., 4) uint32."""
    c = [counter[..., i].astype(np.uint64) for i in range(4)]
    k0, k1 = int(key[0]) & 0xFFFFFFFF, int(key[1]) & 0xFFFFFFFF
    for _ in range(10):
        p0 = M0 * c[0]
        p1 = M1 * c[2]
        n0 = ((p1 >> np.uint64(32)) ^ c[1] ^ np.uint64(k0)) & MASK32
        n1 = p1 & MASK32
        n2 = ((p0 >> np.uint64(32)) ^ c[3] ^ np.uint64(k1)) & MASK32
        n3 = p0 & MASK32
        c = [n0, n1, n2, n3]
        k0 = (k0 + W0) & 0xFFFFFFFF
        k1 = (k1 + W1) & 0xFFFFFFFF
    return np.stack(c, axis=-1).astype(np.uint32)


def dropout_threshold(p: float) -> int:
    if not p > 0:
        return 0
    return min(255, int(np.floor(np.float32(p) * np.float32(256.0) + np.float32(0.5))))


def keep_mask(B: int, Hq: int, Sq: int, Sk: int, p: float, seed: int, offset: int) -> tuple[np.ndarray, float]:
    """(mask bool (B, Hq, Sq, Sk), scale of the kept entries = 256 / (256 - threshold))."""
    thr = dropout_threshold(p)
    if thr == 0:
        return np.ones((B, Hq, Sq, Sk), dtype=bool), 1.0
    nblk = (Sk + 15) // 16
    out = np.empty((B, Hq, Sq, nblk * 16), dtype=np.uint8)
    key = (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    blk = np.arange(nblk, dtype=np.uint32)[None, :]
    row = np.arange(Sq, dtype=np.uint32)[:, None]
    for b in range(B):
        for h in range(Hq):
            hi = (offset + b * Hq + h) & 0xFFFFFFFFFFFFFFFF
            ctr = np.empty((Sq, nblk, 4), dtype=np.uint32)
            ctr[..., 0] = blk
            ctr[..., 1] = row
            ctr[..., 2] = hi & 0xFFFFFFFF
            ctr[..., 3] = hi >> 32
            words = philox4x32_10(ctr, key)                     # (Sq, nblk, 4)
            # little-endian bytes of the four words, in order, are the 16 columns of the block
            out[b, h] = words.astype("<u4").view(np.uint8).reshape(Sq, nblk * 16)
    return out[..., :Sk] >= thr, 256.0 / (256 - thr)
