"""Calls into the C ABI for plain ``torch.cuda`` tensors.

The `mojo` device layer (``flash_ops.py``) sits beside this; tests and the benchmark also use
it directly, the way the reference's GPU tests call the bridge with hand-built buffers
(tests/test_eager_kernels.py:9754-9765).  Nothing here computes attention: every function
validates metadata, allocates outputs with torch's CUDA allocator and enqueues library
kernels on torch's current stream.
"""

from __future__ import annotations

import math

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise NotImplementedError(f"b200fa supports float32, bfloat16 and float16, got {dtype}") from None


def t4(t: torch.Tensor) -> _lib.Tensor4:
    return _lib.Tensor4.make(t.data_ptr(), tuple(t.shape), tuple(t.stride()))


def _stream_and_device(t: torch.Tensor) -> tuple[int, int]:
    dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
    return torch.cuda.current_stream(dev).cuda_stream, dev


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)


def flash_fwd(q, k, v, *, causal, scale: float | None = None, out=None, lse=None, status=None,
              simt: bool = False, dropout=None):
    """out, lse = attention forward on CUDA tensors shaped (B, H, S, D).

    ``out`` defaults to a new contiguous (B, Hq, Sq, D) tensor; pass a pre-allocated (possibly
    strided) tensor to choose the storage layout.  ``lse`` is fp32 (B, Hq, Sq).  ``causal`` is a
    bool (True: diagonal from the top-left corner) or one of ``_lib.CAUSAL_*``; ``dropout`` is
    None or ``(p, philox_seed, philox_offset)``.
    """
    if q.device.type != "cuda":
        raise RuntimeError("b200fa kernels need CUDA memory; there is no CPU implementation")
    B, Hq, Sq, D = q.shape
    if scale is None:
        scale = default_scale(D)
    if out is None:
        out = torch.empty((B, Hq, Sq, D), dtype=q.dtype, device=q.device)
    if lse is None:
        lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    stream, dev = _stream_and_device(q)
    rc = _lib.fwd(t4(q), t4(k), t4(v), t4(out), lse.data_ptr(), dtype_code(q.dtype), causal, float(scale),
                  stream, dev, status.data_ptr() if status is not None else 0, simt=simt, dropout=dropout)
    if rc != _lib.OK:
        raise _lib.B200FAError(rc, "b200fa_fwd")
    return out, lse


def flash_fwd_splitkv(q, k, v, *, causal, scale: float | None = None, out=None, lse=None, workspace=None):
    """out, lse = the split-KV (decode) forward on CUDA tensors shaped (B, H, S, D); needs
    ``(Hq / Hkv) * Sq <= 16``."""
    if q.device.type != "cuda":
        raise RuntimeError("b200fa kernels need CUDA memory; there is no CPU implementation")
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    if scale is None:
        scale = default_scale(D)
    if out is None:
        out = torch.empty((B, Hq, Sq, D), dtype=q.dtype, device=q.device)
    if lse is None:
        lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    need = _lib.fwd_splitkv_workspace_bytes(B, Hq, Hkv, Sq, Sk, D)
    if workspace is None:
        workspace = torch.empty((need,), dtype=torch.uint8, device=q.device)
    stream, dev = _stream_and_device(q)
    rc = _lib.fwd_splitkv(t4(q), t4(k), t4(v), t4(out), lse.data_ptr(), workspace.data_ptr(),
                          workspace.numel() * workspace.element_size(), dtype_code(q.dtype), causal, float(scale),
                          stream, dev)
    if rc != _lib.OK:
        raise _lib.B200FAError(rc, "b200fa_fwd_splitkv")
    return out, lse


def flash_bwd(dout, q, k, v, out, lse, *, causal, scale: float | None = None, dq=None, dk=None,
              dv=None, workspace=None, status=None, simt: bool = False, parts: int = 7, dropout=None):
    """dq, dk, dv = attention backward on CUDA tensors shaped (B, H, S, D)."""
    if q.device.type != "cuda":
        raise RuntimeError("b200fa kernels need CUDA memory; there is no CPU implementation")
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    if scale is None:
        scale = default_scale(D)
    if dq is None:
        dq = torch.empty((B, Hq, S, D), dtype=q.dtype, device=q.device)
    if dk is None:
        dk = torch.empty(tuple(k.shape), dtype=q.dtype, device=q.device)
    if dv is None:
        dv = torch.empty(tuple(v.shape), dtype=q.dtype, device=q.device)
    code = dtype_code(q.dtype)
    need = _lib.bwd_workspace_bytes(B, Hq, Hkv, S, D, code)
    if workspace is None:
        workspace = torch.empty((need,), dtype=torch.uint8, device=q.device)
    stream, dev = _stream_and_device(q)
    rc = _lib.bwd(t4(q), t4(k), t4(v), t4(out), t4(dout), lse.data_ptr(), t4(dq), t4(dk), t4(dv),
                  workspace.data_ptr(), workspace.numel() * workspace.element_size(), code, causal, float(scale),
                  stream, dev, status.data_ptr() if status is not None else 0, simt=simt, parts=parts,
                  dropout=dropout)
    if rc != _lib.OK:
        raise _lib.B200FAError(rc, "b200fa_bwd")
    return dq, dk, dv
