"""Host side of the two flash-attention aten ops on the `mojo` device.

Thin Python over the C ABI: eligibility gate, layout routing, output/scratch allocation and
the aten return contracts.  It mirrors, function by function, the FA4 section of the
reference's eager layer (torch_mojo_backend/eager_kernels/aten_fast.py:6971-7408 and
7699-7839); every device computation happens inside ``libb200fa.so``.  There is no fallback:
an ineligible call raises ``NotImplementedError``.
"""

from __future__ import annotations

import math

import torch

from . import _lib
from .tensor import TorchMojoTensor, payload

_DTYPE_CODES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}

#: per-op call counters, the analogue of the reference's EAGER_CALL_COUNTERS
#: (torch_mojo_backend/mojo_device/mojo_device_aten_ops.py:84-109)
CALL_COUNTERS = {
    "aten::_scaled_dot_product_flash_attention": 0,
    "aten::_scaled_dot_product_flash_attention_backward": 0,
}


def _stream_for(index: int) -> int:
    """The CUDA stream (as an integer handle) every mojo op on device `index` is ordered on."""
    return torch.cuda.current_stream(index).cuda_stream


# --------------------------------------------------------------------------- eligibility
def flash_inputs(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None,
                 enable_gqa=False):
    """Return ``(q, k, v)`` payload tensors if the call is served by the kernels, else None.

    Metadata only — no device work.  Wider than the reference's gate
    (aten_fast.py:6971-7043, which needs causal, 16-bit, equal head counts and sm_90a):
    fp32/bf16/fp16, causal or not, ``Hq % Hkv == 0`` (needs ``enable_gqa`` when they differ),
    ``Sq == Sk`` when causal (a causal mask over ``Sq != Sk`` has a top-left and a bottom-right
    convention - torch's CPU SDPA and the reference's kernels disagree - so neither is offered;
    without a mask any ``Sq``, ``Sk`` pair is served), head_dim 64 or 128, no mask, no dropout,
    finite positive scale.
    """
    q, k, v = payload(query), payload(key), payload(value)
    if q is None or k is None or v is None or attn_mask is not None:
        return None
    if not isinstance(dropout_p, (int, float)) or isinstance(dropout_p, bool) or float(dropout_p) != 0.0:
        return None
    if not isinstance(is_causal, bool):
        return None
    if q._device_index != k._device_index or q._device_index != v._device_index:
        return None
    if q._dtype not in _DTYPE_CODES or k._dtype != q._dtype or v._dtype != q._dtype:
        return None
    if len(q._shape) != 4 or len(k._shape) != 4 or tuple(k._shape) != tuple(v._shape):
        return None
    batch, heads_q, seq_q, head_dim = q._shape
    kb, heads_kv, seq_k, kd = k._shape
    if kb != batch or kd != head_dim or (is_causal and seq_q != seq_k):
        return None
    if batch <= 0 or heads_q <= 0 or heads_kv <= 0 or seq_q <= 0 or seq_k <= 0 or head_dim not in (64, 128):
        return None
    if heads_q % heads_kv != 0 or (heads_q != heads_kv and not enable_gqa):
        return None
    if scale is not None:
        if not isinstance(scale, (int, float)) or isinstance(scale, bool):
            return None
        if not math.isfinite(float(scale)) or float(scale) <= 0.0:
            return None
    return q, k, v


# --------------------------------------------------------------------------- layout routing
def kernel_ready_layout(t: TorchMojoTensor) -> bool:
    """True when the kernels can read `t` (logical BHSD) in place: unit head_dim stride,
    every other stride a non-negative multiple of 16 bytes, 16-byte aligned base.  Covers the
    reference's two zero-copy routes — contiguous BHSD (aten_fast.py:7085-7103) and the
    gapped BTHD view of a fused-QKV projection (aten_fast.py:7046-7082) — and any other
    strided view with those properties."""
    if t._strides[3] != 1 or t._ptr % 16 != 0:
        return False
    for dim in range(3):
        stride = t._strides[dim]
        if stride < 0 or (stride * t._itemsize) % 16 != 0:
            return False
        if t._shape[dim] > 1 and stride == 0:
            return False
    return t._shape[2] <= 1 or t._strides[2] >= t._shape[3]


def bthd_stored(t: TorchMojoTensor) -> bool:
    """True when logical (B,H,S,D) `t` is stored sequence-major (B,S,H,D), i.e. it is a
    ``transpose(1, 2)`` view — nanoGPT's layout (aten_fast.py:7106-7113)."""
    _, heads, seq, _ = t._shape
    return heads > 1 and seq > 1 and t._strides[3] == 1 and t._strides[1] < t._strides[2]


def prepare(t: TorchMojoTensor) -> TorchMojoTensor:
    """`t` itself if the kernels can read it in place, else a dense BHSD copy (the
    reference's dense-copy route, aten_fast.py:7266-7281)."""
    return t if kernel_ready_layout(t) else t._materialize_contiguous()


def _alloc_like_layout(shape, dtype, index, sequence_major: bool) -> TorchMojoTensor:
    """A (B,H,S,D) tensor, stored BHSD or — to match a BTHD-stored input — as (B,S,H,D)
    memory viewed through ``transpose(1, 2)`` (aten_fast.py:7282-7285)."""
    if not sequence_major:
        return TorchMojoTensor._alloc(shape, dtype, index)
    b, h, s, d = shape
    return TorchMojoTensor._alloc_strided(shape, (s * h * d, d, h * d, 1), dtype, index)


def _t4(t: TorchMojoTensor) -> _lib.Tensor4:
    return _lib.Tensor4.make(t._ptr, t._shape, t._strides)


def _check(rc: int, where: str) -> None:
    if rc == _lib.OK:
        return
    if rc in (_lib.ERR_UNSUPPORTED, _lib.ERR_BAD_DTYPE):
        raise NotImplementedError(f"{where}: {_lib.strerror(rc)}")
    raise _lib.B200FAError(rc, where)


# --------------------------------------------------------------------------- forward
def flash_forward(q: TorchMojoTensor, k: TorchMojoTensor, v: TorchMojoTensor, is_causal: bool,
                  scale: float | None):
    """Allocate ``out`` (same dtype as q) and ``lse`` (fp32, (B,Hq,Sq)), enqueue the forward
    kernel, return ``(out, lse, q_used, k_used, v_used)`` like
    ``fast_fa4_16bit_d64_causal_forward`` (aten_fast.py:7151-7285)."""
    batch, heads_q, seq, head_dim = q._shape
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    q_used, k_used, v_used = prepare(q), prepare(k), prepare(v)
    out = _alloc_like_layout(q._shape, q._dtype, q._device_index, bthd_stored(q_used))
    lse = TorchMojoTensor._alloc((batch, heads_q, seq), torch.float32, q._device_index)
    rc = _lib.fwd(_t4(q_used), _t4(k_used), _t4(v_used), _t4(out), lse._ptr, _DTYPE_CODES[q._dtype],
                  bool(is_causal), float(scale), _stream_for(q._device_index), q._device_index, 0)
    _check(rc, "b200fa_fwd")
    return out, lse, q_used, k_used, v_used


def scaled_dot_product_flash_attention(query, key, value, dropout_p=0.0, is_causal=False,
                                       return_debug_mask=False, *, scale=None):
    """``aten::_scaled_dot_product_flash_attention`` on the mojo device.

    Returns the CUDA-shaped 9-tuple ``(out, logsumexp, cum_seq_q=None, cum_seq_k=None, max_q,
    max_k, rng_state uint64[2], unused uint64[], debug_attn_mask empty(0))`` exactly as the
    reference does (aten_fast.py:7699-7734).  Dropout is always 0, so the Philox slots are
    shape/dtype placeholders.
    """
    if dropout_p != 0.0 or return_debug_mask:
        raise NotImplementedError(
            "aten::_scaled_dot_product_flash_attention on mojo: dropout and return_debug_mask are not supported"
        )
    inputs = flash_inputs(query, key, value, None, dropout_p, is_causal, scale, enable_gqa=True)
    if inputs is None:
        raise NotImplementedError(
            "aten::_scaled_dot_product_flash_attention on mojo needs fp32/bf16/fp16 (B,H,S,D) tensors with "
            "head_dim 64 or 128, Sq == Sk when causal, Hq % Hkv == 0 and a positive finite scale"
        )
    q, k, v = inputs
    CALL_COUNTERS["aten::_scaled_dot_product_flash_attention"] += 1
    out, lse, _, _, _ = flash_forward(q, k, v, is_causal, scale)
    index = q._device_index
    rng_state = TorchMojoTensor._alloc((2,), torch.uint64, index)
    unused = TorchMojoTensor._alloc((), torch.uint64, index)
    debug_attn_mask = TorchMojoTensor._alloc((0,), q._dtype, index)
    return (out, lse, None, None, q._shape[2], k._shape[2], rng_state, unused, debug_attn_mask)


# --------------------------------------------------------------------------- backward
def flash_backward(dout, q, k, v, out, lse, is_causal: bool, scale: float):
    """Allocate dq/dk/dv and the scratch, enqueue the backward kernels, return the grads
    (``fast_fa4_16bit_d64_causal_backward``, aten_fast.py:7288-7408).  Gradients are stored in
    the layout of the tensor they belong to (BTHD-stored for BTHD-stored q/k/v)."""
    batch, heads_q, seq, head_dim = q._shape
    heads_kv = k._shape[1]
    index = q._device_index
    q_used, k_used, v_used = prepare(q), prepare(k), prepare(v)
    out_used, dout_used = prepare(out), prepare(dout)
    lse_used = lse._contig()
    dq = _alloc_like_layout(q._shape, q._dtype, index, bthd_stored(q_used))
    dk = _alloc_like_layout(k._shape, q._dtype, index, bthd_stored(k_used))
    dv = _alloc_like_layout(v._shape, q._dtype, index, bthd_stored(v_used))
    code = _DTYPE_CODES[q._dtype]
    nbytes = _lib.bwd_workspace_bytes(batch, heads_q, heads_kv, seq, head_dim, code)
    workspace = TorchMojoTensor._alloc((nbytes,), torch.uint8, index)
    rc = _lib.bwd(_t4(q_used), _t4(k_used), _t4(v_used), _t4(out_used), _t4(dout_used), lse_used._ptr,
                  _t4(dq), _t4(dk), _t4(dv), workspace._ptr, nbytes, code, bool(is_causal), float(scale),
                  _stream_for(index), index, 0)
    _check(rc, "b200fa_bwd")
    # `workspace` drops here: the allocator re-uses it only for work queued later on this stream
    return dq, dk, dv


def scaled_dot_product_flash_attention_backward(grad_out, query, key, value, out, logsumexp, cum_seq_q,
                                                cum_seq_k, max_q, max_k, dropout_p, is_causal, philox_seed,
                                                philox_offset, *, scale=None):
    """``aten::_scaled_dot_product_flash_attention_backward`` on the mojo device
    (aten_fast.py:7737-7839): validates the 14 positional arguments, then one bridge call."""
    if dropout_p != 0.0 or cum_seq_q is not None or cum_seq_k is not None:
        raise NotImplementedError("mojo flash attention backward: dropout / varlen are not supported")
    inputs = flash_inputs(query, key, value, None, dropout_p, bool(is_causal), scale, enable_gqa=True)
    g, o, l = payload(grad_out), payload(out), payload(logsumexp)
    if inputs is None or g is None or o is None or l is None:
        raise NotImplementedError("mojo flash attention backward: unsupported or payload-less arguments")
    q, k, v = inputs
    batch, heads_q, seq, head_dim = q._shape
    if int(max_q) != seq or int(max_k) != k._shape[2]:
        raise NotImplementedError("mojo flash attention backward: max_q/max_k must equal the sequence lengths")
    if tuple(g._shape) != tuple(q._shape) or tuple(o._shape) != tuple(q._shape):
        raise RuntimeError("mojo flash attention backward: grad_out/out shape mismatch")
    if g._dtype != q._dtype or o._dtype != q._dtype:
        raise RuntimeError("mojo flash attention backward: grad_out/out dtype mismatch")
    if l._dtype != torch.float32 or tuple(l._shape) != (batch, heads_q, seq):
        raise RuntimeError("mojo flash attention backward: logsumexp must be fp32 (B, Hq, Sq)")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    CALL_COUNTERS["aten::_scaled_dot_product_flash_attention_backward"] += 1
    return flash_backward(g, q, k, v, o, l, bool(is_causal), float(scale))
