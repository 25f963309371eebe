"""Host side of the two flash-attention aten ops on the `mojo` device.

Thin Python over the C ABI: eligibility gate, layout routing, output/scratch allocation and
the aten return contracts.  It mirrors, function by function, the FA4 section of the
reference's eager layer (torch_mojo_backend/eager_kernels/aten_fast.py:6971-7408 and
7699-7839); every device computation happens inside ``libb200fa.so``.  There is no fallback:
an ineligible call raises ``NotImplementedError`` from the forward.
"""

from __future__ import annotations

import math
import os

import torch

from . import _lib, device_module
from .tensor import TorchMojoTensor, payload

_DTYPE_CODES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}

#: per-op call counters, the analogue of the reference's EAGER_CALL_COUNTERS
#: (torch_mojo_backend/mojo_device/mojo_device_aten_ops.py:84-109)
CALL_COUNTERS = {
    "aten::_scaled_dot_product_flash_attention": 0,
    "aten::_scaled_dot_product_flash_attention_backward": 0,
    "backward_recomputed_forward": 0,
    "forward_split_kv": 0,
}

#: a decode-shaped forward (few query rows, long key sequence) goes to the split-KV kernels
_SPLITKV_MIN_KEYS = 512


def _decode_shaped(batch: int, heads_q: int, heads_kv: int, seq_q: int, seq_k: int) -> bool:
    """A forward that the split-KV kernels serve faster than the prefill kernel: at most 16 query
    rows per KV head over a long key sequence.  The split-KV pass reads K and V once per KV head at
    0.8-1.0 of the HBM copy rate whatever the row count (measured on B200: B16 Hq32 Hkv8 Sq4
    Sk16384, 0.19 ms against the prefill kernel's 0.75)."""
    rows = (heads_q // heads_kv) * seq_q
    return seq_k >= _SPLITKV_MIN_KEYS and rows <= _lib.SPLITKV_MAX_ROWS


def _log(msg: str) -> None:
    """B200FA_LOG=1 prints one line per native call (the reference gates its eager logging the
    same way, torch_mojo_backend/flags.py:6-33)."""
    if os.environ.get("B200FA_LOG", "0") not in ("", "0"):
        print(f"[b200fa] {msg}", flush=True)


def _stream_for(index: int) -> int:
    """The CUDA stream (as an integer handle) every mojo op on device `index` is ordered on."""
    return torch.cuda.current_stream(index).cuda_stream


# --------------------------------------------------------------------------- device status word
# One uint32 per device that every kernel launched from here may write when an internal wait
# runs out of its budget.  It is read back at explicit synchronisation points only
# (torch.mojo.synchronize, check_status), never on the launch path.
_status_words: dict[int, TorchMojoTensor] = {}


def _status_ptr(index: int) -> int:
    word = _status_words.get(index)
    if word is None:
        word = TorchMojoTensor._alloc((1,), torch.int32, index)
        word._cuda_view().zero_()
        _status_words[index] = word
    return word._ptr


def check_status(index: int | None = None) -> None:
    """Synchronise with the device and raise ``B200FAError(ERR_TIMEOUT)`` if a kernel launched
    through the mojo ops gave up on an internal wait since the last check (its outputs are then
    not to be trusted).  The word is cleared, so the next call starts clean."""
    indices = list(_status_words) if index is None else [index]
    for i in indices:
        word = _status_words.get(i)
        if word is None:
            continue
        value = int(word._cuda_view().item()) & 0xFFFFFFFF   # synchronises
        if value:
            word._cuda_view().zero_()
            rc = _lib.status_to_error(value)
            raise _lib.B200FAError(rc, f"a mojo flash-attention kernel reported status 0x{value:08x}")


# --------------------------------------------------------------------------- eligibility
def flash_inputs(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None,
                 enable_gqa=False):
    """Return ``(q, k, v)`` payload tensors if the call is served by the kernels, else None.

    Metadata only — no device work.  Wider than the reference's gate
    (aten_fast.py:6971-7043, which needs causal, 16-bit, equal head counts, Sq == Sk and sm_90a):
    fp32/bf16/fp16, causal or not (is_causal over ``Sq != Sk`` follows torch's rule: the diagonal
    starts at the top-left corner), ``Hq % Hkv == 0`` (needs ``enable_gqa`` when they differ),
    head_dim 64 or 128, no attn_mask, ``0 <= dropout_p < 1`` (16-bit tensors, or fp32), finite
    positive scale.
    """
    q, k, v = payload(query), payload(key), payload(value)
    if q is None or k is None or v is None or attn_mask is not None:
        return None
    if not isinstance(dropout_p, (int, float)) or isinstance(dropout_p, bool):
        return None
    if not (0.0 <= float(dropout_p) < 1.0):
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
    if kb != batch or kd != head_dim:
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


def _dropout_arg(dropout_p: float, philox):
    """None without dropout, else the (p, seed, offset) triple the library takes."""
    if not dropout_p:
        return None
    seed, offset = philox
    return (float(dropout_p), int(seed), int(offset))


# --------------------------------------------------------------------------- forward
def flash_forward(q: TorchMojoTensor, k: TorchMojoTensor, v: TorchMojoTensor, is_causal: bool,
                  scale: float | None, dropout_p: float = 0.0, philox=(0, 0)):
    """Allocate ``out`` (same dtype as q) and ``lse`` (fp32, (B,Hq,Sq)), enqueue the forward
    kernel, return ``(out, lse, q_used, k_used, v_used)`` like
    ``fast_fa4_16bit_d64_causal_forward`` (aten_fast.py:7151-7285).  A decode-shaped call (all
    query rows of a GQA group fit one split-KV thread block, long key sequence, no dropout) goes
    to the split-KV kernels, the counterpart of the reference's decode path
    (aten_fast.py:9171-9203)."""
    batch, heads_q, seq, head_dim = q._shape
    heads_kv, seq_k = k._shape[1], k._shape[2]
    index = q._device_index
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    q_used, k_used, v_used = prepare(q), prepare(k), prepare(v)
    out = _alloc_like_layout(q._shape, q._dtype, index, bthd_stored(q_used))
    lse = TorchMojoTensor._alloc((batch, heads_q, seq), torch.float32, index)
    code = _DTYPE_CODES[q._dtype]
    if not dropout_p and _decode_shaped(batch, heads_q, heads_kv, seq, seq_k):
        nbytes = _lib.fwd_splitkv_workspace_bytes(batch, heads_q, heads_kv, seq, seq_k, head_dim)
        workspace = TorchMojoTensor._alloc((nbytes,), torch.uint8, index)
        _log(f"fwd_splitkv B={batch} Hq={heads_q} Hkv={heads_kv} Sq={seq} Sk={seq_k} D={head_dim}")
        rc = _lib.fwd_splitkv(_t4(q_used), _t4(k_used), _t4(v_used), _t4(out), lse._ptr, workspace._ptr, nbytes,
                              code, bool(is_causal), float(scale), _stream_for(index), index, _status_ptr(index))
        _check(rc, "b200fa_fwd_splitkv")
        CALL_COUNTERS["forward_split_kv"] += 1
        return out, lse, q_used, k_used, v_used
    _log(f"fwd B={batch} Hq={heads_q} Hkv={heads_kv} Sq={seq} Sk={seq_k} D={head_dim} causal={is_causal} p={dropout_p}")
    rc = _lib.fwd(_t4(q_used), _t4(k_used), _t4(v_used), _t4(out), lse._ptr, code, bool(is_causal), float(scale),
                  _stream_for(index), index, _status_ptr(index), dropout=_dropout_arg(dropout_p, philox))
    _check(rc, "b200fa_fwd")
    return out, lse, q_used, k_used, v_used


def scaled_dot_product_flash_attention(query, key, value, dropout_p=0.0, is_causal=False,
                                       return_debug_mask=False, *, scale=None):
    """``aten::_scaled_dot_product_flash_attention`` on the mojo device.

    Returns the CUDA-shaped 9-tuple ``(out, logsumexp, cum_seq_q=None, cum_seq_k=None, max_q,
    max_k, rng_state uint64[2], unused uint64[], debug_attn_mask empty(0))`` like the reference
    (aten_fast.py:7699-7734).  Unlike the reference, whose Philox slots are placeholders because it
    declines dropout, ``rng_state`` holds the real ``(seed, offset)`` the dropout mask was drawn
    from: the device's generator reserves B*Hq counter values per call
    (``torch.mojo._reserve_philox_state``), and the backward regenerates the same mask from it.
    """
    if return_debug_mask:
        raise NotImplementedError(
            "aten::_scaled_dot_product_flash_attention on mojo: return_debug_mask is not supported"
        )
    inputs = flash_inputs(query, key, value, None, dropout_p, is_causal, scale, enable_gqa=True)
    if inputs is None:
        raise NotImplementedError(
            "aten::_scaled_dot_product_flash_attention on mojo needs fp32/bf16/fp16 (B,H,S,D) tensors with "
            "head_dim 64 or 128, Hq % Hkv == 0, 0 <= dropout_p < 1 and a positive finite scale"
        )
    q, k, v = inputs
    CALL_COUNTERS["aten::_scaled_dot_product_flash_attention"] += 1
    index = q._device_index
    dropout_p = float(dropout_p)
    seed = offset = 0
    if dropout_p:
        seed, offset = device_module._reserve_philox_state(index, q._shape[0] * q._shape[1])
    out, lse, _, _, _ = flash_forward(q, k, v, is_causal, scale, dropout_p, (seed, offset))
    rng_state = TorchMojoTensor._alloc((2,), torch.uint64, index)
    if dropout_p:
        # the pair as two signed 64-bit patterns (uint64 copies are not universally supported)
        host = torch.tensor([seed, offset], dtype=torch.uint64).view(torch.int64)
        rng_state._cuda_view().view(torch.int64).copy_(host)
    rng_state._philox = (seed, offset)   # host-side copy: the backward needs no read-back
    unused = TorchMojoTensor._alloc((), torch.uint64, index)
    debug_attn_mask = TorchMojoTensor._alloc((0,), q._dtype, index)
    return (out, lse, None, None, q._shape[2], k._shape[2], rng_state, unused, debug_attn_mask)


# --------------------------------------------------------------------------- backward
def flash_backward(dout, q, k, v, out, lse, is_causal: bool, scale: float, dropout_p: float = 0.0,
                   philox=(0, 0)):
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
    _log(f"bwd B={batch} Hq={heads_q} Hkv={heads_kv} Sq={seq} Sk={k._shape[2]} D={head_dim} causal={is_causal} p={dropout_p}")
    rc = _lib.bwd(_t4(q_used), _t4(k_used), _t4(v_used), _t4(out_used), _t4(dout_used), lse_used._ptr,
                  _t4(dq), _t4(dk), _t4(dv), workspace._ptr, nbytes, code, bool(is_causal), float(scale),
                  _stream_for(index), index, _status_ptr(index), dropout=_dropout_arg(dropout_p, philox))
    _check(rc, "b200fa_bwd")
    # `workspace` drops here: the allocator re-uses it only for work queued later on this stream
    return dq, dk, dv


def _philox_of(philox_seed, dropout_p: float):
    """The (seed, offset) the forward drew its mask from: the host-side copy riding on the
    rng_state tensor, else (a tensor that lost it) a read-back of its two words."""
    if not dropout_p:
        return (0, 0)
    pair = getattr(philox_seed, "_philox", None)
    if pair is not None:
        return pair
    t = payload(philox_seed)
    if t is None:
        raise NotImplementedError("mojo flash attention backward: dropout needs the forward's rng_state")
    words = t._cuda_view().view(torch.int64).cpu().view(torch.uint64)
    return (int(words[0]), int(words[1]))


def scaled_dot_product_flash_attention_backward(grad_out, query, key, value, out, logsumexp, cum_seq_q,
                                                cum_seq_k, max_q, max_k, dropout_p, is_causal, philox_seed,
                                                philox_offset, *, scale=None):
    """``aten::_scaled_dot_product_flash_attention_backward`` on the mojo device
    (aten_fast.py:7737-7839): validates the 14 positional arguments, then one bridge call.

    This runs inside an autograd node, where an exception would take the process down
    (torch_mojo_backend/mojo_device/aten_ops/support.py:67-101), so everything that can be
    refused is refused by the forward; what is left here are programming errors.  Like the
    reference (aten_fast.py:7805-7818), ``out`` / ``logsumexp`` that arrive without their device
    payload do not fail the backward: the forward is recomputed from q, k, v.
    """
    if cum_seq_q is not None or cum_seq_k is not None:
        raise NotImplementedError("mojo flash attention backward: varlen (cum_seq) is not supported")
    dropout_p = float(dropout_p)
    inputs = flash_inputs(query, key, value, None, dropout_p, bool(is_causal), scale, enable_gqa=True)
    g = payload(grad_out)
    if inputs is None or g is None:
        raise NotImplementedError("mojo flash attention backward: unsupported or payload-less q/k/v/grad_out")
    q, k, v = inputs
    batch, heads_q, seq, head_dim = q._shape
    if int(max_q) != seq or int(max_k) != k._shape[2]:
        raise NotImplementedError("mojo flash attention backward: max_q/max_k must equal the sequence lengths")
    if tuple(g._shape) != tuple(q._shape) or g._dtype != q._dtype:
        raise RuntimeError("mojo flash attention backward: grad_out shape/dtype mismatch")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    philox = _philox_of(philox_seed, dropout_p)
    o, l = payload(out), payload(logsumexp)
    usable = (o is not None and l is not None and tuple(o._shape) == tuple(q._shape) and o._dtype == q._dtype
              and l._dtype == torch.float32 and tuple(l._shape) == (batch, heads_q, seq))
    if not usable:
        CALL_COUNTERS["backward_recomputed_forward"] += 1
        o, l, _, _, _ = flash_forward(q, k, v, bool(is_causal), float(scale), dropout_p, philox)
    CALL_COUNTERS["aten::_scaled_dot_product_flash_attention_backward"] += 1
    return flash_backward(g, q, k, v, o, l, bool(is_causal), float(scale), dropout_p, philox)
