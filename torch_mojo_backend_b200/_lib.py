"""ctypes binding of ``libb200fa.so`` (the C ABI declared in ``include/b200fa.h``).

This is the only place Python touches the native library.  It plays the role of the
reference's ``load_fa4_ops()`` (torch_mojo_backend/eager_flash_attention/__init__.py:27-46)
and ``_device_call`` (torch_mojo_backend/eager_kernels/aten_fast.py:99-106), minus the JIT:
the library is built ahead of time by ``build.py`` and must be present — there is no
fallback path, a missing library is an ``ImportError``-style hard failure.
"""

from __future__ import annotations

import ctypes
import os
from typing import Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200fa.so")

F32, BF16, F16 = 0, 1, 2
CAUSAL_NONE, CAUSAL_TOP_LEFT, CAUSAL_BOTTOM_RIGHT = 0, 1, 2
SPLITKV_MAX_ROWS = 16

OK = 0
ERR_BAD_DTYPE = -1
ERR_BAD_SHAPE = -2
ERR_BAD_STRIDE = -3
ERR_MISALIGNED = -4
ERR_WORKSPACE = -5
ERR_UNSUPPORTED = -6
ERR_CUDA = -7
ERR_NULL = -8
ERR_TIMEOUT = -9

#: every symbol include/b200fa.h declares; the CPU test-suite checks the library exports them
EXPORTED_SYMBOLS = (
    "b200fa_fwd",
    "b200fa_bwd_workspace_bytes",
    "b200fa_bwd",
    "b200fa_fwd_simt",
    "b200fa_bwd_simt",
    "b200fa_bwd_parts",
    "b200fa_bwd_no_alloc",
    "b200fa_no_alloc_scratch_bytes",
    "b200fa_fwd_dropout",
    "b200fa_bwd_dropout",
    "b200fa_dropout_threshold",
    "b200fa_dropout_bytes_host",
    "b200fa_fwd_splitkv_workspace_bytes",
    "b200fa_fwd_splitkv",
    "b200fa_set_wait_budget",
    "b200fa_wait_budget",
    "b200fa_set_fwd_tiles",
    "b200fa_fwd_tiles",
    "b200fa_status_to_error",
    "b200fa_selftest_wait_timeout",
    "b200fa_strerror",
    "b200fa_last_error_detail",
    "b200fa_version",
    "b200fa_launch_count",
)


class Tensor4(ctypes.Structure):
    """``b200fa_tensor4``: device pointer + logical (B, H, S, D) shape and element strides."""

    _fields_ = [
        ("ptr", ctypes.c_void_p),
        ("shape", ctypes.c_int64 * 4),
        ("stride", ctypes.c_int64 * 4),
    ]

    @classmethod
    def make(cls, ptr: int, shape: Sequence[int], stride: Sequence[int]) -> "Tensor4":
        if len(shape) != 4 or len(stride) != 4:
            raise ValueError("b200fa tensors are 4-D (batch, heads, seq, head_dim)")
        return cls(ctypes.c_void_p(ptr), (ctypes.c_int64 * 4)(*shape), (ctypes.c_int64 * 4)(*stride))


class B200FAError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        detail = load().b200fa_last_error_detail().decode() if code == ERR_CUDA else ""
        super().__init__(f"{where}: {strerror(code)} (b200fa error {code})" + (f" [{detail}]" if detail else ""))


_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once and declare its signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m torch_mojo_backend_b200.build` "
            "(there is no fallback implementation)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    t4p = ctypes.POINTER(Tensor4)
    fwd_args = [t4p, t4p, t4p, t4p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    bwd_args = [t4p, t4p, t4p, t4p, t4p, ctypes.c_void_p, t4p, t4p, t4p, ctypes.c_void_p, ctypes.c_size_t,
                ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    for name in ("b200fa_fwd", "b200fa_fwd_simt"):
        fn = getattr(lib, name)
        fn.argtypes = fwd_args
        fn.restype = ctypes.c_int
    for name in ("b200fa_bwd", "b200fa_bwd_simt"):
        fn = getattr(lib, name)
        fn.argtypes = bwd_args
        fn.restype = ctypes.c_int
    # the no-alloc backward has b200fa_bwd's signature minus (workspace, workspace_bytes)
    lib.b200fa_bwd_no_alloc.argtypes = bwd_args[:9] + bwd_args[11:]
    lib.b200fa_bwd_no_alloc.restype = ctypes.c_int
    lib.b200fa_no_alloc_scratch_bytes.argtypes = []
    lib.b200fa_no_alloc_scratch_bytes.restype = ctypes.c_size_t
    lib.b200fa_bwd_parts.argtypes = bwd_args + [ctypes.c_int]
    lib.b200fa_bwd_parts.restype = ctypes.c_int
    drop_args = [ctypes.c_float, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int]
    lib.b200fa_fwd_dropout.argtypes = fwd_args[:8] + drop_args + fwd_args[8:]
    lib.b200fa_fwd_dropout.restype = ctypes.c_int
    lib.b200fa_bwd_dropout.argtypes = bwd_args[:14] + drop_args + bwd_args[14:]
    lib.b200fa_bwd_dropout.restype = ctypes.c_int
    lib.b200fa_dropout_threshold.argtypes = [ctypes.c_float]
    lib.b200fa_dropout_threshold.restype = ctypes.c_uint32
    lib.b200fa_dropout_bytes_host.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int64, ctypes.c_int64,
                                              ctypes.c_int64, ctypes.c_void_p]
    lib.b200fa_dropout_bytes_host.restype = None
    lib.b200fa_fwd_splitkv_workspace_bytes.argtypes = [ctypes.c_int64] * 6
    lib.b200fa_fwd_splitkv_workspace_bytes.restype = ctypes.c_size_t
    lib.b200fa_fwd_splitkv.argtypes = [t4p, t4p, t4p, t4p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                       ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_int,
                                       ctypes.c_void_p]
    lib.b200fa_fwd_splitkv.restype = ctypes.c_int
    lib.b200fa_set_wait_budget.argtypes = [ctypes.c_longlong]
    lib.b200fa_set_wait_budget.restype = None
    lib.b200fa_wait_budget.argtypes = []
    lib.b200fa_wait_budget.restype = ctypes.c_longlong
    lib.b200fa_set_fwd_tiles.argtypes = [ctypes.c_int]
    lib.b200fa_set_fwd_tiles.restype = None
    lib.b200fa_fwd_tiles.argtypes = []
    lib.b200fa_fwd_tiles.restype = ctypes.c_int
    lib.b200fa_status_to_error.argtypes = [ctypes.c_uint32]
    lib.b200fa_status_to_error.restype = ctypes.c_int
    lib.b200fa_selftest_wait_timeout.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int]
    lib.b200fa_selftest_wait_timeout.restype = ctypes.c_int
    lib.b200fa_bwd_workspace_bytes.argtypes = [ctypes.c_int64] * 5 + [ctypes.c_int]
    lib.b200fa_bwd_workspace_bytes.restype = ctypes.c_size_t
    lib.b200fa_strerror.argtypes = [ctypes.c_int]
    lib.b200fa_strerror.restype = ctypes.c_char_p
    lib.b200fa_last_error_detail.argtypes = []
    lib.b200fa_last_error_detail.restype = ctypes.c_char_p
    lib.b200fa_version.argtypes = []
    lib.b200fa_version.restype = ctypes.c_int
    lib.b200fa_launch_count.argtypes = []
    lib.b200fa_launch_count.restype = ctypes.c_uint64
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().b200fa_strerror(code).decode()


def version() -> int:
    return load().b200fa_version()


def launch_count() -> int:
    return int(load().b200fa_launch_count())


def bwd_workspace_bytes(B: int, Hq: int, Hkv: int, S: int, D: int, dtype: int) -> int:
    return int(load().b200fa_bwd_workspace_bytes(B, Hq, Hkv, S, D, dtype))


def causal_code(causal) -> int:
    """bool or B200FA_CAUSAL_* -> the integer the library takes (True = top-left, torch's rule)."""
    return int(causal)


def fwd(q: Tensor4, k: Tensor4, v: Tensor4, out: Tensor4, lse_ptr: int, dtype: int, causal,
        scale: float, stream: int, device: int, status_ptr: int = 0, *, simt: bool = False,
        dropout=None) -> int:
    """Raw forward call; returns the library's status code.  `causal` is a bool or one of
    CAUSAL_*; `dropout` is None or ``(p, seed, offset)``."""
    head = (ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(out), ctypes.c_void_p(lse_ptr),
            dtype, causal_code(causal), ctypes.c_float(scale))
    tail = (ctypes.c_void_p(stream), device, ctypes.c_void_p(status_ptr))
    if dropout is not None:
        p, seed, offset = dropout
        return load().b200fa_fwd_dropout(*head, ctypes.c_float(p), ctypes.c_uint64(seed), ctypes.c_uint64(offset),
                                         1 if simt else 0, *tail)
    fn = load().b200fa_fwd_simt if simt else load().b200fa_fwd
    return fn(*head, *tail)


def bwd(q: Tensor4, k: Tensor4, v: Tensor4, out: Tensor4, dout: Tensor4, lse_ptr: int, dq: Tensor4,
        dk: Tensor4, dv: Tensor4, workspace_ptr: int, workspace_bytes: int, dtype: int, causal,
        scale: float, stream: int, device: int, status_ptr: int = 0, *, simt: bool = False,
        parts: int = 7, dropout=None) -> int:
    """Raw backward call; returns the library's status code.  `parts` != 7 runs a subset of
    the three backward kernels (see b200fa_bwd_parts); `dropout` is None or ``(p, seed, offset)``
    and must repeat the forward's."""
    head = (ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(out), ctypes.byref(dout),
            ctypes.c_void_p(lse_ptr), ctypes.byref(dq), ctypes.byref(dk), ctypes.byref(dv),
            ctypes.c_void_p(workspace_ptr), ctypes.c_size_t(workspace_bytes), dtype, causal_code(causal),
            ctypes.c_float(scale))
    tail = (ctypes.c_void_p(stream), device, ctypes.c_void_p(status_ptr))
    if dropout is not None:
        p, seed, offset = dropout
        return load().b200fa_bwd_dropout(*head, ctypes.c_float(p), ctypes.c_uint64(seed), ctypes.c_uint64(offset),
                                         1 if simt else 0, *tail)
    if parts != 7:
        return load().b200fa_bwd_parts(*head, *tail, parts)
    fn = load().b200fa_bwd_simt if simt else load().b200fa_bwd
    return fn(*head, *tail)


def fwd_splitkv_workspace_bytes(B: int, Hq: int, Hkv: int, Sq: int, Sk: int, D: int) -> int:
    return int(load().b200fa_fwd_splitkv_workspace_bytes(B, Hq, Hkv, Sq, Sk, D))


def fwd_splitkv(q: Tensor4, k: Tensor4, v: Tensor4, out: Tensor4, lse_ptr: int, workspace_ptr: int,
                workspace_bytes: int, dtype: int, causal, scale: float, stream: int, device: int,
                status_ptr: int = 0) -> int:
    """Raw split-KV (decode) forward; returns the library's status code."""
    return load().b200fa_fwd_splitkv(
        ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(out), ctypes.c_void_p(lse_ptr),
        ctypes.c_void_p(workspace_ptr), ctypes.c_size_t(workspace_bytes), dtype, causal_code(causal),
        ctypes.c_float(scale), ctypes.c_void_p(stream), device, ctypes.c_void_p(status_ptr))


def dropout_threshold(p: float) -> int:
    return int(load().b200fa_dropout_threshold(ctypes.c_float(p)))


def dropout_bytes_host(seed: int, offset: int, batch_head: int, row: int, col_block: int) -> bytes:
    """The 16 mask bytes of one Philox call, evaluated on the host by the library's own code."""
    buf = (ctypes.c_uint8 * 16)()
    load().b200fa_dropout_bytes_host(seed, offset, batch_head, row, col_block, buf)
    return bytes(buf)


def set_wait_budget(cycles: int) -> None:
    load().b200fa_set_wait_budget(int(cycles))


def wait_budget() -> int:
    return int(load().b200fa_wait_budget())


def set_fwd_tiles(tiles: int) -> None:
    """Query tiles per forward thread block: 0 = chosen per problem, 1 or 2 = forced (tests, measurements)."""
    load().b200fa_set_fwd_tiles(int(tiles))


def fwd_tiles() -> int:
    return int(load().b200fa_fwd_tiles())


def status_to_error(status_value: int) -> int:
    return int(load().b200fa_status_to_error(int(status_value) & 0xFFFFFFFF))


def selftest_wait_timeout(status_ptr: int, budget_cycles: int, stream: int, device: int) -> int:
    return load().b200fa_selftest_wait_timeout(ctypes.c_void_p(status_ptr), int(budget_cycles),
                                               ctypes.c_void_p(stream), device)


def no_alloc_scratch_bytes() -> int:
    return int(load().b200fa_no_alloc_scratch_bytes())


def bwd_no_alloc(q: Tensor4, k: Tensor4, v: Tensor4, out: Tensor4, dout: Tensor4, lse_ptr: int, dq: Tensor4,
                 dk: Tensor4, dv: Tensor4, dtype: int, causal: bool, scale: float, stream: int, device: int,
                 status_ptr: int = 0) -> int:
    """Backward for callers that cannot allocate: the scratch is the library's built-in device
    array (see b200fa_bwd_no_alloc in include/b200fa.h).  The caller passes every input and
    output; this wrapper allocates nothing either.  Returns the library's status code."""
    return load().b200fa_bwd_no_alloc(
        ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(out), ctypes.byref(dout),
        ctypes.c_void_p(lse_ptr), ctypes.byref(dq), ctypes.byref(dk), ctypes.byref(dv), dtype, causal_code(causal),
        ctypes.c_float(scale), ctypes.c_void_p(stream), device, ctypes.c_void_p(status_ptr))
