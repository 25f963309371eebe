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
# B200FA_LIB overrides the library path (used to try experimental builds)
LIB_PATH = os.environ.get("B200FA_LIB") or os.path.join(_HERE, "libb200fa.so")

F32, BF16, F16 = 0, 1, 2

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


def fwd(q: Tensor4, k: Tensor4, v: Tensor4, out: Tensor4, lse_ptr: int, dtype: int, causal: bool,
        scale: float, stream: int, device: int, status_ptr: int = 0, *, simt: bool = False) -> int:
    """Raw forward call; returns the library's status code."""
    fn = load().b200fa_fwd_simt if simt else load().b200fa_fwd
    return fn(ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(out), ctypes.c_void_p(lse_ptr),
              dtype, 1 if causal else 0, ctypes.c_float(scale), ctypes.c_void_p(stream), device,
              ctypes.c_void_p(status_ptr))


def bwd(q: Tensor4, k: Tensor4, v: Tensor4, out: Tensor4, dout: Tensor4, lse_ptr: int, dq: Tensor4,
        dk: Tensor4, dv: Tensor4, workspace_ptr: int, workspace_bytes: int, dtype: int, causal: bool,
        scale: float, stream: int, device: int, status_ptr: int = 0, *, simt: bool = False,
        parts: int = 7) -> int:
    """Raw backward call; returns the library's status code.  `parts` != 7 runs a subset of
    the three backward kernels (see b200fa_bwd_parts)."""
    if parts != 7:
        return load().b200fa_bwd_parts(
            ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(out), ctypes.byref(dout),
            ctypes.c_void_p(lse_ptr), ctypes.byref(dq), ctypes.byref(dk), ctypes.byref(dv),
            ctypes.c_void_p(workspace_ptr), ctypes.c_size_t(workspace_bytes), dtype, 1 if causal else 0,
            ctypes.c_float(scale), ctypes.c_void_p(stream), device, ctypes.c_void_p(status_ptr), parts)
    fn = load().b200fa_bwd_simt if simt else load().b200fa_bwd
    return fn(ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(out), ctypes.byref(dout),
              ctypes.c_void_p(lse_ptr), ctypes.byref(dq), ctypes.byref(dk), ctypes.byref(dv),
              ctypes.c_void_p(workspace_ptr), ctypes.c_size_t(workspace_bytes), dtype, 1 if causal else 0,
              ctypes.c_float(scale), ctypes.c_void_p(stream), device, ctypes.c_void_p(status_ptr))


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
        ctypes.c_void_p(lse_ptr), ctypes.byref(dq), ctypes.byref(dk), ctypes.byref(dv), dtype, 1 if causal else 0,
        ctypes.c_float(scale), ctypes.c_void_p(stream), device, ctypes.c_void_p(status_ptr))
