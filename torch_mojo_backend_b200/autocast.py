"""``AutocastPrivateUse1`` policy rows for the attention ops.

The reference casts SDPA and the flash op to the autocast dtype
(torch_mojo_backend/mojo_device/mojo_device_autocast.py:73-91); this is how a bf16-autocast
nanoGPT block reaches the 16-bit kernels.  Everything else falls through.
"""

from __future__ import annotations

import functools
from collections.abc import Mapping

import torch

_AUTOCAST_KEYSET = torch._C.DispatchKeySet(torch._C.DispatchKey.AutocastPrivateUse1)
_registered = False
_fallback_library = None
_aten_library = None


def _cast_mojo_floating(value, dtype):
    if isinstance(value, torch.Tensor):
        if value.device.type == "mojo" and value.is_floating_point() and value.dtype != dtype:
            return value.to(dtype=dtype)
        return value
    if isinstance(value, tuple):
        return tuple(_cast_mojo_floating(v, dtype) for v in value)
    if isinstance(value, list):
        return [_cast_mojo_floating(v, dtype) for v in value]
    if isinstance(value, Mapping):
        return {k: _cast_mojo_floating(v, dtype) for k, v in value.items()}
    return value


def _lower_precision_wrapper(op):
    @functools.wraps(op)
    def wrapper(*args, **kwargs):
        # the casts must redispatch below AutocastPrivateUse1 or they would re-enter this layer
        with torch._C._ExcludeDispatchKeyGuard(_AUTOCAST_KEYSET):
            dtype = torch.get_autocast_dtype("mojo")
            return op(*_cast_mojo_floating(args, dtype), **_cast_mojo_floating(kwargs, dtype))

    return wrapper


def register_autocast_ops() -> None:
    global _registered, _fallback_library, _aten_library
    if _registered:
        return
    _fallback_library = torch.library.Library("_", "IMPL", "AutocastPrivateUse1")
    _fallback_library.fallback(torch.library.fallthrough_kernel)
    _aten_library = torch.library.Library("aten", "IMPL", "AutocastPrivateUse1")
    for op in (
        torch.ops.aten.scaled_dot_product_attention.default,
        torch.ops.aten._scaled_dot_product_flash_attention.default,
    ):
        _aten_library.impl(op._schema.name, _lower_precision_wrapper(op))
    _registered = True
