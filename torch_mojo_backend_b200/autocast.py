"""Autocast for the attention ops of the mojo device.

Under ``torch.autocast("mojo", dtype=...)`` the two attention entry points cast their q, k and v
to the autocast dtype before dispatching on, which is how a bf16-autocast nanoGPT block reaches
the 16-bit tensor-core kernels (the reference lists the same two ops among its lower-precision
autocast rows, torch_mojo_backend/mojo_device/mojo_device_autocast.py:73-91).  Every other op
falls through the autocast key untouched.
"""

from __future__ import annotations

import torch

_AUTOCAST_KEY = torch._C.DispatchKeySet(torch._C.DispatchKey.AutocastPrivateUse1)
_libraries: list = []   # keeps the torch.library objects (and with them the registrations) alive


def _to_autocast_dtype(t):
    dtype = torch.get_autocast_dtype("mojo")
    if isinstance(t, torch.Tensor) and t.device.type == "mojo" and t.is_floating_point() and t.dtype != dtype:
        return t.to(dtype)
    return t


def _sdpa(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *, scale=None, enable_gqa=False):
    # below the autocast key, or the casts and the call would come straight back here
    with torch._C._ExcludeDispatchKeyGuard(_AUTOCAST_KEY):
        q, k, v = (_to_autocast_dtype(t) for t in (query, key, value))
        return torch.ops.aten.scaled_dot_product_attention.default(
            q, k, v, attn_mask, dropout_p, is_causal, scale=scale, enable_gqa=enable_gqa)


def _flash(query, key, value, dropout_p=0.0, is_causal=False, return_debug_mask=False, *, scale=None):
    with torch._C._ExcludeDispatchKeyGuard(_AUTOCAST_KEY):
        q, k, v = (_to_autocast_dtype(t) for t in (query, key, value))
        return torch.ops.aten._scaled_dot_product_flash_attention.default(
            q, k, v, dropout_p, is_causal, return_debug_mask, scale=scale)


def register_autocast_ops() -> None:
    if _libraries:
        return
    everything_else = torch.library.Library("_", "IMPL", "AutocastPrivateUse1")
    everything_else.fallback(torch.library.fallthrough_kernel)
    attention = torch.library.Library("aten", "IMPL", "AutocastPrivateUse1")
    attention.impl("scaled_dot_product_attention", _sdpa)
    attention.impl("_scaled_dot_product_flash_attention", _flash)
    _libraries.extend((everything_else, attention))
