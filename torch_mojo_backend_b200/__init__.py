"""B200-native flash attention behind the `mojo` PyTorch device.

``register_mojo_devices()`` installs the device (PrivateUse1 renamed ``mojo``), the two flash
attention aten ops, the SDPA autograd router and the autocast rows — the reference's
``register_mojo_devices`` (torch_mojo_backend/mojo_device/register.py:217-275) cut down to the
flash-attention path.  The kernels live in ``libb200fa.so`` (C ABI in ``include/b200fa.h``).
"""

from __future__ import annotations

import torch

_registered = False


def register_mojo_devices() -> None:
    """Enable the mojo device globally and register its aten ops (idempotent)."""
    global _registered
    if _registered:
        return
    from torch.utils.backend_registration import _setup_privateuseone_for_python_backend

    from . import _lib, aten_ops, autocast, autograd, device_module

    _lib.load()  # fail now, loudly, if the native library is missing
    torch.__future__.set_swap_module_params_on_conversion(True)
    _setup_privateuseone_for_python_backend("mojo", backend_module=device_module)
    for op_name, func in aten_ops._aten_ops_registry:
        torch.library.impl(op_name, "privateuseone")(func)
    autograd.register_autograd_ops()
    autocast.register_autocast_ops()
    _registered = True


def from_cuda(t: torch.Tensor):
    """Zero-copy: view a CUDA tensor's memory as a mojo tensor (same physical GPU)."""
    from .tensor import TorchMojoTensor

    return TorchMojoTensor._from_cuda(t)


def pinned_empty(shape, dtype: torch.dtype) -> torch.Tensor:
    """A page-locked CPU tensor usable for non-blocking copies to and from mojo tensors."""
    from .tensor import pinned_empty as _pinned_empty

    return _pinned_empty(shape, dtype)


def to_cuda(t) -> torch.Tensor:
    """Zero-copy: the CUDA tensor aliasing a mojo tensor's memory."""
    return t._cuda_view()


def __getattr__(name):
    if name == "HostAttentionPipeline":
        from .host_pipeline import HostAttentionPipeline

        return HostAttentionPipeline
    raise AttributeError(name)


__all__ = ["register_mojo_devices", "from_cuda", "to_cuda", "pinned_empty", "HostAttentionPipeline"]
