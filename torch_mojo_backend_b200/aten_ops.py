"""The mojo device's aten registration table (PrivateUse1 kernels).

The analogue of the reference's table (torch_mojo_backend/mojo_device/mojo_device_aten_ops.py:
153-410), cut down to the flash-attention pair plus the storage plumbing the dispatcher and the
autograd engine need around it: factories, copies/transfers and metadata-only views
(reference: aten_ops/factories.py:17-58, aten_ops/transfer.py:60-185).  None of these support
ops computes attention; they move bytes or rewrite shape/stride metadata.
"""

from __future__ import annotations

import torch

from . import device_module, flash_ops
from .tensor import TorchMojoTensor, payload

_aten_ops_registry: list[tuple[str, object]] = []


def register_aten_op(op_name: str):
    def decorator(func):
        _aten_ops_registry.append((op_name, func))
        return func

    return decorator


def _index_of(device) -> int:
    if device is None:
        return device_module.current_device()
    device = torch.device(device)
    return device_module.current_device() if device.index is None else device.index


# ------------------------------------------------------------------------- factories
@register_aten_op("aten::empty.memory_format")
def mojo_empty_memory_format(size, *, dtype=None, layout=None, device=None, pin_memory=None, memory_format=None):
    dtype = torch.get_default_dtype() if dtype is None else dtype
    return TorchMojoTensor._alloc(tuple(size), dtype, _index_of(device))


@register_aten_op("aten::empty_strided")
def mojo_empty_strided(size, stride, *, dtype=None, layout=None, device=None, pin_memory=None):
    dtype = torch.get_default_dtype() if dtype is None else dtype
    return TorchMojoTensor._alloc_strided(tuple(size), tuple(stride), dtype, _index_of(device))


# ------------------------------------------------------------------------- copies / transfers
@register_aten_op("aten::_copy_from")
def mojo_copy_from(self, dest, non_blocking: bool = False):
    src, dst = payload(self), payload(dest)
    if src is not None and dst is not None:
        dst._cuda_view().copy_(src._cuda_view(), non_blocking=non_blocking)
        return dest
    if src is not None:
        # device -> host (or a foreign CUDA tensor); copy_ handles cast and layout
        dest.copy_(src._cuda_view(), non_blocking=non_blocking)
        return dest
    if dst is None:
        raise RuntimeError("aten::_copy_from reached the mojo backend without a mojo tensor")
    if dst._numel:
        dst._cuda_view().copy_(self.detach(), non_blocking=non_blocking)
    return dest


@register_aten_op("aten::_to_copy")
def mojo_to_copy(self, *, dtype=None, layout=None, device=None, pin_memory=None, non_blocking=False,
                 memory_format=None):
    src = payload(self)
    target = torch.device(device) if device is not None else None
    if src is None:
        # foreign tensor moving onto the mojo device
        t = self.detach()
        if dtype is not None and t.dtype != dtype:
            t = t.to(dtype)
        index = _index_of(target)
        if t.device.type == "cuda":
            out = TorchMojoTensor._alloc(tuple(t.shape), t.dtype, index)
            if out._numel:
                out._cuda_view().copy_(t, non_blocking=non_blocking)
            return out
        return TorchMojoTensor._from_cpu(t.cpu() if t.device.type != "cpu" else t, index, non_blocking=non_blocking)
    out_dtype = src._dtype if dtype is None else dtype
    if target is None or target.type == "mojo":
        index = src._device_index if target is None or target.index is None else target.index
        out = TorchMojoTensor._alloc(src._shape, out_dtype, index)
        if out._numel:
            out._cuda_view().copy_(src._cuda_view(), non_blocking=non_blocking)
        return out
    if target.type == "cpu":
        if out_dtype != src._dtype:
            # cast on the device first: a host-side cast would read the pinned buffer of an
            # asynchronous copy before the copy has landed
            converted = TorchMojoTensor._alloc(src._shape, out_dtype, src._device_index)
            if converted._numel:
                converted._cuda_view().copy_(src._cuda_view())
            src = converted
        return src._to_cpu_tensor(non_blocking=non_blocking)
    if target.type == "cuda":
        return src._cuda_view().to(device=target, dtype=out_dtype, copy=True)
    raise NotImplementedError(f"mojo tensors cannot be copied to {target}")


@register_aten_op("aten::clone")
def mojo_clone(self, *, memory_format=None):
    src = payload(self)
    if memory_format in (None, torch.preserve_format) and not src._is_contiguous:
        out = TorchMojoTensor._alloc_strided(src._shape, _dense_strides_like(src), src._dtype, src._device_index)
    else:
        out = TorchMojoTensor._alloc(src._shape, src._dtype, src._device_index)
    if out._numel:
        out._cuda_view().copy_(src._cuda_view())
    return out


def _dense_strides_like(t: TorchMojoTensor):
    """Dense strides that keep t's dimension order (what preserve_format means for a
    non-overlapping strided tensor)."""
    order = sorted(range(len(t._shape)), key=lambda d: (t._strides[d], -d))
    strides = [0] * len(t._shape)
    acc = 1
    for d in order:
        strides[d] = acc
        acc *= max(t._shape[d], 1)
    return tuple(strides)


# ------------------------------------------------------------------------- in-place fills used around the path
@register_aten_op("aten::zero_")
def mojo_zero_(self):
    t = payload(self)
    if t._numel:
        t._cuda_view().zero_()
    return self


@register_aten_op("aten::fill_.Scalar")
def mojo_fill_scalar(self, value):
    t = payload(self)
    if t._numel:
        t._cuda_view().fill_(value)
    return self


@register_aten_op("aten::add_.Tensor")
def mojo_add_tensor_(self, other, *, alpha=1):
    """Gradient accumulation (AccumulateGrad) and the version-counter tests touch this."""
    t = payload(self)
    o = payload(other)
    t._cuda_view().add_(o._cuda_view() if o is not None else other, alpha=alpha)
    return self


@register_aten_op("aten::add.Tensor")
def mojo_add_tensor(self, other, *, alpha=1):
    """The autograd engine sums two gradients of the same leaf with this (a tensor used twice in
    one attention call, e.g. as key and value); an unregistered op inside the engine would take
    the process down."""
    a, b = payload(self), payload(other)
    lhs = a._cuda_view() if a is not None else self
    rhs = b._cuda_view() if b is not None else other
    ref = a if a is not None else b
    result = torch.add(lhs, rhs, alpha=alpha)
    out = TorchMojoTensor._alloc(tuple(result.shape), result.dtype, ref._device_index)
    if out._numel:
        out._cuda_view().copy_(result)
    return out


# ------------------------------------------------------------------------- metadata-only views
def _meta_like(t: TorchMojoTensor) -> torch.Tensor:
    extent = t._offset + 1 + sum((d - 1) * s for d, s in zip(t._shape, t._strides)) if t._numel else t._offset + 1
    base = torch.empty((extent,), dtype=t._dtype, device="meta")
    return torch.as_strided(base, t._shape, t._strides, t._offset)


def _wrap_view(base: TorchMojoTensor, meta: torch.Tensor) -> TorchMojoTensor:
    return TorchMojoTensor._view_of(base, tuple(meta.shape), tuple(meta.stride()), meta.storage_offset())


def _register_view(op_name: str, overload):
    """View ops only rewrite (shape, strides, offset): evaluate them on a meta tensor with the
    same geometry and re-wrap the holder (reference: torch_mojo_tensor.py:400-418)."""

    def impl(self, *args, **kwargs):
        base = payload(self)
        result = overload(_meta_like(base), *args, **kwargs)
        if isinstance(result, (tuple, list)):
            return type(result)(_wrap_view(base, m) for m in result) if isinstance(result, tuple) else [
                _wrap_view(base, m) for m in result
            ]
        return _wrap_view(base, result)

    impl.__name__ = "mojo_" + op_name.replace("::", "_").replace(".", "_")
    _aten_ops_registry.append((op_name, impl))


for _name, _overload in (
    ("aten::view", torch.ops.aten.view.default),
    ("aten::_unsafe_view", torch.ops.aten._unsafe_view.default),
    ("aten::_reshape_alias", torch.ops.aten._reshape_alias.default),
    ("aten::transpose.int", torch.ops.aten.transpose.int),
    ("aten::permute", torch.ops.aten.permute.default),
    ("aten::t", torch.ops.aten.t.default),
    ("aten::split.Tensor", torch.ops.aten.split.Tensor),
    ("aten::split_with_sizes", torch.ops.aten.split_with_sizes.default),
    ("aten::select.int", torch.ops.aten.select.int),
    ("aten::slice.Tensor", torch.ops.aten.slice.Tensor),
    ("aten::unsqueeze", torch.ops.aten.unsqueeze.default),
    ("aten::squeeze.dim", torch.ops.aten.squeeze.dim),
    ("aten::expand", torch.ops.aten.expand.default),
    ("aten::as_strided", torch.ops.aten.as_strided.default),
    ("aten::alias", torch.ops.aten.alias.default),
    ("aten::detach", torch.ops.aten.detach.default),
    ("aten::unbind.int", torch.ops.aten.unbind.int),
):
    _register_view(_name, _overload)


# ------------------------------------------------------------------------- the hot path
register_aten_op("aten::_scaled_dot_product_flash_attention")(flash_ops.scaled_dot_product_flash_attention)
register_aten_op("aten::_scaled_dot_product_flash_attention_backward")(
    flash_ops.scaled_dot_product_flash_attention_backward
)
