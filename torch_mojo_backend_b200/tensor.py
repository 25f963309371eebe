"""``TorchMojoTensor``: the mojo-device tensor and its storage contract.

Mirrors the reference's wrapper (torch_mojo_backend/mojo_device/torch_mojo_tensor.py:309-418):
the torch-side TensorImpl is a storage-less ``PrivateUse1`` wrapper subclass; the real
allocation is a dtype-erased byte buffer owned by a refcounted *holder*; views share the holder
and differ only in Python metadata (``_ptr`` has the storage offset applied, ``_strides`` and
``_offset`` are in elements).  Here the holder is a flat ``uint8`` CUDA tensor from torch's
caching allocator, so allocation, kernels and the stream-ordered free all ride torch's current
CUDA stream, and ``_ptr`` is a plain CUDA device address the C ABI consumes directly.
"""

from __future__ import annotations

import math
import weakref

import torch

from . import device_module

_WRAPPER_DEVICE_TYPE = "privateuseone"


def _row_major_strides(shape) -> tuple[int, ...]:
    strides = []
    acc = 1
    for dim in reversed(tuple(shape)):
        strides.append(acc)
        acc *= max(int(dim), 1)
    return tuple(reversed(strides))


def _compute_contiguous(shape, strides) -> bool:
    expected = 1
    for dim, stride in zip(reversed(tuple(shape)), reversed(tuple(strides))):
        if dim == 1:
            continue
        if stride != expected:
            return False
        expected *= dim
    return True


def _host_unregister(ptr: int) -> None:
    try:
        torch.cuda.cudart().cudaHostUnregister(ptr)
    except Exception:
        pass


def pinned_empty(shape, dtype: torch.dtype) -> torch.Tensor:
    """A page-locked CPU tensor for asynchronous transfers.

    Once a PrivateUse1 backend is registered, ``torch.empty(pin_memory=True)`` and
    ``Tensor.pin_memory()`` ask that backend for a pinned allocator, which a Python backend
    cannot provide; this registers ordinary host memory with the CUDA driver instead.  The
    registration is dropped when the returned tensor object is collected.
    """
    t = torch.empty(tuple(shape), dtype=dtype)
    nbytes = t.numel() * t.element_size()
    if nbytes:
        rc = torch.cuda.cudart().cudaHostRegister(t.data_ptr(), nbytes, 0)
        if int(rc) != 0:
            raise RuntimeError(f"cudaHostRegister failed with error {int(rc)}")
        weakref.finalize(t, _host_unregister, t.data_ptr())
    return t


def _alloc_holder(nbytes: int, index: int) -> torch.Tensor:
    """One device allocation: a flat byte buffer on CUDA device `index` (never zero bytes)."""
    return torch.empty((max(int(nbytes), 1),), dtype=torch.uint8, device=torch.device("cuda", index))


def _holder_ptr(holder: torch.Tensor) -> int:
    return holder.data_ptr()


class TorchMojoTensor(torch.Tensor):
    """Eager mojo tensor: a storage-less wrapper plus the Python payload
    ``_holder, _ptr, _shape, _strides, _offset, _dtype, _itemsize, _numel, _device_index,
    _torch_device, _is_contiguous``."""

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        if not all(issubclass(cls, t) for t in types):
            return NotImplemented
        # Redispatch below the Python key so the call reaches the PrivateUse1 kernels
        # registered in aten_ops.py (reference: deferred_compile.py:53-58).
        with torch._C._DisableTorchDispatch():
            return func(*args, **(kwargs or {}))

    __torch_function__ = torch._C._disabled_torch_function_impl

    # ------------------------------------------------------------------ construction
    @classmethod
    def _make(cls, holder, ptr, shape, strides, offset, dtype, index, contiguous=None) -> "TorchMojoTensor":
        shape = tuple(int(s) for s in shape)
        strides = tuple(int(s) for s in strides)
        res = torch.Tensor._make_wrapper_subclass(
            cls,
            shape,
            strides=strides,
            storage_offset=int(offset),
            dtype=dtype,
            layout=torch.strided,
            device=torch.device(_WRAPPER_DEVICE_TYPE, 0),
            requires_grad=False,
        )
        res._holder = holder
        res._ptr = int(ptr)
        res._shape = shape
        res._strides = strides
        res._offset = int(offset)
        res._dtype = dtype
        res._itemsize = torch.empty((), dtype=dtype).element_size()
        res._numel = math.prod(shape)
        res._device_index = int(index)
        res._torch_device = torch.device("mojo", int(index))
        res._is_contiguous = _compute_contiguous(shape, strides) if contiguous is None else contiguous
        return res

    @classmethod
    def _alloc(cls, shape, dtype: torch.dtype, index: int | None = None) -> "TorchMojoTensor":
        """A new contiguous uninitialised tensor (one device allocation)."""
        index = device_module.current_device() if index is None else index
        shape = tuple(int(s) for s in shape)
        itemsize = torch.empty((), dtype=dtype).element_size()
        holder = _alloc_holder(math.prod(shape) * itemsize, index)
        return cls._make(holder, _holder_ptr(holder), shape, _row_major_strides(shape), 0, dtype, index, True)

    @classmethod
    def _alloc_strided(cls, shape, strides, dtype: torch.dtype, index: int | None = None) -> "TorchMojoTensor":
        """A new tensor with the given (non-overlapping) strides, e.g. BTHD-stored BHSD."""
        index = device_module.current_device() if index is None else index
        shape = tuple(int(s) for s in shape)
        strides = tuple(int(s) for s in strides)
        itemsize = torch.empty((), dtype=dtype).element_size()
        extent = 1 + sum((d - 1) * s for d, s in zip(shape, strides)) if math.prod(shape) else 0
        holder = _alloc_holder(extent * itemsize, index)
        return cls._make(holder, _holder_ptr(holder), shape, strides, 0, dtype, index)

    @classmethod
    def _view_of(cls, base: "TorchMojoTensor", shape, strides, offset, contiguous=None) -> "TorchMojoTensor":
        """A zero-copy view sharing base's holder; `offset` is absolute, in elements."""
        ptr = base._ptr + (int(offset) - base._offset) * base._itemsize
        view = cls._make(base._holder, ptr, shape, strides, offset, base._dtype, base._device_index, contiguous)
        if hasattr(base, "_philox"):
            # the (seed, offset) pair an rng_state tensor carries on the host survives detach / alias
            view._philox = base._philox
        return view

    @classmethod
    def _from_cuda(cls, t: torch.Tensor) -> "TorchMojoTensor":
        """Adopt a CUDA tensor's memory without copying (the holder keeps it alive)."""
        if t.device.type != "cuda":
            raise RuntimeError(f"_from_cuda needs a CUDA tensor, got {t.device}")
        t = t.detach()
        return cls._make(t, t.data_ptr(), tuple(t.shape), tuple(t.stride()), 0, t.dtype, t.device.index or 0)

    @classmethod
    def _from_cpu(cls, cpu_tensor: torch.Tensor, index: int | None = None, *, non_blocking: bool = False):
        """H2D: allocate and enqueue a copy from a CPU tensor."""
        t = cpu_tensor.detach()
        if t.device.type != "cpu":
            raise RuntimeError(f"_from_cpu requires a CPU source tensor, got {t.device}")
        out = cls._alloc(tuple(t.shape), t.dtype, index)
        if out._numel:
            out._cuda_view().copy_(t, non_blocking=non_blocking)
        return out

    # ------------------------------------------------------------------ payload access
    def _cuda_view(self) -> torch.Tensor:
        """The same memory as a plain CUDA tensor (for copies and DLPack export)."""
        holder = self._holder
        if holder.dtype == torch.uint8 and holder.dim() == 1:
            nbytes = holder.numel() - holder.numel() % self._itemsize
            typed = holder[:nbytes].view(self._dtype) if nbytes else holder.new_empty((0,), dtype=self._dtype)
            return torch.as_strided(typed, self._shape, self._strides, self._offset)
        # adopted foreign CUDA tensor: offset is relative to its own first element
        flat_extent_ok = holder.dtype == self._dtype
        if not flat_extent_ok:
            raise RuntimeError("adopted holder dtype changed under a view")
        return torch.as_strided(holder, self._shape, self._strides, holder.storage_offset() + self._offset)

    def _to_cpu_tensor(self, *, non_blocking: bool = False) -> torch.Tensor:
        if self._numel == 0:
            return torch.empty(self._shape, dtype=self._dtype)
        src = self._cuda_view()
        if non_blocking:
            dst = pinned_empty(self._shape, self._dtype)
            dst.copy_(src, non_blocking=True)
            return dst
        return src.cpu()

    def _materialize_contiguous(self) -> "TorchMojoTensor":
        out = TorchMojoTensor._alloc(self._shape, self._dtype, self._device_index)
        if self._numel:
            out._cuda_view().copy_(self._cuda_view())
        return out

    def _contig(self) -> "TorchMojoTensor":
        return self if self._is_contiguous else self._materialize_contiguous()

    # ------------------------------------------------------------------ interop
    def __dlpack__(self, *, stream=None, **_unused):
        return self._contig()._cuda_view().__dlpack__()

    def __dlpack_device__(self):
        return self._cuda_view().__dlpack_device__()

    def __reduce_ex__(self, protocol):
        """Pickle as a plain CPU tensor (reference: torch_mojo_tensor.py:572-583)."""
        if hasattr(self, "_holder"):
            return self._to_cpu_tensor().__reduce_ex__(protocol)
        return super().__reduce_ex__(protocol)

    def __repr__(self):
        if hasattr(self, "_holder"):
            return f"TorchMojoTensor({self._to_cpu_tensor()!r}, device='{self.device}')"
        return super().__repr__()

    @property
    def device(self):
        if hasattr(self, "_torch_device"):
            return self._torch_device
        return super().device


def payload(t) -> "TorchMojoTensor | None":
    """The tensor itself if it is a mojo tensor carrying its payload, else None (the
    reference's ``_t`` helper)."""
    if isinstance(t, TorchMojoTensor) and hasattr(t, "_holder"):
        return t
    return None
