"""The ``torch.mojo`` backend module: device bookkeeping, synchronisation and Philox state.

Same surface as the reference's device module
(torch_mojo_backend/mojo_device/torch_mojo_device_module.py:15-199): ``device_count``,
``current_device``/``set_device``, the ``device`` context manager, ``synchronize`` and the
per-device ``(seed, counter)`` RNG state with ``_reserve_philox_state``.  Here ``mojo:i`` is
CUDA device ``i`` of this process (one process per GPU when scaling out).
"""

from __future__ import annotations

import threading

import torch

_current_device = 0
_UINT64_MASK = (1 << 64) - 1
_DEFAULT_RNG_SEED = 67_280_421_310_721
_rng_default_seed = _DEFAULT_RNG_SEED
_rng_states: dict[int, tuple[int, int]] = {}
_rng_lock = threading.Lock()


def _is_in_bad_fork() -> bool:
    return False


def is_available() -> bool:
    return torch.cuda.is_available()


def is_initialized() -> bool:
    return True


def device_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def current_device() -> int:
    return _current_device


def set_device(device_idx: int) -> None:
    global _current_device
    count = device_count()
    if device_idx < 0 or (count and device_idx >= count):
        raise ValueError(f"Invalid device index {device_idx}")
    _current_device = device_idx


class device:
    """Context manager that swaps the current mojo device (``torch.cuda.device`` analogue;
    ``torch.serialization`` needs it for ``map_location="mojo"``)."""

    def __init__(self, device: "int | str | torch.device | None") -> None:
        if device is None:
            self.idx = -1
        elif isinstance(device, int):
            self.idx = device
        else:
            index = torch.device(device).index
            self.idx = -1 if index is None else index

    def __enter__(self) -> None:
        self.prev_idx = _current_device
        if self.idx >= 0 and self.idx != _current_device:
            set_device(self.idx)

    def __exit__(self, *exc_info: object) -> bool:
        if self.idx >= 0 and self.prev_idx != _current_device:
            set_device(self.prev_idx)
        return False


def _resolve_index(device: "int | str | torch.device | None") -> int:
    if device is None:
        return _current_device
    if isinstance(device, int):
        return device
    torch_device = torch.device(device)
    if torch_device.type != "mojo":
        raise ValueError(f"expected a mojo device, got {torch_device}")
    return _current_device if torch_device.index is None else torch_device.index


def synchronize(device: "int | str | torch.device | None" = None) -> None:
    """Wait for every kernel and copy issued on the device's stream."""
    torch.cuda.synchronize(_resolve_index(device))


# ---------------------------------------------------------------------------- RNG state
def _normalize_rng_seed(seed) -> int:
    value = int(seed)
    if value < -(1 << 63) or value > _UINT64_MASK:
        raise ValueError("Overflow when unpacking long long")
    return value & _UINT64_MASK


def _rng_device_index(device=None) -> int:
    index = _resolve_index(device)
    count = device_count()
    if index < 0 or (count and index >= count):
        raise ValueError(f"Invalid device index {index}")
    return index


def manual_seed_all(seed) -> None:
    """Reset every device to the same Philox seed and counter zero."""
    global _rng_default_seed
    normalized = _normalize_rng_seed(seed)
    with _rng_lock:
        _rng_default_seed = normalized
        _rng_states.clear()


def manual_seed(seed) -> None:
    manual_seed_all(seed)


def get_rng_state(device=None) -> torch.Tensor:
    """The device's exact ``(seed, counter)`` as 16 little-endian bytes."""
    index = _rng_device_index(device)
    with _rng_lock:
        seed, counter = _rng_states.setdefault(index, (_rng_default_seed, 0))
    encoded = seed.to_bytes(8, "little") + counter.to_bytes(8, "little")
    return torch.tensor(list(encoded), dtype=torch.uint8)


def set_rng_state(new_state, device=None) -> None:
    if not isinstance(new_state, torch.Tensor):
        raise TypeError("Mojo RNG state must be a torch.Tensor")
    state = new_state.detach().cpu().contiguous()
    if state.dtype != torch.uint8 or state.numel() != 16:
        raise ValueError("Mojo RNG state must be a 16-element uint8 tensor")
    encoded = bytes(state.reshape(-1).tolist())
    index = _rng_device_index(device)
    with _rng_lock:
        _rng_states[index] = (int.from_bytes(encoded[:8], "little"), int.from_bytes(encoded[8:], "little"))


def _reserve_philox_state(device, counter_increment: int) -> tuple[int, int]:
    """Atomically reserve a Philox counter interval; returns (seed, base counter)."""
    if type(counter_increment) is not int or counter_increment < 0:
        raise ValueError("Philox counter increment must be a nonnegative integer")
    index = _rng_device_index(device)
    with _rng_lock:
        seed, counter = _rng_states.setdefault(index, (_rng_default_seed, 0))
        if counter_increment > _UINT64_MASK - counter:
            raise OverflowError("Philox counter reservation would wrap uint64")
        _rng_states[index] = (seed, counter + counter_increment)
    return seed, counter


def get_amp_supported_dtype():
    return [torch.float16, torch.bfloat16]
