"""The ``torch.mojo`` backend module.

torch looks functions up on this module by name (``device_count``, ``current_device``,
``set_device``, ``device``, ``synchronize``, ``manual_seed_all``, ``get_rng_state`` ...: the
contract of ``torch.utils.backend_registration``), so the names match the reference's module
(torch_mojo_backend/mojo_device/torch_mojo_device_module.py:15-199); what is behind them is this
package's: ``mojo:i`` is CUDA device ``i`` of the process (one process per GPU when scaling out),
``synchronize`` also surfaces a kernel that gave up on an internal wait, and the per-device
Philox generator state feeds the dropout mask of the flash-attention kernels.
"""

from __future__ import annotations

import threading

import torch

_current = 0


def _is_in_bad_fork() -> bool:
    return False


def is_available() -> bool:
    return torch.cuda.is_available()


def is_initialized() -> bool:
    return True


def device_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def current_device() -> int:
    return _current


def _checked_index(index: int) -> int:
    count = device_count()
    if index < 0 or (count and index >= count):
        raise ValueError(f"Invalid device index {index}")
    return index


def set_device(device_idx: int) -> None:
    global _current
    _current = _checked_index(int(device_idx))


def _index_of(device) -> int:
    """Device ordinal of an int / str / torch.device / None (None and index-less: the current one)."""
    if device is None:
        return _current
    if isinstance(device, int):
        return device
    dev = torch.device(device)
    if dev.type != "mojo":
        raise ValueError(f"expected a mojo device, got {dev}")
    return _current if dev.index is None else dev.index


class device:
    """``with torch.mojo.device(i):`` — makes ``mojo:i`` current inside the block
    (``torch.serialization`` relies on it for ``map_location="mojo"``)."""

    def __init__(self, device) -> None:
        self._target = None if device is None else (device if isinstance(device, int) else torch.device(device).index)

    def __enter__(self) -> None:
        self._saved = _current
        if self._target is not None and self._target >= 0:
            set_device(self._target)

    def __exit__(self, *exc) -> bool:
        if _current != self._saved:
            set_device(self._saved)
        return False


def synchronize(device=None) -> None:
    """Wait for every kernel and copy issued on the device, then raise if one of the
    flash-attention kernels reported that it gave up on an internal wait."""
    index = _index_of(device)
    torch.cuda.synchronize(index)
    from . import flash_ops

    flash_ops.check_status(index)


def get_amp_supported_dtype():
    return [torch.float16, torch.bfloat16]


# ---------------------------------------------------------------------------- Philox generator state
# Per device: a 64-bit seed and a 64-bit counter.  An op that needs random bits reserves an
# interval of the counter (``_reserve_philox_state``) and keys its Philox calls with
# (seed, reserved offset + its own index), so two calls never draw the same numbers and a
# restored state replays them.  The 16-byte state tensor is seed then counter, little-endian,
# the same encoding the reference uses (torch_mojo_device_module.py:121-156).
_U64 = (1 << 64) - 1


class _Generators:
    def __init__(self) -> None:
        self.lock = threading.Lock()
        self.default_seed = 67_280_421_310_721   # torch's default CUDA generator seed
        self.state: dict[int, list[int]] = {}    # index -> [seed, counter]

    def of(self, index: int) -> list[int]:
        return self.state.setdefault(index, [self.default_seed, 0])


_gen = _Generators()


def manual_seed_all(seed) -> None:
    """Every device restarts from `seed` with its counter at zero."""
    value = int(seed)
    if not -(1 << 63) <= value <= _U64:
        raise ValueError("Overflow when unpacking long long")
    with _gen.lock:
        _gen.default_seed = value & _U64
        _gen.state.clear()


def manual_seed(seed) -> None:
    manual_seed_all(seed)


def get_rng_state(device=None) -> torch.Tensor:
    index = _checked_index(_index_of(device))
    with _gen.lock:
        seed, counter = _gen.of(index)
    raw = seed.to_bytes(8, "little") + counter.to_bytes(8, "little")
    return torch.frombuffer(bytearray(raw), dtype=torch.uint8).clone()


def set_rng_state(new_state, device=None) -> None:
    if not isinstance(new_state, torch.Tensor):
        raise TypeError("Mojo RNG state must be a torch.Tensor")
    flat = new_state.detach().cpu().contiguous().reshape(-1)
    if flat.dtype != torch.uint8 or flat.numel() != 16:
        raise ValueError("Mojo RNG state must be a 16-element uint8 tensor")
    raw = bytes(flat.tolist())
    index = _checked_index(_index_of(device))
    with _gen.lock:
        _gen.state[index] = [int.from_bytes(raw[:8], "little"), int.from_bytes(raw[8:], "little")]


def _reserve_philox_state(device, counter_increment: int) -> tuple[int, int]:
    """Take `counter_increment` values off the device's counter; returns (seed, first value)."""
    if type(counter_increment) is not int or counter_increment < 0:
        raise ValueError("Philox counter increment must be a nonnegative integer")
    index = _checked_index(_index_of(device))
    with _gen.lock:
        entry = _gen.of(index)
        seed, first = entry
        if first + counter_increment > _U64:
            raise OverflowError("Philox counter reservation would wrap uint64")
        entry[1] = first + counter_increment
    return seed, first
