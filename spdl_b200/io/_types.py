"""Value types at the boundary: configuration, storage and buffers.

These mirror the objects the reference's extension module hands to Python:

* ``CUDAConfig``   -- ``src/libspdl/cuda/types.h:32-39``, built by ``cuda_config``
  (``src/spdl/io/_config.py:115-178``).
* ``CPUStorage``   -- ``src/libspdl/core/storage.h`` / pinned variant
  ``src/libspdl/cuda/storage.cpp:22-38``, built by ``cpu_storage``
  (``src/spdl/io/_config.py:296-328``).
* ``CPUBuffer``    -- ``src/libspdl/core/buffer.h``; array interface as in
  ``src/spdl/io/lib/core/buffer.cpp:44-55``.
* ``CUDABuffer``   -- ``src/libspdl/cuda/buffer.h:28-77``; ``__cuda_array_interface__`` as in
  ``src/spdl/io/lib/cuda/buffer.cpp:55-65``.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Any, Callable, Sequence

import numpy as np

from .. import _lib

__all__ = ["CUDAConfig", "CPUStorage", "CPUBuffer", "CUDABuffer", "cuda_config", "cpu_storage"]

Allocator = tuple[Callable[[int, int, int], int], Callable[[int], None]]


@dataclass(frozen=True)
class CUDAConfig:
    """Target device, stream and (optionally) allocator of a CUDA operation."""

    device_index: int
    stream: int = 0x2  # cudaStreamPerThread
    allocator: Allocator | None = None


def cuda_config(device_index: int, stream: int = 0x2,
                allocator: Allocator | None = None) -> CUDAConfig:
    """Specify the CUDA device and memory management.

    Same signature and defaults as ``spdl.io.cuda_config``: ``stream`` is the ``uintptr_t`` of a
    CUDA stream (``0x2`` = per-thread default stream, ``0`` = legacy default stream);
    ``allocator`` is a pair ``(alloc(size, device, stream) -> address, free(address))`` such as
    ``torch.cuda.caching_allocator_alloc`` / ``torch.cuda.caching_allocator_delete``.
    """
    if not isinstance(device_index, int) or isinstance(device_index, bool):
        raise TypeError("device_index must be an int")
    if not isinstance(stream, int):
        raise TypeError("stream must be an int (uintptr_t of a CUDA stream)")
    if allocator is not None:
        if not (isinstance(allocator, (tuple, list)) and len(allocator) == 2
                and all(callable(f) for f in allocator)):
            raise TypeError("allocator must be a pair of callables (alloc, free)")
        allocator = (allocator[0], allocator[1])
    return CUDAConfig(device_index, stream, allocator)


class CPUStorage:
    """A block of host memory, optionally page-locked."""

    def __init__(self, size: int, pin_memory: bool = True) -> None:
        if isinstance(size, bool) or not isinstance(size, int):
            raise TypeError("size must be an int")
        if size < 0:
            # the reference takes size_t: a negative value fails argument conversion
            raise TypeError("size must be non-negative")
        if size == 0:
            raise RuntimeError("`size` must be greater than 0.")
        self.size = size
        self.pinned = bool(pin_memory)
        self._ptr: int | None = None
        self._np: np.ndarray | None = None
        if self.pinned:
            p = ctypes.c_void_p()
            _lib.check(_lib.lib().b2_alloc_pinned(ctypes.byref(p), size))
            self._ptr = p.value
        else:
            self._np = np.empty(size, np.uint8)
            self._ptr = self._np.ctypes.data

    @property
    def data_ptr(self) -> int:
        assert self._ptr is not None
        return self._ptr

    def is_pinned(self) -> bool:
        return self.pinned

    def as_array(self) -> np.ndarray:
        if self._np is not None:
            return self._np
        buf = (ctypes.c_uint8 * self.size).from_address(self.data_ptr)
        arr = np.frombuffer(buf, np.uint8)
        arr.flags.writeable = True
        return arr

    def __del__(self) -> None:
        if getattr(self, "pinned", False) and getattr(self, "_ptr", None):
            try:
                _lib.lib().b2_free_pinned(self._ptr)
            except Exception:  # interpreter shutdown
                pass
            self._ptr = None


def cpu_storage(size: int, pin_memory: bool = True) -> CPUStorage:
    """Allocate a block of host memory (page-locked by default) for ``convert_frames``."""
    return CPUStorage(size, pin_memory)


_TYPESTR = {"u": "u", "i": "i", "f": "f"}


def _typestr(elem_class: str, depth: int) -> str:
    if elem_class not in _TYPESTR:
        raise RuntimeError(f"Unsupported class {elem_class}.")
    return f"|{_TYPESTR[elem_class]}{depth}"


class CPUBuffer:
    """Contiguous host array: storage + shape + element class/depth."""

    def __init__(self, shape: Sequence[int], elem_class: str = "u", depth: int = 1,
                 storage: CPUStorage | np.ndarray | None = None) -> None:
        self.shape = tuple(int(s) for s in shape)
        self.elem_class, self.depth = elem_class, int(depth)
        nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.depth
        if storage is None:
            storage = CPUStorage(max(nbytes, 1), pin_memory=False)
        elif isinstance(storage, CPUStorage) and storage.size < nbytes:
            # src/libspdl/core/buffer.cpp:56-64
            raise RuntimeError(
                f"The provided storage does not have enough capacity. ({storage.size} < {nbytes})")
        self.storage = storage
        self.nbytes = nbytes

    @property
    def data_ptr(self) -> int:
        s = self.storage
        return s.data_ptr if isinstance(s, CPUStorage) else s.ctypes.data

    def is_pinned(self) -> bool:
        return isinstance(self.storage, CPUStorage) and self.storage.is_pinned()

    @property
    def __array_interface__(self) -> dict[str, Any]:
        return {"version": 3, "shape": self.shape,
                "typestr": _typestr(self.elem_class, self.depth),
                "data": (self.data_ptr, False), "strides": None}


class CUDABuffer:
    """Owning device array exposing ``__cuda_array_interface__`` (version 2)."""

    def __init__(self, ptr: int, shape: Sequence[int], device_index: int, stream: int,
                 elem_class: str = "u", depth: int = 1,
                 deleter: Callable[[int], None] | None = None, owner: Any = None) -> None:
        self._ptr = int(ptr)
        self.shape = tuple(int(s) for s in shape)
        self._device_index = int(device_index)
        self._stream = int(stream)
        self.elem_class, self.depth = elem_class, int(depth)
        self._deleter = deleter
        self._owner = owner  # anything that must outlive this buffer

    @property
    def device_index(self) -> int:
        return self._device_index

    @property
    def data_ptr(self) -> int:
        return self._ptr

    @property
    def nbytes(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) * self.depth

    @property
    def __cuda_array_interface__(self) -> dict[str, Any]:
        return {"version": 2, "shape": self.shape,
                "typestr": _typestr(self.elem_class, self.depth),
                "data": (self._ptr, False), "strides": None, "stream": self._stream}

    def __del__(self) -> None:
        d, self._deleter = getattr(self, "_deleter", None), None
        if d is not None and getattr(self, "_ptr", 0):
            try:
                d(self._ptr)
            except Exception:
                pass


_PSEUDO_STREAMS = (0, 1, 2)  # default, legacy and per-thread stream handles


def _default_allocator(device: int, stream: int) -> Allocator:
    """Allocator used when the config carries none.

    The reference calls ``cudaMalloc``/``cudaFree`` per buffer
    (``src/libspdl/cuda/storage.cpp:44-58``); ``cudaFree`` waits for the device, which is what
    makes it safe to free a buffer whose kernel is still queued.  That pair is kept for the
    pseudo stream handles ``0``, ``1`` and ``2``: they name a different real stream in every
    thread, so a caching allocator keyed by the handle could hand a block freed in one thread to
    another thread's stream while the first thread's kernel still runs
    (``docs/source/io/pytorch_cuda_race_condition.rst`` of the reference describes that race).
    For a real stream handle, and when torch has initialised CUDA, torch's caching allocator is
    used instead, so a steady-state call allocates without touching the driver.
    """
    if stream not in _PSEUDO_STREAMS:
        try:
            import torch

            if torch.cuda.is_available():
                return (torch.cuda.caching_allocator_alloc, torch.cuda.caching_allocator_delete)
        except Exception:
            pass

    def alloc(size: int, dev: int, stream: int) -> int:
        p = ctypes.c_void_p()
        _lib.check(_lib.lib().b2_device_alloc(ctypes.byref(p), size, dev))
        return int(p.value or 0)

    def free(ptr: int) -> None:
        _lib.lib().b2_device_free(ptr, device)

    return alloc, free


def cuda_buffer(shape: Sequence[int], cfg: CUDAConfig, elem_class: str = "u",
                depth: int = 1) -> CUDABuffer:
    """Allocate an owning device buffer through ``cfg.allocator`` (or the default).

    Follows ``cuda_buffer`` / ``CUDAStorage`` (``src/libspdl/cuda/buffer.cpp:41-52``,
    ``src/libspdl/cuda/storage.cpp:60-101``): zero-size allocations are an error.
    """
    shape = tuple(int(s) for s in shape)
    nbytes = int(np.prod(shape, dtype=np.int64)) * depth
    if nbytes == 0:
        raise RuntimeError("`size` must be greater than 0.")
    alloc, free = cfg.allocator if cfg.allocator is not None else _default_allocator(
        cfg.device_index, cfg.stream)
    ptr = int(alloc(nbytes, cfg.device_index, cfg.stream))
    if ptr == 0:
        raise RuntimeError("Failed to allocate CUDA memory")
    return CUDABuffer(ptr, shape, cfg.device_index, cfg.stream, elem_class, depth, deleter=free)
