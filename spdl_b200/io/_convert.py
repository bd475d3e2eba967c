"""Zero-copy casts of buffers to array libraries.

Mirrors ``spdl.io.to_numpy`` / ``to_torch`` / ``to_numba`` / ``to_jax`` and the two protocol
classes of ``src/spdl/io/_convert.py:28-200``.
"""

from __future__ import annotations

from typing import Any, Protocol, runtime_checkable

import numpy as np

__all__ = ["to_numpy", "to_torch", "to_numba", "to_jax", "ArrayInterface", "CUDAArrayInterface"]


@runtime_checkable
class ArrayInterface(Protocol):
    """Objects that expose host memory through ``__array_interface__`` (NumPy's protocol)."""

    @property
    def __array_interface__(self) -> dict[str, Any]: ...


@runtime_checkable
class CUDAArrayInterface(Protocol):
    """Objects that expose device memory through ``__cuda_array_interface__``."""

    @property
    def __cuda_array_interface__(self) -> dict[str, Any]: ...


def to_numpy(buffer: Any) -> np.ndarray:
    """View a host buffer (``__array_interface__``) as a NumPy array without copying."""
    if not hasattr(buffer, "__array_interface__"):
        raise RuntimeError(f"{type(buffer).__name__} does not expose `__array_interface__`.")
    return np.array(buffer, copy=False)


def to_torch(buffer: Any, dtype: Any = None):
    """View a buffer as a PyTorch tensor without copying.

    CUDA buffers go through ``__cuda_array_interface__`` and the tensor's ``data_ptr`` is checked
    against the buffer's pointer; 0-element arrays raise ``ValueError``.  ``dtype`` optionally
    reinterprets the element type (e.g. ``torch.bfloat16`` for 2-byte outputs).
    """
    import torch

    iface = getattr(buffer, "__cuda_array_interface__", None)
    if iface is not None:
        if any(s == 0 for s in iface.get("shape", [])):
            raise ValueError("An array without elements cannot be wrapped.")
        data_ptr = iface["data"][0]
        tensor = torch.as_tensor(buffer, device=f"cuda:{buffer.device_index}")
        if tensor.data_ptr() != data_ptr:
            # torch made a copy (or produced nothing): the result would not alias the buffer
            raise RuntimeError(
                f"PyTorch did not wrap the buffer in place: buffer at {data_ptr:#x}, tensor at "
                f"{tensor.data_ptr():#x} (device {buffer.device_index}).")
    else:
        tensor = torch.as_tensor(to_numpy(buffer))
    if dtype is not None and tensor.dtype != dtype:
        tensor = tensor.view(dtype)
    return tensor


def to_numba(buffer: Any):
    """A Numba ``DeviceNDArray`` over a CUDA buffer, or a NumPy array over a host buffer, without
    copying (``src/spdl/io/_convert.py:156-173``).  Numba is imported on first use."""
    if hasattr(buffer, "__cuda_array_interface__"):
        from numba import cuda  # raises ImportError where Numba is not installed

        return cuda.as_cuda_array(buffer)
    return to_numpy(buffer)


def to_jax(buffer: Any):
    """A JAX array over a host buffer (``src/spdl/io/_convert.py:176-186``).  JAX is imported on
    first use."""
    import jax

    return jax.numpy.array(to_numpy(buffer), copy=False)
