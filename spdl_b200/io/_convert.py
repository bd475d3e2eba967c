"""Zero-copy casts of buffers to array libraries.

Mirrors ``spdl.io.to_numpy`` / ``spdl.io.to_torch`` (``src/spdl/io/_convert.py:100-153``).
"""

from __future__ import annotations

from typing import Any

import numpy as np

__all__ = ["to_numpy", "to_torch"]


def to_numpy(buffer: Any) -> np.ndarray:
    """View a host buffer (``__array_interface__``) as a NumPy array without copying."""
    if not hasattr(buffer, "__array_interface__"):
        raise RuntimeError("The given object does not have `__array_interface__` attribute.")
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
            raise ValueError("0-element array is not supported.")
        data_ptr = iface["data"][0]
        tensor = torch.as_tensor(buffer, device=f"cuda:{buffer.device_index}")
        if tensor.data_ptr() == 0:
            raise RuntimeError(
                "Failed to convert to PyTorch Tensor. "
                f"src: {data_ptr}, dst: {tensor.data_ptr()}, device: {buffer.device_index}")
        if tensor.data_ptr() != data_ptr:
            raise RuntimeError(
                "[INTERNAL ERROR] Failed to perform zero-copy conversion to PyTorch Tensor. "
                f"src: {data_ptr}, dst: {tensor.data_ptr()}, device: {buffer.device_index}")
    else:
        tensor = torch.as_tensor(to_numpy(buffer))
    if dtype is not None and tensor.dtype != dtype:
        tensor = tensor.view(dtype)
    return tensor
