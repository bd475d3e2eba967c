"""``transfer_tensor``: move CPU tensors to the GPU on a dedicated per-thread stream.

Mirrors ``spdl.io.transfer_tensor`` (``src/spdl/io/_transfer.py:33-177``): containers are
walked recursively; each CPU tensor is pinned and copied with ``non_blocking=True`` on a stream
owned by the calling thread on ``cuda:{LOCAL_RANK}``; the stream is synchronised before
returning; the last ``num_caches`` batches are kept alive so the caching allocator cannot hand
their memory to another stream while a consumer still reads it.
"""

from __future__ import annotations

import dataclasses
import os
import threading
from functools import partial
from typing import Any, Callable, TypeVar

T = TypeVar("T")

__all__ = ["transfer_tensor"]


def _recursive_apply(fn: Callable[[Any], Any], obj: Any) -> Any:
    if isinstance(obj, tuple) and hasattr(obj, "_fields"):  # namedtuple
        return type(obj)(*(_recursive_apply(fn, v) for v in obj))
    if isinstance(obj, (list, tuple)):
        return type(obj)(_recursive_apply(fn, v) for v in obj)
    if isinstance(obj, dict):
        return type(obj)((k, _recursive_apply(fn, v)) for k, v in obj.items())
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        init = {f.name: _recursive_apply(fn, getattr(obj, f.name))
                for f in dataclasses.fields(obj) if f.init}
        new = type(obj)(**init)
        for f in dataclasses.fields(obj):
            if not f.init:
                object.__setattr__(new, f.name, _recursive_apply(fn, getattr(obj, f.name)))
        return new
    return fn(obj)


def _transfer(obj: Any, device: Any, pinned_cache: set) -> Any:
    import torch

    if isinstance(obj, torch.Tensor) and obj.is_cpu:
        pinned = obj.pin_memory()
        pinned_cache.add(pinned)
        obj = pinned.to(device, non_blocking=True)
    return obj


class _DataTransfer:
    def __init__(self, device: Any, num_caches: int) -> None:
        import torch

        self._device = device
        self._stream = torch.cuda.Stream(device)
        self._batch_cache: list[Any] = [None for _ in range(num_caches)]

    def __call__(self, batch: T) -> T:
        import torch

        pinned_cache: set = set()
        fn = partial(_transfer, device=self._device, pinned_cache=pinned_cache)
        with torch.cuda.stream(self._stream):
            batch = _recursive_apply(fn, batch)
        self._stream.synchronize()
        self._batch_cache.append(batch)
        self._batch_cache.pop(0)
        return batch


_THREAD_LOCAL = threading.local()


def _get_transfer_func(num_caches: int) -> _DataTransfer:
    import torch

    if not hasattr(_THREAD_LOCAL, "transfer"):
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if local_rank >= torch.cuda.device_count():
            raise RuntimeError("The local rank is larger than the number of available GPUs.")
        _THREAD_LOCAL.transfer = _DataTransfer(torch.device(f"cuda:{local_rank}"), num_caches)
    return _THREAD_LOCAL.transfer


def transfer_tensor(batch: T, /, *, num_caches: int = 4) -> T:
    """Transfer the CPU tensors inside ``batch`` (tensor, list, tuple, dict or dataclass) to the
    GPU chosen by ``LOCAL_RANK`` on a stream private to the calling thread."""
    return _get_transfer_func(num_caches)(batch)
