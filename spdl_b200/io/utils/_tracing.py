"""Tracing and per-call counters for the frame path.

The reference wraps its launchers in ``TRACE_EVENT`` (Perfetto, or torch profiler ranges with
``SPDL_USE_TORCH_RECORD_FUNCTION``; ``src/libspdl/core/detail/tracing.h:11-73``,
``src/libspdl/cuda/detail/color_conversion.cu:167,187``) and exposes
``spdl.io.utils.tracing()/trace_event()`` (``src/spdl/io/utils/_tracing.py:23-107``).  Here the
events are NVTX ranges, visible to any CUDA profiler, switched on with ``tracing()`` or the
environment variable ``SPDL_B200_TRACE=1``; the counters are always on (a few dict updates per
call).
"""

from __future__ import annotations

import os
import threading
from contextlib import contextmanager

__all__ = ["tracing", "trace_event", "call_stats", "reset_call_stats"]

_enabled = os.environ.get("SPDL_B200_TRACE", "0") == "1"
_lock = threading.Lock()
_stats: dict[str, dict[str, int]] = {}


def _nvtx():
    import torch

    return torch.cuda.nvtx


@contextmanager
def tracing(enable: bool = True):
    """Turn NVTX ranges around the library calls on (or off) inside the block."""
    global _enabled
    prev, _enabled = _enabled, bool(enable)
    try:
        yield
    finally:
        _enabled = prev


@contextmanager
def trace_event(name: str):
    """An NVTX range named ``name`` when tracing is on; nothing otherwise."""
    if not _enabled:
        yield
        return
    nvtx = _nvtx()
    nvtx.range_push(name)
    try:
        yield
    finally:
        nvtx.range_pop()


def record(name: str, units: int, bytes_in: int, bytes_out: int) -> None:
    """Count one call of ``name``: frames or images processed and algorithmic bytes."""
    with _lock:
        s = _stats.setdefault(name, {"calls": 0, "units": 0, "bytes_in": 0, "bytes_out": 0})
        s["calls"] += 1
        s["units"] += int(units)
        s["bytes_in"] += int(bytes_in)
        s["bytes_out"] += int(bytes_out)


def call_stats() -> dict[str, dict[str, int]]:
    """Per-entry-point totals since the last reset: calls, units, bytes in, bytes out."""
    with _lock:
        return {k: dict(v) for k, v in _stats.items()}


def reset_call_stats() -> None:
    with _lock:
        _stats.clear()
