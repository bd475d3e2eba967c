"""Build-feature probes, as ``spdl.io.utils`` (``src/spdl/io/utils/_build.py``)."""

from ... import _lib
from ._tracing import call_stats, reset_call_stats, trace_event, tracing

__all__ = ["built_with_cuda", "built_with_nvcodec", "built_with_nvjpeg", "call_stats",
           "reset_call_stats", "trace_event", "tracing"]


def built_with_cuda() -> bool:
    """True when ``libb2frames.so`` is present and loads."""
    try:
        _lib.lib()
        return True
    except (RuntimeError, OSError):
        return False


def built_with_nvcodec() -> bool:
    """Always False: the video decoder engine is not part of this package."""
    return False


def built_with_nvjpeg() -> bool:
    """Always False: JPEG decoding is not part of this package."""
    return False
