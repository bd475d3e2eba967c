"""libswscale through ctypes: the arithmetic of the reference's CPU colour path.

The reference's CPU route converts decoded yuv420p frames to rgb24 inside a libavfilter graph,
i.e. in FFmpeg's libswscale (``src/libspdl/core/detail/ffmpeg/filter_graph.cpp:50-65``, one
filter thread at ``:52``), and then copies them into one contiguous buffer
(``src/libspdl/core/detail/ffmpeg/conversion.cpp:171-216``).  spdl itself cannot be built here,
but a libswscale (FFmpeg 8 ABI) ships inside the opencv wheel; this module drives it directly
for the timed CPU baseline.  TEST/BENCH INFRASTRUCTURE ONLY.
"""

from __future__ import annotations

import ctypes
import glob
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_SWS = None
_AVU = None
SWS_BILINEAR = 2
SWS_ACCURATE_RND = 0x40000
SWS_CS_ITU709, SWS_CS_ITU601 = 1, 5


def _find(name: str) -> str | None:
    try:
        import cv2  # noqa: F401

        base = os.path.join(os.path.dirname(os.path.dirname(cv2.__file__)),
                            "opencv_python_headless.libs")
    except Exception:
        return None
    hits = sorted(glob.glob(os.path.join(base, f"lib{name}-*.so*")))
    return hits[0] if hits else None


def available() -> bool:
    return load() is not None


def load():
    global _SWS, _AVU
    if _SWS is None:
        pa, ps = _find("avutil"), _find("swscale")
        if not pa or not ps:
            return None
        try:
            _AVU = ctypes.CDLL(pa, mode=ctypes.RTLD_GLOBAL)
            _SWS = ctypes.CDLL(ps)
        except OSError:
            return None
        _AVU.av_get_pix_fmt.argtypes = [ctypes.c_char_p]
        _AVU.av_get_pix_fmt.restype = ctypes.c_int
        _SWS.sws_getContext.restype = ctypes.c_void_p
        _SWS.sws_getContext.argtypes = [ctypes.c_int] * 3 + [ctypes.c_int] * 3 + [ctypes.c_int] + \
            [ctypes.c_void_p] * 3
        _SWS.sws_getCoefficients.restype = ctypes.POINTER(ctypes.c_int)
        _SWS.sws_getCoefficients.argtypes = [ctypes.c_int]
        _SWS.sws_setColorspaceDetails.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int),
                                                  ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                                  ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                  ctypes.c_int]
        _SWS.sws_scale.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                   ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int,
                                   ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_int)]
        _SWS.sws_scale.restype = ctypes.c_int
        _SWS.sws_freeContext.argtypes = [ctypes.c_void_p]
    return _SWS


class I420ToRGB:
    """One converter (one ``SwsContext``): yuv420p ``w x h`` -> rgb24, limited (or, with
    ``full_range``, full) -> full range."""

    def __init__(self, w: int, h: int, colorspace: int = SWS_CS_ITU709, dst_fmt: str = "rgb24",
                 full_range: bool = False):
        sws = load()
        if sws is None:
            raise RuntimeError("libswscale is not available on this machine")
        src = _AVU.av_get_pix_fmt(b"yuv420p")
        dst = _AVU.av_get_pix_fmt(dst_fmt.encode())
        self.w, self.h = w, h
        self.ctx = sws.sws_getContext(w, h, src, w, h, dst, SWS_BILINEAR, None, None, None)
        if not self.ctx:
            raise RuntimeError("sws_getContext failed")
        coefs = sws.sws_getCoefficients(colorspace)
        sws.sws_setColorspaceDetails(self.ctx, coefs, int(full_range), coefs, 1, 0, 1 << 16, 1 << 16)

    def __call__(self, i420: np.ndarray, out: np.ndarray) -> None:
        """``i420``: ``[h*3/2, w]`` u8 (Y rows, U block, V block); ``out``: ``[h, w, 3]`` u8."""
        w, h = self.w, self.h
        base = i420.ctypes.data
        src = (ctypes.c_void_p * 4)(base, base + w * h, base + w * h + (w // 2) * (h // 2), None)
        stride = (ctypes.c_int * 4)(w, w // 2, w // 2, 0)
        dst = (ctypes.c_void_p * 4)(out.ctypes.data, None, None, None)
        dstride = (ctypes.c_int * 4)(3 * w, 0, 0, 0)
        rows = load().sws_scale(self.ctx, src, stride, 0, h, dst, dstride)
        if rows != h:
            raise RuntimeError(f"sws_scale converted {rows} of {h} rows")

    def __del__(self):
        if getattr(self, "ctx", None) and _SWS is not None:
            _SWS.sws_freeContext(self.ctx)
            self.ctx = None


class BatchConverter:
    """Converts ``[N, h*3/2, w]`` I420 batches into one contiguous ``[N, h, w, 3]`` buffer with a
    pool of ``threads`` workers, one ``SwsContext`` each (ctypes drops the GIL in ``sws_scale``)."""

    def __init__(self, w: int, h: int, threads: int, colorspace: int = SWS_CS_ITU709):
        self.threads = max(1, int(threads))
        self.conv = [I420ToRGB(w, h, colorspace) for _ in range(self.threads)]
        self.pool = ThreadPoolExecutor(self.threads)

    def __call__(self, batch: np.ndarray, out: np.ndarray) -> None:
        n = batch.shape[0]

        def work(t: int) -> None:
            for i in range(t, n, self.threads):
                self.conv[t](batch[i], out[i])

        list(self.pool.map(work, range(min(self.threads, n))))

    def close(self) -> None:
        self.pool.shutdown()
