"""ctypes binding of ``libb2frames.so`` (declared in ``include/b2frames.h``).

The library is the only compute path of this package.  If it is missing the import of any
function here raises; nothing falls back to CPU or to another library.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t,
                    c_uint32, c_uint64, c_void_p)
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libb2frames.so"

# enums of include/b2frames.h
NV12, I420 = 0, 1
NCHW, NHWC = 0, 1
U8, F32, BF16 = 0, 1, 2
RGB, BGR = 0, 1
ARITH_REFERENCE, ARITH_SWSCALE = 0, 1
STATUS_IMAGE_TOO_WIDE, STATUS_WAIT_EXPIRED, STATUS_BAD_GEOMETRY = 1, 2, 4
DEBUG_EXPIRE_WAIT = 1

#: every symbol include/b2frames.h declares
EXPORTS = (
    "b2_last_error", "b2_abi_version", "b2_init", "b2_device_count", "b2_stream_synchronize",
    "b2_nv12_to_planar_rgb", "b2_nv12_to_planar_bgr", "b2_convert_dense", "b2_convert_resize",
    "b2_touched_rows", "b2_copy_rows", "b2_copy_host", "b2_pack_host", "b2_gather_surfaces", "b2_transfer_h2d",
    "b2_transfer_h2d_async", "b2_transfer_h2d_staged", "b2_transfer_d2h", "b2_transfer_d2h_staged",
    "b2_alloc_pinned", "b2_free_pinned", "b2_device_alloc", "b2_device_free", "b2_frame_checksum",
)


class DenseArgs(Structure):
    _fields_ = [
        ("struct_size", c_uint32), ("device", c_int32),
        ("y", c_void_p), ("u", c_void_p), ("v", c_void_p),
        ("y_table", c_void_p), ("u_table", c_void_p), ("v_table", c_void_p),
        ("y_pitch", c_int64), ("uv_pitch", c_int64),
        ("y_frame_stride", c_int64), ("uv_frame_stride", c_int64),
        ("src_format", c_int32), ("width", c_int32), ("height", c_int32), ("num_frames", c_int32),
        ("matrix_coeff", c_int32), ("full_range", c_int32),
        ("dst", c_void_p), ("dst_frame_stride", c_int64),
        ("layout", c_int32), ("dtype", c_int32), ("order", c_int32),
        ("scale", c_float * 3), ("bias", c_float * 3),
        ("reserved0", c_int32), ("arith", c_int32), ("reserved1", c_int32),
    ]


class ImageDesc(Structure):
    _fields_ = [
        ("y_off", c_uint64), ("u_off", c_uint64), ("v_off", c_uint64),
        ("y_pitch", c_int32), ("uv_pitch", c_int32), ("src_w", c_int32), ("src_h", c_int32),
        ("crop_x", c_int32), ("crop_y", c_int32), ("scale_x", c_float), ("scale_y", c_float),
        ("resized_w", c_int32), ("resized_h", c_int32),
    ]


class ResizeArgs(Structure):
    _fields_ = [
        ("struct_size", c_uint32), ("device", c_int32),
        ("base", c_void_p), ("descs", c_void_p),
        ("num_images", c_int32), ("src_format", c_int32),
        ("out_w", c_int32), ("out_h", c_int32),
        ("matrix_coeff", c_int32), ("full_range", c_int32),
        ("layout", c_int32), ("dtype", c_int32), ("order", c_int32),
        ("max_src_w", c_int32),
        ("dst", c_void_p), ("dst_image_stride", c_int64),
        ("scale", c_float * 3), ("bias", c_float * 3),
        ("arith", c_int32), ("frames_per_group", c_int32),
        ("dst_plane_stride", c_int64), ("dst_group_stride", c_int64),
        ("pad_value", c_float * 3), ("debug_flags", c_int32),
        ("status", c_void_p),
        ("luma_row_map", c_void_p), ("chroma_row_map", c_void_p),
    ]


_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


def _declare(lib: ctypes.CDLL) -> None:
    lib.b2_last_error.restype = c_char_p
    lib.b2_last_error.argtypes = []
    lib.b2_abi_version.restype = c_int
    lib.b2_init.argtypes = [c_int]
    lib.b2_device_count.argtypes = [POINTER(c_int)]
    lib.b2_stream_synchronize.argtypes = [c_int, c_void_p]
    planar = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int]
    lib.b2_nv12_to_planar_rgb.argtypes = planar
    lib.b2_nv12_to_planar_bgr.argtypes = planar
    lib.b2_convert_dense.argtypes = [POINTER(DenseArgs), c_void_p]
    lib.b2_convert_resize.argtypes = [POINTER(ResizeArgs), c_void_p]
    lib.b2_touched_rows.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, POINTER(c_int32),
                                    POINTER(c_int32)]
    lib.b2_copy_rows.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int,
                                 c_int64, c_int]
    lib.b2_gather_surfaces.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                                       c_void_p]
    lib.b2_transfer_h2d.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p]
    lib.b2_transfer_h2d_async.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_void_p]
    lib.b2_transfer_h2d_staged.argtypes = [c_void_p, c_void_p, c_size_t, c_void_p, c_size_t, c_int,
                                           c_void_p]
    lib.b2_copy_host.argtypes = [c_void_p, c_void_p, c_size_t]
    lib.b2_pack_host.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int]
    lib.b2_transfer_d2h.argtypes = [c_void_p, c_void_p, c_size_t, c_int]
    lib.b2_transfer_d2h_staged.argtypes = [c_void_p, c_void_p, c_size_t, c_void_p, c_size_t, c_int,
                                           c_void_p]
    lib.b2_alloc_pinned.argtypes = [POINTER(c_void_p), c_size_t]
    lib.b2_free_pinned.argtypes = [c_void_p]
    lib.b2_device_alloc.argtypes = [POINTER(c_void_p), c_size_t, c_int]
    lib.b2_device_free.argtypes = [c_void_p, c_int]
    lib.b2_frame_checksum.argtypes = [c_void_p, c_int64, c_int, c_void_p, c_int, c_void_p]
    for name in EXPORTS:
        if name not in ("b2_last_error",):
            getattr(lib, name).restype = c_int


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises ``RuntimeError`` if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not LIB_PATH.exists():
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python -m spdl_b200._build`. "
                        "There is no fallback implementation.")
                handle = ctypes.CDLL(str(LIB_PATH))
                _declare(handle)
                _lib = handle
    return _lib


def check(status: int) -> None:
    """Turn a non-zero status into the exception the reference binding would raise."""
    if status != 0:
        msg = lib().b2_last_error().decode("utf-8", "replace")
        raise RuntimeError(msg or f"libb2frames call failed with status {status}")
