"""CPU oracle for the post-decode frame path.  TEST INFRASTRUCTURE ONLY.

``frame_oracle.c`` restates the reference's colour arithmetic
(``src/libspdl/cuda/detail/color_conversion.cu:20-137``) and defines the fused
resize semantics; this module builds it with ``make`` and wraps it with numpy.
Only the test-suite, the smoke check and the benchmark's CPU-baseline leg import
this package.  The shipped package (``spdl_b200``) never does, and has no CPU
fallback of its own.

``ref_kernel()`` loads ``_ref/libspdl_ref_nv12.so`` -- the reference's own kernel
source compiled unmodified for sm_100a by the ``ref`` target of the Makefile --
when it has been built; it needs a GPU to run.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB: ctypes.CDLL | None = None

NV12, I420, RGBP, RGBI = 0, 1, 2, 3
NCHW, NHWC = 0, 1
U8, F32, BF16 = 0, 1, 2
RGB, BGR = 0, 1
FMA_NONE, FMA_LUMA_FIRST, FMA_CHROMA_FIRST, FMA_DEVICE = 0, 1, 2, 4
#: which arithmetic converts a pixel: the reference's CUDA kernel, or libswscale's integers
ARITH_REFERENCE, ARITH_SWSCALE = 0, 1

#: The fusion order that reproduces the reference kernel as nvcc compiles it for
#: sm_100a (checked on a B200 over all 256^3 inputs; see tests/golden).
DEVICE_FMA_MODE = FMA_DEVICE


def build(ref: bool = False) -> None:
    """Compile ``liboracle.so`` (and, with ``ref=True``, the reference kernel)."""
    targets = ["all"] + (["ref"] if ref else [])
    subprocess.run(["make", "-s", "-C", str(_HERE), *targets], check=True)


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = _HERE / "liboracle.so"
        src = _HERE / "frame_oracle.c"
        if not path.exists() or path.stat().st_mtime < src.stat().st_mtime:
            build()
        _LIB = ctypes.CDLL(str(path))
        _LIB.orc_checksum.restype = ctypes.c_uint64
        _LIB.orc_checksum.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
    return _LIB


class _DenseArgs(ctypes.Structure):
    _fields_ = [
        ("y", ctypes.c_void_p), ("u", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("y_pitch", ctypes.c_int64), ("uv_pitch", ctypes.c_int64),
        ("y_frame_stride", ctypes.c_int64), ("uv_frame_stride", ctypes.c_int64),
        ("src_format", ctypes.c_int32), ("width", ctypes.c_int32),
        ("height", ctypes.c_int32), ("num_frames", ctypes.c_int32),
        ("coeff", ctypes.c_int32), ("full_range", ctypes.c_int32), ("fma_mode", ctypes.c_int32),
        ("dst", ctypes.c_void_p), ("dst_frame_stride", ctypes.c_int64),
        ("layout", ctypes.c_int32), ("dtype", ctypes.c_int32), ("order", ctypes.c_int32),
        ("scale_bias", ctypes.c_float * 6),
        ("arith", ctypes.c_int32),
    ]


class ImageDesc(ctypes.Structure):
    """Per-image descriptor; binary layout shared with the C ABI (64 bytes)."""

    _fields_ = [
        ("y_off", ctypes.c_uint64), ("u_off", ctypes.c_uint64), ("v_off", ctypes.c_uint64),
        ("y_pitch", ctypes.c_int32), ("uv_pitch", ctypes.c_int32),
        ("src_w", ctypes.c_int32), ("src_h", ctypes.c_int32),
        ("crop_x", ctypes.c_int32), ("crop_y", ctypes.c_int32),
        ("scale_x", ctypes.c_float), ("scale_y", ctypes.c_float),
        ("resized_w", ctypes.c_int32), ("resized_h", ctypes.c_int32),
    ]


DESC_DTYPE = np.dtype(
    [("y_off", "<u8"), ("u_off", "<u8"), ("v_off", "<u8"), ("y_pitch", "<i4"), ("uv_pitch", "<i4"),
     ("src_w", "<i4"), ("src_h", "<i4"), ("crop_x", "<i4"), ("crop_y", "<i4"),
     ("scale_x", "<f4"), ("scale_y", "<f4"), ("resized_w", "<i4"), ("resized_h", "<i4")]
)
assert DESC_DTYPE.itemsize == 64 == ctypes.sizeof(ImageDesc)


class _ResizeArgs(ctypes.Structure):
    _fields_ = [
        ("base", ctypes.c_void_p), ("descs", ctypes.c_void_p),
        ("num_images", ctypes.c_int32), ("src_format", ctypes.c_int32),
        ("out_w", ctypes.c_int32), ("out_h", ctypes.c_int32),
        ("coeff", ctypes.c_int32), ("full_range", ctypes.c_int32), ("fma_mode", ctypes.c_int32),
        ("layout", ctypes.c_int32), ("dtype", ctypes.c_int32), ("order", ctypes.c_int32),
        ("dst", ctypes.c_void_p), ("dst_image_stride", ctypes.c_int64),
        ("scale_bias", ctypes.c_float * 6),
        ("arith", ctypes.c_int32), ("frames_per_group", ctypes.c_int32),
        ("dst_plane_stride", ctypes.c_int64), ("dst_group_stride", ctypes.c_int64),
        ("pad_value", ctypes.c_float * 3),
    ]


def matrix(coeff: int = 1, full_range: bool = False) -> tuple[np.ndarray, int]:
    m = np.zeros(9, np.float32)
    y_off = ctypes.c_int(0)
    lib().orc_matrix(int(coeff), int(bool(full_range)), m.ctypes.data_as(ctypes.c_void_p),
                     ctypes.byref(y_off))
    return m.reshape(3, 3), y_off.value


def pixel(y: int, u: int, v: int, coeff: int = 1, full_range: bool = False,
          mode: int | None = None) -> tuple[int, int, int]:
    out = (ctypes.c_uint8 * 3)()
    lib().orc_pixel(int(y), int(u), int(v), int(coeff), int(bool(full_range)),
                    DEVICE_FMA_MODE if mode is None else mode, out)
    return tuple(out)


def pixel_exact(y: int, u: int, v: int, coeff: int = 1) -> tuple[int, int, int]:
    out = (ctypes.c_uint8 * 3)()
    lib().orc_pixel_exact(int(y), int(u), int(v), int(coeff), out)
    return tuple(out)


def exhaustive(coeff: int = 1, full_range: bool = False, mode: int | None = None,
               arith: int = ARITH_REFERENCE) -> np.ndarray:
    """``[256,256,256,3]`` u8: converted bytes for every (y,u,v)."""
    out = np.empty((256, 256, 256, 3), np.uint8)
    if arith == ARITH_SWSCALE:
        lib().orc_sws_exhaustive(int(coeff), int(bool(full_range)),
                                 out.ctypes.data_as(ctypes.c_void_p))
    else:
        lib().orc_exhaustive(int(coeff), int(bool(full_range)),
                             DEVICE_FMA_MODE if mode is None else mode,
                             out.ctypes.data_as(ctypes.c_void_p))
    return out


def sws_coeffs(cs: int = 1, full_range: bool = False) -> dict[str, int]:
    """libswscale's 16-bit converter constants for colourspace number ``cs``."""
    out = (ctypes.c_int * 6)()
    lib().orc_sws_coeffs(int(cs), int(bool(full_range)), out)
    return dict(zip(("yc", "vr", "ug", "vg", "ub", "yo"), out))


def sws_pixel(y: int, u: int, v: int, cs: int = 1, full_range: bool = False) -> tuple[int, int, int]:
    out = (ctypes.c_uint8 * 3)()
    lib().orc_sws_pixel(int(y), int(u), int(v), int(cs), int(bool(full_range)), out)
    return tuple(out)


_NP_OUT = {U8: np.uint8, F32: np.float32, BF16: np.uint16}


def scale_bias(mean=None, std=None) -> np.ndarray:
    """``out = v*scale + bias`` with ``scale = 1/(255*std)``, ``bias = -mean/std``
    (``mean``/``std`` in 0..1 units, per OUTPUT channel slot); identity when both are None."""
    if mean is None and std is None:
        return np.array([1, 1, 1, 0, 0, 0], np.float32)
    mean = np.asarray(mean if mean is not None else (0, 0, 0), np.float64)
    std = np.asarray(std if std is not None else (1 / 255.0,) * 3, np.float64)
    return np.concatenate([1.0 / (255.0 * std), -mean / std]).astype(np.float32)


def convert_dense(y: np.ndarray, u: np.ndarray, v: np.ndarray | None, *, width: int, height: int,
                  num_frames: int, y_pitch: int, uv_pitch: int, y_frame_stride: int,
                  uv_frame_stride: int, src_format: int = NV12, coeff: int = 1,
                  full_range: bool = False, layout: int = NCHW, dtype: int = U8, order: int = RGB,
                  sb: np.ndarray | None = None, mode: int | None = None,
                  out: np.ndarray | None = None, arith: int = ARITH_REFERENCE) -> np.ndarray:
    """General dense conversion over raw planes (u8 numpy arrays, any shape, C-contiguous)."""
    shape = (num_frames, 3, height, width) if layout == NCHW else (num_frames, height, width, 3)
    if out is None:
        out = np.zeros(shape, _NP_OUT[dtype])
    a = _DenseArgs()
    a.y, a.u = y.ctypes.data, u.ctypes.data
    a.v = v.ctypes.data if v is not None else None
    a.y_pitch, a.uv_pitch = y_pitch, uv_pitch
    a.y_frame_stride, a.uv_frame_stride = y_frame_stride, uv_frame_stride
    a.src_format, a.width, a.height, a.num_frames = src_format, width, height, num_frames
    a.coeff, a.full_range = coeff, int(bool(full_range))
    a.fma_mode = DEVICE_FMA_MODE if mode is None else mode
    a.dst, a.dst_frame_stride = out.ctypes.data, 0
    a.layout, a.dtype, a.order = layout, dtype, order
    sb = scale_bias() if sb is None else np.asarray(sb, np.float32)
    a.scale_bias = (ctypes.c_float * 6)(*sb.tolist())
    a.arith = int(arith)
    lib().orc_convert_dense(ctypes.byref(a))
    return out


def nv12_to_planar(nv12: np.ndarray, coeff: int = 1, order: int = RGB, **kw) -> np.ndarray:
    """The reference entry point: ``[N, H*3/2, W]`` u8 -> ``[N,3,H,W]`` u8
    (``src/libspdl/cuda/color_conversion.cpp:29-76``)."""
    if nv12.ndim != 3:
        raise RuntimeError(f"Expected 3D buffer [num_frames, h*1.5, width]. Found: {nv12.ndim}D")
    n, h2, w = nv12.shape
    if h2 % 3:
        raise RuntimeError(f"The height of NV12 image (h*1.5) must be divisible by 3. Found: {h2}")
    h = h2 // 3 * 2
    nv12 = np.ascontiguousarray(nv12)
    return convert_dense(nv12, nv12.reshape(-1)[h * w:], None, width=w, height=h, num_frames=n,
                         y_pitch=w, uv_pitch=w, y_frame_stride=h2 * w, uv_frame_stride=h2 * w,
                         coeff=coeff, order=order, **kw)


def convert_resize(base: np.ndarray, descs: np.ndarray, *, out_w: int, out_h: int,
                   src_format: int = NV12, coeff: int = 1, full_range: bool = False,
                   layout: int = NCHW, dtype: int = U8, order: int = RGB,
                   sb: np.ndarray | None = None, mode: int | None = None,
                   arith: int = ARITH_REFERENCE, pad_value=(0.0, 0.0, 0.0),
                   clip_frames: int = 0, out: np.ndarray | None = None) -> np.ndarray:
    """Fused convert -> bilinear -> crop / letterbox -> scale/bias over a packed byte buffer and
    a descriptor table (``DESC_DTYPE``).  ``clip_frames=T`` writes ``[N/T, 3, T, h, w]`` (planar
    only).  ``out`` may be a pre-filled array of the result's shape (images with nonsensical
    descriptors are left untouched in it)."""
    assert descs.dtype.itemsize == 64 and descs.flags.c_contiguous
    n = len(descs)
    shape = (n, 3, out_h, out_w) if layout == NCHW else (n, out_h, out_w, 3)
    if clip_frames:
        assert layout == NCHW and n % clip_frames == 0
        shape = (n // clip_frames, 3, clip_frames, out_h, out_w)
    if out is None:
        out = np.zeros(shape, _NP_OUT[dtype])
    assert out.shape == shape and out.flags.c_contiguous
    a = _ResizeArgs()
    a.base, a.descs = base.ctypes.data, descs.ctypes.data
    a.num_images, a.src_format, a.out_w, a.out_h = n, src_format, out_w, out_h
    a.coeff, a.full_range = coeff, int(bool(full_range))
    a.fma_mode = DEVICE_FMA_MODE if mode is None else mode
    a.layout, a.dtype, a.order = layout, dtype, order
    a.dst, a.dst_image_stride = out.ctypes.data, 0
    sb = scale_bias() if sb is None else np.asarray(sb, np.float32)
    a.scale_bias = (ctypes.c_float * 6)(*sb.tolist())
    a.arith = int(arith)
    a.pad_value = (ctypes.c_float * 3)(*[float(v) for v in pad_value])
    if clip_frames:
        plane = out_h * out_w
        a.frames_per_group, a.dst_image_stride = int(clip_frames), plane
        a.dst_plane_stride, a.dst_group_stride = clip_frames * plane, 3 * clip_frames * plane
    lib().orc_convert_resize(ctypes.byref(a))
    return out


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    return (x.astype(np.uint32) << 16).view(np.float32)


def gather_frames(surfaces: list[np.ndarray], width: int, height: int) -> np.ndarray:
    """Pitched ``[H*3/2, pitch]`` surfaces -> packed ``[N, H*3/2, W]``
    (``src/libspdl/cuda/nvdec/detail/buffer.cpp:31-74``)."""
    n, h2 = len(surfaces), height + height // 2
    out = np.empty((n, h2, width), np.uint8)
    ptrs = (ctypes.c_void_p * n)(*[s.ctypes.data for s in surfaces])
    pitches = (ctypes.c_int64 * n)(*[s.strides[0] for s in surfaces])
    lib().orc_gather_frames(ptrs, pitches, n, width, height, out.ctypes.data_as(ctypes.c_void_p))
    return out


def checksum(a: np.ndarray) -> int:
    a = np.ascontiguousarray(a)
    return int(lib().orc_checksum(a.ctypes.data, a.nbytes))


# ---- the reference kernel itself (GPU only) ---------------------------------------------------

_REF: ctypes.CDLL | None = None


def ref_kernel_path() -> Path:
    return _HERE / "_ref" / "libspdl_ref_nv12.so"


def ref_kernel() -> ctypes.CDLL | None:
    """The reference's own kernel, compiled unmodified; ``None`` if it was not built."""
    global _REF
    if _REF is None and ref_kernel_path().exists():
        _REF = ctypes.CDLL(str(ref_kernel_path()))
        for name in ("ref_nv12_to_planar_rgb", "ref_nv12_to_planar_bgr"):
            fn = getattr(_REF, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                           ctypes.c_int] + [ctypes.c_int] * 4
    return _REF
