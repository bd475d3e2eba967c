"""The ``spdl.io`` functions of the post-decode frame path, backed by ``libb2frames.so``.

Reference counterparts (paths within facebookresearch/spdl):

* ``nv12_to_rgb`` / ``nv12_to_bgr``      ``src/spdl/io/_core.py:1201-1267`` ->
  ``src/spdl/io/lib/cuda/color_conversion.cpp:23-76`` ->
  ``src/libspdl/cuda/color_conversion.cpp:29-97``
* ``transfer_buffer``                     ``src/spdl/io/_core.py:1168-1183`` ->
  ``src/spdl/io/lib/cuda/transfer.cpp:55-95`` -> ``src/libspdl/cuda/transfer.cpp:37-89``
* ``transfer_buffer_cpu``                 ``src/spdl/io/_core.py:1186-1195`` ->
  ``src/libspdl/cuda/transfer.cpp:91-118``
* ``FrameBatcher``                        ``src/libspdl/cuda/nvdec/detail/buffer.cpp:18-92``

``convert_nv12`` and ``convert_resize`` have no single counterpart: they fuse the conversion
with the permute / float / normalise / resize steps that reference users run as separate passes
(``examples/imagenet_classification.py:95-106``).
"""

from __future__ import annotations

import ctypes
import threading
from typing import Any, Sequence

import numpy as np

from .. import _lib
from .._lib import (ARITH_REFERENCE, ARITH_SWSCALE, BF16, BGR, F32, I420, NCHW, NHWC, NV12, RGB,
                    U8)
from ._types import CPUBuffer, CUDABuffer, CUDAConfig, cuda_buffer
from .utils import _tracing

__all__ = [
    "nv12_to_rgb", "nv12_to_bgr", "convert_nv12", "convert_resize", "make_image_descs",
    "check_resize_status", "touched_rows",
    "transfer_buffer", "transfer_buffer_cpu", "synchronize_stream", "FrameBatcher",
    "frame_checksum", "DESC_DTYPE",
]

#: numpy view of ``b2_image_desc`` (64 bytes)
DESC_DTYPE = np.dtype(
    [("y_off", "<u8"), ("u_off", "<u8"), ("v_off", "<u8"), ("y_pitch", "<i4"), ("uv_pitch", "<i4"),
     ("src_w", "<i4"), ("src_h", "<i4"), ("crop_x", "<i4"), ("crop_y", "<i4"),
     ("scale_x", "<f4"), ("scale_y", "<f4"), ("resized_w", "<i4"), ("resized_h", "<i4")]
)

_LAYOUTS = {"NCHW": NCHW, "NHWC": NHWC, NCHW: NCHW, NHWC: NHWC}
_DTYPES = {"uint8": U8, "u8": U8, "float32": F32, "fp32": F32, "f32": F32, "bfloat16": BF16,
           "bf16": BF16}
_ORDERS = {"rgb": RGB, "bgr": BGR}
RGB_PLANAR, RGB_INTERLEAVED = 2, 3
_FORMATS = {"nv12": NV12, "i420": I420, "yuv420p": I420, "rgb_planar": RGB_PLANAR,
            "rgb24": RGB_INTERLEAVED, "rgb_interleaved": RGB_INTERLEAVED}
_OUT_ELEM = {U8: ("u", 1), F32: ("f", 4), BF16: ("u", 2)}  # bf16 is exposed as 2-byte words
_ARITHS = {"reference": ARITH_REFERENCE, "cuda": ARITH_REFERENCE, "swscale": ARITH_SWSCALE,
           "ffmpeg": ARITH_SWSCALE}
_STATUS_TEXT = {
    _lib.STATUS_IMAGE_TOO_WIDE: "an image is wider than max_src_w and was skipped",
    _lib.STATUS_WAIT_EXPIRED: "a wait for staged source rows ran out and output rows were skipped",
    _lib.STATUS_BAD_GEOMETRY: "a descriptor has an empty source or a non-positive scale and was "
                              "skipped",
}


def _cai(obj: Any) -> tuple[int, tuple[int, ...], str]:
    """(pointer, shape, typestr) of a C-contiguous CUDA array."""
    iface = getattr(obj, "__cuda_array_interface__", None)
    if iface is None:
        raise TypeError(
            f"Expected an object with __cuda_array_interface__ (CUDABuffer, torch CUDA tensor); "
            f"found {type(obj).__name__}.")
    shape = tuple(int(s) for s in iface["shape"])
    strides = iface.get("strides")
    if strides is not None and 0 not in shape:
        # The stride of a dimension of size 1 never enters an address, so producers may report
        # anything for it; every other dimension must have the packed stride.
        acc = int(iface["typestr"][2:])
        for size, stride in zip(reversed(shape), reversed(tuple(strides))):
            if size != 1 and int(stride) != acc:
                raise RuntimeError("The input CUDA array must be C-contiguous.")
            acc *= size
    return int(iface["data"][0]), shape, iface["typestr"]


def _device_of(obj: Any, cfg: CUDAConfig) -> None:
    dev = getattr(obj, "device_index", None)
    if dev is None:
        d = getattr(obj, "device", None)
        dev = getattr(d, "index", None)
    if dev is not None and dev != cfg.device_index:
        raise RuntimeError(
            f"The buffer is on device {dev} but device_config targets {cfg.device_index}.")


def _scale_bias(mean, std) -> tuple[np.ndarray, np.ndarray]:
    """``scale = 1/(255*std)``, ``bias = -mean/std`` per output channel slot, in fp32, so that
    ``v*scale + bias == (v/255 - mean)/std``.  With neither given the float output is ``v``."""
    if mean is None and std is None:
        return np.ones(3, np.float32), np.zeros(3, np.float32)
    mean = np.asarray((0.0, 0.0, 0.0) if mean is None else mean, np.float64).reshape(3)
    std = np.asarray((1 / 255.0,) * 3 if std is None else std, np.float64).reshape(3)
    if np.any(std == 0):
        raise RuntimeError("std must be non-zero.")
    return (1.0 / (255.0 * std)).astype(np.float32), (-mean / std).astype(np.float32)


def synchronize_stream(device_config: CUDAConfig) -> None:
    """Block until the stream of ``device_config`` is idle."""
    _lib.check(_lib.lib().b2_stream_synchronize(device_config.device_index,
                                                device_config.stream))


# ---- colour conversion: the reference entry points -------------------------------------------


def _nv12_planar(buffers: Any, device_config: CUDAConfig, coeff: int, sync: bool,
                 bgr: bool) -> CUDABuffer:
    ptr, shape, typestr = _cai(buffers)
    if len(shape) != 3:
        raise RuntimeError(
            f"Expected 3D buffer [num_frames, h*1.5, width]. Found: {len(shape)}D")
    if typestr[1:] != "u1":
        raise RuntimeError(f"Expected uint8 buffer. Found: {typestr}")
    n, h2, w = shape
    if h2 % 3:
        raise RuntimeError(
            f"The height of NV12 image (h*1.5) must be divisible by 3. Found: {h2}")
    _device_of(buffers, device_config)
    h = h2 // 3 * 2
    out = cuda_buffer((n, 3, h, w), device_config)
    L = _lib.lib()
    # The reference launcher runs on the calling thread's current device.
    args = _lib.DenseArgs()
    args.struct_size = ctypes.sizeof(_lib.DenseArgs)
    args.device = device_config.device_index
    args.y, args.u = ptr, ptr + h * w
    args.y_pitch = args.uv_pitch = w
    args.y_frame_stride = args.uv_frame_stride = h2 * w
    args.src_format, args.width, args.height, args.num_frames = NV12, w, h, n
    args.matrix_coeff, args.full_range = int(coeff), 0
    args.dst, args.dst_frame_stride = out.data_ptr, 0
    args.layout, args.dtype, args.order = NCHW, U8, BGR if bgr else RGB
    args.scale = (ctypes.c_float * 3)(1, 1, 1)
    args.bias = (ctypes.c_float * 3)(0, 0, 0)
    with _tracing.trace_event("b2::nv12_to_planar"):
        _lib.check(L.b2_convert_dense(ctypes.byref(args), device_config.stream))
    _tracing.record("nv12_to_planar", n, n * h2 * w, out.nbytes)
    out._owner = buffers  # keep the source alive until the consumer lets go of the result
    if sync:
        synchronize_stream(device_config)
    return out


def nv12_to_rgb(buffers: Any, *, device_config: CUDAConfig, coeff: int = 1,
                sync: bool = False) -> CUDABuffer:
    """Convert a batch of NV12 images ``[num_frames, H*1.5, W]`` to planar RGB
    ``(num_frames, 3, H, W)``.

    ``coeff`` selects the matrix (1 BT709 default, 4 FCC, 5 BT470, 6 BT601, 7 SMPTE240M,
    8 YCgCo, 9 BT2020, 10 BT2020C; anything else is silently 1).  The kernel runs on
    ``device_config.stream``; with ``sync=True`` the call waits for it.
    """
    return _nv12_planar(buffers, device_config, coeff, sync, bgr=False)


def nv12_to_bgr(buffers: Any, *, device_config: CUDAConfig, coeff: int = 1,
                sync: bool = False) -> CUDABuffer:
    """Same as :func:`nv12_to_rgb`, but the order of the colour channels is BGR."""
    return _nv12_planar(buffers, device_config, coeff, sync, bgr=True)


# ---- colour conversion: general dense form ----------------------------------------------------


def convert_nv12(buffers: Any, *, device_config: CUDAConfig, coeff: int = 1,
                 full_range: bool = False, src_format: str = "nv12", layout: str = "NCHW",
                 dtype: str = "uint8", order: str = "rgb", mean=None, std=None,
                 arith: str = "reference", sync: bool = False) -> CUDABuffer:
    """Convert ``[N, H*1.5, W]`` NV12 or I420 frames in one pass to ``NCHW``/``NHWC``
    ``uint8``/``float32``/``bfloat16`` RGB or BGR, optionally normalised.

    ``arith="reference"`` computes what the reference's CUDA kernel computes;
    ``arith="swscale"`` computes what its CPU route computes (libswscale's integer yuv420p ->
    rgb24 conversion, the end of the ``format=pix_fmts=rgb24`` filter graph), with ``coeff`` read
    as libswscale's colourspace number (1 BT.709; 5, 6 and anything unknown BT.601).

    For float outputs the value is ``(v/255 - mean)/std`` per output channel when ``mean``/
    ``std`` are given (0..1 units, in output channel order), else the plain 0..255 value.
    ``bfloat16`` results are exposed as 2-byte words (``|u2``); view them as ``torch.bfloat16``.
    I420 input is the layout ``convert_frames`` produces for ``yuv420p``: Y rows, then the U
    plane and the V plane as contiguous ``H/2 x W/2`` blocks.
    """
    ptr, shape, typestr = _cai(buffers)
    if len(shape) != 3:
        raise RuntimeError(
            f"Expected 3D buffer [num_frames, h*1.5, width]. Found: {len(shape)}D")
    if typestr[1:] != "u1":
        raise RuntimeError(f"Expected uint8 buffer. Found: {typestr}")
    n, h2, w = shape
    if h2 % 3:
        raise RuntimeError(
            f"The height of NV12 image (h*1.5) must be divisible by 3. Found: {h2}")
    try:
        fmt, lay, dt, od, ar = (_FORMATS[src_format.lower()], _LAYOUTS[layout], _DTYPES[dtype],
                                _ORDERS[order.lower()], _ARITHS[arith.lower()])
    except KeyError as e:
        raise RuntimeError(f"Unsupported option: {e}") from None
    h = h2 // 3 * 2
    if fmt == I420 and w % 2:
        # the U and V blocks are [H/2, W/2] planes only when W is even
        raise RuntimeError(f"I420 width must be even. Found: {w}")
    _device_of(buffers, device_config)
    ec, depth = _OUT_ELEM[dt]
    oshape = (n, 3, h, w) if lay == NCHW else (n, h, w, 3)
    out = cuda_buffer(oshape, device_config, ec, depth)
    scale, bias = _scale_bias(mean, std)
    a = _lib.DenseArgs()
    a.struct_size = ctypes.sizeof(_lib.DenseArgs)
    a.device = device_config.device_index
    a.y = ptr
    if fmt == NV12:
        a.u, a.uv_pitch = ptr + h * w, w
    else:
        a.u, a.v, a.uv_pitch = ptr + h * w, ptr + h * w + (h // 2) * (w // 2), w // 2
    a.y_pitch = w
    a.y_frame_stride = a.uv_frame_stride = h2 * w
    a.src_format, a.width, a.height, a.num_frames = fmt, w, h, n
    a.matrix_coeff, a.full_range = int(coeff), int(bool(full_range))
    a.dst, a.dst_frame_stride = out.data_ptr, 0
    a.layout, a.dtype, a.order, a.arith = lay, dt, od, ar
    a.scale = (ctypes.c_float * 3)(*scale.tolist())
    a.bias = (ctypes.c_float * 3)(*bias.tolist())
    with _tracing.trace_event("b2::convert_dense"):
        _lib.check(_lib.lib().b2_convert_dense(ctypes.byref(a), device_config.stream))
    _tracing.record("convert_nv12", n, n * h2 * w, out.nbytes)
    out._owner = buffers
    if sync:
        synchronize_stream(device_config)
    return out


# ---- fused resize ------------------------------------------------------------------------------


def make_image_descs(widths: Sequence[int], heights: Sequence[int], *, src_format: str = "nv12",
                     offsets: Sequence[int] | None = None, resize: tuple[int, int] | None = None,
                     resize_shorter: int | None = None, crop: tuple[int, int] | None = None,
                     out_size: tuple[int, int] | None = None,
                     src_crop: tuple[int, int, int, int] | None = None,
                     scale_mode: str | None = None) -> tuple[np.ndarray, tuple[int, int]]:
    """Build the descriptor table of a (possibly ragged) packed batch.

    Images are packed back to back (``offsets[i]`` = byte offset of image ``i``; computed when
    omitted), each as Y rows then chroma (NV12: interleaved UV rows; I420: U block, V block), or,
    for sources that are already RGB (``"rgb_planar"``: three planes, ``"rgb24"``: interleaved --
    the layouts a JPEG decoder emits), as ``3*w*h`` bytes.
    Geometry: ``resize=(w, h)`` stretches every image to that size; ``resize_shorter=s`` scales
    the shorter side to ``s`` and the longer to ``int(s * long / short)``; then
    ``crop=(w, h)`` takes the centre window with offset ``int(round((dim - crop) / 2))``.
    ``scale_mode`` (with ``resize``) keeps the aspect ratio the way the reference's filter
    strings do (``src/spdl/io/_preprocessing.py:214-229``; ``"pad"`` is the reference's default):
    ``"pad"`` scales the image to fit inside ``w x h``
    (``scale=...:force_original_aspect_ratio=decrease``: the other side becomes
    ``min(round(h * iw / ih), w)`` resp. ``min(round(w * ih / iw), h)``) and centres it on a
    ``w x h`` canvas (``pad=w:h:x=-1:y=-1``: offset ``(w - iw) // 2``, rounded down to an even
    number for 4:2:0 sources, as the pad filter aligns to the chroma grid); pixels outside the
    image take ``convert_resize``'s ``pad_color``.  ``"crop"`` scales the image to cover
    ``w x h`` (``force_original_aspect_ratio=increase``) and cuts the centre ``w x h`` window
    (``crop=w:h``: offset ``(iw - w) // 2``, even for 4:2:0 sources).
    ``src_crop=(left, top, right, bottom)`` first cuts that many pixels off each side of every
    source image, the order of the reference's decoder options (crop, then scale:
    ``src/libspdl/cuda/nvdec/detail/utils.cpp:133-220``); for NV12/I420 the four values must be
    even, as the decoder requires (``src/libspdl/cuda/nvdec/decoder.cpp:29-64``).
    Returns ``(descs, (out_w, out_h))``.
    """
    w = np.asarray(widths, np.int64)
    h = np.asarray(heights, np.int64)
    if w.shape != h.shape or w.ndim != 1:
        raise RuntimeError("widths and heights must be 1-D and of equal length")
    if np.any(w < 1) or np.any(h < 1):
        raise RuntimeError("image sizes must be positive")
    fmt = _FORMATS[src_format.lower()]
    n = len(w)
    cw, chh = (w + 1) // 2, (h + 1) // 2
    frame_bytes = 3 * w * h if fmt in (RGB_PLANAR, RGB_INTERLEAVED) else w * h + 2 * cw * chh
    w0, h0 = w, h  # full image size: fixes the plane layout; (w, h) below is the source window
    if src_crop is not None:
        w = w0 - int(src_crop[0]) - int(src_crop[2])
        h = h0 - int(src_crop[1]) - int(src_crop[3])
        if np.any(w < 1) or np.any(h < 1):
            raise RuntimeError("src_crop leaves nothing of an image")
    if offsets is None:
        off = np.concatenate([[0], np.cumsum(frame_bytes)[:-1]]) if n else np.zeros(0, np.int64)
    else:
        off = np.asarray(offsets, np.int64)
    if resize is not None and resize_shorter is not None:
        raise RuntimeError("give either resize or resize_shorter")
    if scale_mode not in (None, "pad", "crop"):
        raise ValueError(f"Unexpected `scale_mode` value ({scale_mode}). "
                         'Expected values are "pad", "crop", or None.')
    if scale_mode is not None and resize is None:
        raise RuntimeError("scale_mode needs resize=(w, h)")
    # (px, py): where the resized image starts on the canvas that crop / the output window refer
    # to; (canvas_w, canvas_h): that canvas.  Without scale_mode the canvas is the resized image.
    px = py = np.zeros(n, np.int64)
    canvas = None
    if resize is not None and scale_mode is not None:
        tw_, th_ = int(resize[0]), int(resize[1])
        if tw_ < 1 or th_ < 1:
            raise RuntimeError("resize must be positive")
        fit_w = (th_ * w + h // 2) // h  # round(th * iw / ih), halves away from zero
        fit_h = (tw_ * h + w // 2) // w
        pick = np.minimum if scale_mode == "pad" else np.maximum
        rw = np.maximum(pick(fit_w, tw_), 1)
        rh = np.maximum(pick(fit_h, th_), 1)
        # distance between the canvas and the image origins: the canvas is larger in "pad" mode
        # (vf_pad: x = (w - iw) / 2), the image in "crop" mode (vf_crop: x = (iw - w) / 2)
        px, py = np.abs(tw_ - rw) // 2, np.abs(th_ - rh) // 2
        if fmt in (NV12, I420):
            # both filters place 4:2:0 frames on the chroma grid (round down)
            px, py = px - (px % 2), py - (py % 2)
        if scale_mode == "crop":
            px, py = -px, -py
        canvas = (np.full(n, tw_, np.int64), np.full(n, th_, np.int64))
    elif resize is not None:
        rw = np.full(n, int(resize[0]), np.int64)
        rh = np.full(n, int(resize[1]), np.int64)
    elif resize_shorter is not None:
        s = int(resize_shorter)
        rw = np.where(w <= h, s, (s * w) // h)
        rh = np.where(w <= h, (s * h) // w, s)
    else:
        rw, rh = w.copy(), h.copy()
    cvw, cvh = canvas if canvas is not None else (rw, rh)
    if crop is not None:
        ow, oh = int(crop[0]), int(crop[1])
        if np.any(cvw < ow) or np.any(cvh < oh):
            raise RuntimeError("crop window larger than the resized image")
        cx = np.rint((cvw - ow) / 2.0).astype(np.int64)
        cy = np.rint((cvh - oh) / 2.0).astype(np.int64)
    else:
        if n and (np.any(cvw != cvw[0]) or np.any(cvh != cvh[0])):
            raise RuntimeError("without crop every image must resize to the same size")
        ow, oh = (int(cvw[0]), int(cvh[0])) if n else (0, 0)
        cx = cy = np.zeros(n, np.int64)
    cx, cy = cx - px, cy - py  # output (0,0) in the resized image's own grid
    if out_size is not None and tuple(out_size) != (ow, oh):
        raise RuntimeError(f"out_size {out_size} does not match the geometry {(ow, oh)}")
    d = np.zeros(n, DESC_DTYPE)
    d["y_off"] = off
    d["u_off"] = off + w0 * h0
    d["y_pitch"] = w0
    if fmt == NV12:
        d["uv_pitch"] = 2 * cw
    elif fmt == I420:
        d["v_off"] = off + w0 * h0 + cw * chh
        d["uv_pitch"] = cw
    elif fmt == RGB_PLANAR:
        d["v_off"] = off + 2 * w0 * h0
        d["uv_pitch"] = w0
    else:
        d["u_off"] = 0
        d["y_pitch"] = 3 * w0
    d["src_w"], d["src_h"] = w, h
    if src_crop is not None:
        left, top, right, bottom = (int(v) for v in src_crop)
        if min(left, top, right, bottom) < 0:
            raise RuntimeError("src_crop values must be non-negative")
        yuv = fmt in (NV12, I420)
        if yuv and any(v % 2 for v in (left, top, right, bottom)):
            raise RuntimeError("src_crop values must be even for NV12/I420 sources")
        if np.any(w0 - left - right < 1) or np.any(h0 - top - bottom < 1):
            raise RuntimeError("src_crop leaves nothing of an image")
        # move the plane origins to the window's top-left corner; pitches stay those of the
        # full image
        def shift(name: str, delta) -> None:
            d[name] = d[name].astype(np.int64) + np.asarray(delta, np.int64)

        if fmt == RGB_INTERLEAVED:
            shift("y_off", top * 3 * w0 + 3 * left)
        else:
            shift("y_off", top * w0 + left)
        if fmt == NV12:
            shift("u_off", (top // 2) * 2 * cw + left)
        elif fmt == I420:
            shift("u_off", (top // 2) * cw + left // 2)
            shift("v_off", (top // 2) * cw + left // 2)
        elif fmt == RGB_PLANAR:
            shift("u_off", top * w0 + left)
            shift("v_off", top * w0 + left)
    d["crop_x"], d["crop_y"] = cx, cy
    d["scale_x"] = w.astype(np.float32) / rw.astype(np.float32)
    d["scale_y"] = h.astype(np.float32) / rh.astype(np.float32)
    if scale_mode == "pad":
        d["resized_w"], d["resized_h"] = rw, rh  # beyond this the kernel writes the pad colour
    return d, (ow, oh)


def touched_rows(desc: np.ndarray, *, src_format: str = "nv12", out_h: int
                 ) -> tuple[np.ndarray, np.ndarray]:
    """Which source rows one descriptor's vertical geometry reads when ``out_h`` output rows are
    produced: ``(luma_map, chroma_map)``, ``int32`` arrays over the source rows of the first plane
    and of the half-height planes (empty for RGB sources), holding each touched row's index among
    the touched rows of its plane and ``-1`` elsewhere.  Computed by the library with the
    kernel's own arithmetic.  A caller that uploads only those rows, in order, passes the maps to
    :func:`convert_resize` (``row_maps=``): a 4K frame resized to 224x224 needs a quarter of its
    rows on the device."""
    rec = np.ascontiguousarray(np.asarray(desc, DESC_DTYPE).reshape(-1)[:1])
    fmt = _FORMATS[src_format.lower()]
    h = int(rec["src_h"][0])
    if h < 1:
        raise RuntimeError("the descriptor has an empty source")
    luma = np.empty(h, np.int32)
    chroma = np.empty((h + 1) // 2 if fmt in (NV12, I420) else 0, np.int32)
    nl, nc = ctypes.c_int32(), ctypes.c_int32()
    _lib.check(_lib.lib().b2_touched_rows(
        rec.ctypes.data, fmt, int(out_h), luma.ctypes.data,
        chroma.ctypes.data if chroma.size else None, ctypes.byref(nl), ctypes.byref(nc)))
    return luma, chroma


_status_lock = threading.Lock()
_status_words: dict[tuple[int, int], CUDABuffer] = {}


def _status_word(cfg: CUDAConfig) -> CUDABuffer:
    """The device word ``b2_convert_resize`` reports skipped work in: one per (device, stream),
    zeroed when it is created and again after every non-zero reading."""
    key = (cfg.device_index, int(cfg.stream))
    with _status_lock:
        word = _status_words.get(key)
        if word is None:
            word = _status_words[key] = transfer_buffer(np.zeros(1, np.int32), device_config=cfg)
    return word


def check_resize_status(device_config: CUDAConfig) -> None:
    """Wait for the stream and raise ``RuntimeError`` if any ``convert_resize`` call queued on it
    since the last check left output unwritten (see ``b2_resize_status_bits``)."""
    word = _status_word(device_config)
    synchronize_stream(device_config)
    host = np.zeros(1, np.int32)
    _lib.check(_lib.lib().b2_transfer_d2h(host.ctypes.data, word.data_ptr, 4,
                                          device_config.device_index))
    bits = int(host[0])
    if bits:
        zero = np.zeros(1, np.int32)
        _lib.check(_lib.lib().b2_transfer_h2d(word.data_ptr, zero.ctypes.data, 4, 0,
                                              device_config.device_index, device_config.stream))
        what = "; ".join(t for b, t in _STATUS_TEXT.items() if bits & b)
        raise RuntimeError(f"convert_resize left output unwritten: {what} (status {bits})")


def convert_resize(base: Any, descs: Any, *, out_size: tuple[int, int], max_src_w: int,
                   device_config: CUDAConfig, src_format: str = "nv12", coeff: int = 1,
                   full_range: bool = False, layout: str = "NCHW", dtype: str = "uint8",
                   order: str = "rgb", mean=None, std=None, arith: str = "reference",
                   pad_color: tuple[float, float, float] = (0.0, 0.0, 0.0),
                   clip_frames: int | None = None, row_maps: tuple[Any, Any] | None = None,
                   sync: bool = False, _debug_flags: int = 0) -> CUDABuffer:
    """Fused colour conversion, bilinear resize, crop / letterbox and normalise over a packed
    batch.

    ``base`` is a device byte buffer holding every image, ``descs`` a device copy of the table
    from :func:`make_image_descs` (``[N]`` of ``DESC_DTYPE``, i.e. ``N*64`` bytes), ``out_size``
    is ``(out_w, out_h)`` and ``max_src_w`` the widest source image in the table.
    Returns ``[N,3,out_h,out_w]`` (``NCHW``) or ``[N,out_h,out_w,3]``.  With ``clip_frames=T``
    (planar layout, ``N`` a multiple of ``T``) consecutive groups of ``T`` images are stacked as
    clips in the channel-first video layout ``[N/T, 3, T, out_h, out_w]`` that
    ``examples/video_classification/utils/pipeline.py:137`` reaches with a ``permute``.
    ``pad_color`` is the R, G, B (0..255) of letterbox pixels (``scale_mode="pad"``).
    ``arith`` as in :func:`convert_nv12`.  ``row_maps=(luma_map, chroma_map)``: device copies of
    the arrays of :func:`touched_rows`, for a batch of equal geometry whose buffer holds only the
    touched rows of every image, back to back (the descriptors' plane offsets then point into
    that compacted buffer; ``chroma_map`` is ``None`` for RGB sources).

    The table lives in device memory, so what the host cannot check -- an image wider than
    ``max_src_w``, a nonsensical descriptor -- is reported by the kernel in a device status word:
    with ``sync=True`` the call raises ``RuntimeError`` when any image or row was skipped; with
    ``sync=False`` call :func:`check_resize_status` at a point where waiting is acceptable.
    """
    bptr, _, _ = _cai(base)
    dptr, dshape, dtypestr = _cai(descs)
    nbytes = int(np.prod(dshape, dtype=np.int64)) * int(dtypestr[2:])
    if nbytes % 64:
        raise RuntimeError("descs must be a whole number of 64-byte descriptors")
    n = nbytes // 64
    try:
        fmt, lay, dt, od, ar = (_FORMATS[src_format.lower()], _LAYOUTS[layout], _DTYPES[dtype],
                                _ORDERS[order.lower()], _ARITHS[arith.lower()])
    except KeyError as e:
        raise RuntimeError(f"Unsupported option: {e}") from None
    ow, oh = int(out_size[0]), int(out_size[1])
    _device_of(base, device_config)
    ec, depth = _OUT_ELEM[dt]
    oshape = (n, 3, oh, ow) if lay == NCHW else (n, oh, ow, 3)
    t = int(clip_frames) if clip_frames else 0
    if t:
        if lay != NCHW:
            raise RuntimeError("clip_frames needs the planar (NCHW) layout")
        if t < 1 or n % t:
            raise RuntimeError(f"{n} images do not divide into clips of {t} frames")
        oshape = (n // t, 3, t, oh, ow)
    out = cuda_buffer(oshape, device_config, ec, depth)
    scale, bias = _scale_bias(mean, std)
    status = _status_word(device_config)
    a = _lib.ResizeArgs()
    a.struct_size = ctypes.sizeof(_lib.ResizeArgs)
    a.device = device_config.device_index
    a.base, a.descs = bptr, dptr
    a.num_images, a.src_format, a.out_w, a.out_h = n, fmt, ow, oh
    a.matrix_coeff, a.full_range = int(coeff), int(bool(full_range))
    a.layout, a.dtype, a.order, a.arith = lay, dt, od, ar
    a.max_src_w = int(max_src_w)
    a.dst, a.dst_image_stride = out.data_ptr, 0
    if t:
        a.frames_per_group, a.dst_image_stride = t, oh * ow
        a.dst_plane_stride, a.dst_group_stride = t * oh * ow, 3 * t * oh * ow
    a.scale = (ctypes.c_float * 3)(*scale.tolist())
    a.bias = (ctypes.c_float * 3)(*bias.tolist())
    a.pad_value = (ctypes.c_float * 3)(*[float(v) for v in pad_color])
    a.debug_flags = int(_debug_flags)
    if row_maps is not None:
        a.luma_row_map = _cai(row_maps[0])[0]
        a.chroma_row_map = _cai(row_maps[1])[0] if row_maps[1] is not None else None
    a.status = status.data_ptr
    with _tracing.trace_event("b2::convert_resize"):
        _lib.check(_lib.lib().b2_convert_resize(ctypes.byref(a), device_config.stream))
    _tracing.record("convert_resize", n, 0, out.nbytes)
    out._owner = (base, descs, row_maps)
    if sync:
        check_resize_status(device_config)
    return out


class _DeviceSpan:
    """A bare device address range, for ``convert_resize`` over images that live in separate
    allocations (their descriptors hold offsets from the lowest address)."""

    def __init__(self, ptr: int, nbytes: int, device_index: int) -> None:
        self.device_index = device_index
        self.__cuda_array_interface__ = {"version": 2, "shape": (int(nbytes),), "typestr": "|u1",
                                         "data": (int(ptr), False), "strides": None}


def resize_image_list(images: Sequence[Any], *, device_config: CUDAConfig,
                      src_format: str = "rgb24", resize: tuple[int, int] | None = None,
                      resize_shorter: int | None = None, crop: tuple[int, int] | None = None,
                      scale_mode: str | None = None,
                      pad_color: tuple[float, float, float] = (0.0, 0.0, 0.0),
                      layout: str = "NCHW", dtype: str = "uint8", order: str = "rgb", mean=None,
                      std=None, sync: bool = False) -> CUDABuffer:
    """Resize, crop and normalise a list of decoded images of different sizes in one launch.

    ``images`` are device arrays (anything with ``__cuda_array_interface__``: the buffers a JPEG
    decoder returns, torch tensors), each C-contiguous ``uint8``: ``[H, W, 3]`` for
    ``src_format="rgb24"``, ``[3, H, W]`` for ``"rgb_planar"``.  They are read where they lie
    -- nothing is packed or copied -- and the result is one ``[N,3,h,w]`` / ``[N,h,w,3]`` batch.
    This is what follows the decoder in the reference's ``load_image_batch_nvjpeg``
    (``src/spdl/io/_composite.py:486-524``: decode, resize one image at a time with NPP, stack).
    """
    fmt = src_format.lower()
    if fmt not in ("rgb24", "rgb_planar"):
        raise RuntimeError(f"Unsupported source format for an image list: {src_format}")
    if len(images) == 0:
        raise RuntimeError("The image list is empty.")
    ptrs, ws, hs = [], [], []
    for img in images:
        ptr, shape, typestr = _cai(img)
        if typestr not in ("|u1", "<u1", "=u1") or len(shape) != 3:
            raise RuntimeError(f"Images must be 3-D uint8 arrays, got {typestr} {tuple(shape)}")
        h, w, c = shape if fmt == "rgb24" else (shape[1], shape[2], shape[0])
        if c != 3:
            raise RuntimeError(f"Images must have three channels, got shape {tuple(shape)}")
        _device_of(img, device_config)
        ptrs.append(ptr)
        ws.append(w)
        hs.append(h)
    base = min(ptrs)
    end = max(p + 3 * w * h for p, w, h in zip(ptrs, ws, hs))
    descs, out_size = make_image_descs(ws, hs, src_format=fmt, offsets=[p - base for p in ptrs],
                                       resize=resize, resize_shorter=resize_shorter, crop=crop,
                                       scale_mode=scale_mode)
    table = transfer_buffer(descs.view(np.uint8), device_config=device_config)
    out = convert_resize(_DeviceSpan(base, end - base, device_config.device_index), table,
                         out_size=out_size, max_src_w=max(ws), device_config=device_config,
                         src_format=fmt, layout=layout, dtype=dtype, order=order, mean=mean,
                         std=std, pad_color=pad_color, sync=sync)
    out._owner = (list(images), table)  # inputs must outlive the queued kernel
    return out


def resize_host_images(images: Sequence[Any], *, device_config: CUDAConfig,
                       src_format: str = "rgb24", resize: tuple[int, int] | None = None,
                       resize_shorter: int | None = None, crop: tuple[int, int] | None = None,
                       scale_mode: str | None = None,
                       pad_color: tuple[float, float, float] = (0.0, 0.0, 0.0),
                       layout: str = "NCHW", dtype: str = "uint8", order: str = "rgb",
                       coeff: int = 1, full_range: bool = False, arith: str = "reference",
                       mean=None, std=None) -> CUDABuffer:
    """Upload a list of decoded HOST images of different sizes and resize, crop, convert and
    normalise them in one launch.

    ``images`` are C-contiguous ``uint8`` NumPy arrays or CPU tensors: ``[H, W, 3]`` for
    ``src_format="rgb24"``, ``[3, H, W]`` for ``"rgb_planar"``, and the packed planes a decoder
    leaves for ``"i420"`` / ``"nv12"`` -- ``[H*3/2, W]``, the luma rows followed by the chroma
    (even ``W`` and ``H``).  The images are packed back to back (16-byte aligned) into the
    calling thread's page-locked staging buffer by several host threads (``b2_pack_host``), go
    up in ONE asynchronous copy on ``device_config.stream`` and are read by the fused kernel
    through an offset table; the call returns when the result is complete.

    The reference's ``load_image_batch`` (``src/spdl/io/_composite.py:438-463``) resizes every
    image on the CPU so that ``convert_frames`` can batch equal sizes, then uploads the batch.
    """
    fmt = src_format.lower()
    fmt = "i420" if fmt == "yuv420p" else fmt
    if fmt not in ("rgb24", "rgb_planar", "i420", "nv12"):
        raise RuntimeError(f"Unsupported source format for an image list: {src_format}")
    if len(images) == 0:
        raise RuntimeError("The image list is empty.")
    arrays, ws, hs = [], [], []
    for img in images:
        if hasattr(img, "is_cuda") and hasattr(img, "numpy"):  # torch tensor
            if img.is_cuda:
                raise RuntimeError("resize_host_images expects CPU images.")
            img = img.contiguous().numpy()
        arr = np.ascontiguousarray(img)
        want_dims = 2 if fmt in ("i420", "nv12") else 3
        if arr.dtype != np.uint8 or arr.ndim != want_dims:
            raise RuntimeError(
                f"Images must be {want_dims}-D uint8 arrays, got {arr.dtype} {arr.shape}")
        if fmt == "rgb24":
            h, w, c = arr.shape
        elif fmt == "rgb_planar":
            c, h, w = arr.shape
        else:
            h2, w = arr.shape
            if h2 % 3 or (h2 // 3 * 2) % 2 or w % 2:
                raise RuntimeError(f"Planes of an even-sized 4:2:0 image are [H*3/2, W]. Found: "
                                   f"{arr.shape}")
            h, c = h2 // 3 * 2, 3
        if c != 3:
            raise RuntimeError(f"Images must have three channels, got shape {arr.shape}")
        arrays.append(arr)
        ws.append(w)
        hs.append(h)
    n = len(arrays)
    sizes = np.array([a.nbytes for a in arrays], np.int64)
    offsets = np.zeros(n, np.int64)
    np.cumsum((sizes[:-1] + 15) & ~15, out=offsets[1:])
    total = int(offsets[-1] + sizes[-1])
    host = _staging_arena().reserve(total)
    srcs = np.array([a.ctypes.data for a in arrays], np.uint64)
    L = _lib.lib()
    _lib.check(L.b2_pack_host(host, srcs.ctypes.data, sizes.ctypes.data, offsets.ctypes.data, n))
    base = cuda_buffer((total,), device_config, "u", 1)
    _lib.check(L.b2_transfer_h2d_async(base.data_ptr, host, total, device_config.device_index,
                                       device_config.stream))
    descs, out_size = make_image_descs(ws, hs, src_format=fmt, offsets=offsets, resize=resize,
                                       resize_shorter=resize_shorter, crop=crop,
                                       scale_mode=scale_mode)
    table = transfer_buffer(descs.view(np.uint8), device_config=device_config)
    # sync=True: the staging buffer is this thread's, and free again when the call returns
    out = convert_resize(base, table, out_size=out_size, max_src_w=max(ws),
                         device_config=device_config, src_format=fmt, coeff=coeff,
                         full_range=full_range, arith=arith, layout=layout, dtype=dtype,
                         order=order, mean=mean, std=std, pad_color=pad_color, sync=True)
    _tracing.record("resize_host_images", n, total, out.nbytes)
    return out


# ---- transfer ----------------------------------------------------------------------------------

_NP_CLASS = {"u": "u", "i": "i", "f": "f", "b": "u"}
_warned_legacy_stream = False


def _warn_legacy_stream_once() -> None:
    global _warned_legacy_stream
    if not _warned_legacy_stream:
        _warned_legacy_stream = True
        import warnings

        warnings.warn(
            "The CPU buffer is page-locked (pinned), but the legacy default CUDA stream (0) is "
            "used. This is likely not what you intend. Please use a non-default CUDA stream to "
            "overlap the data transfer with kernel execution.", RuntimeWarning, stacklevel=3)


_STAGED_MIN_BYTES = 8 << 20   # pageable sources from this size on are staged by this package
_PER_THREAD_STREAM = 0x2      # cudaStreamPerThread: what a blocking copy of this library uses
_STAGING_BYTES = 32 << 20     # page-locked staging per calling thread (two halves of 16 MiB)
_STAGING_LOCAL = threading.local()


def _staging_arena():
    arena = getattr(_STAGING_LOCAL, "arena", None)
    if arena is None:
        from ._transfer import _StagingArena

        arena = _STAGING_LOCAL.arena = _StagingArena()
    return arena


def transfer_buffer(buffer: Any, *, device_config: CUDAConfig) -> CUDABuffer:
    """Move host data to the GPU; shape and element type are preserved.

    Accepts a :class:`CPUBuffer`, a NumPy array or a CPU torch tensor (non-contiguous inputs are
    made contiguous first).  Pinned sources are copied asynchronously on
    ``device_config.stream`` and the stream is then synchronised; small pageable sources use a
    blocking copy, large ones (8 MiB and more) go through a page-locked staging buffer of the
    calling thread, staged by several host threads while the previous part uploads (about twice
    the rate of the driver's pageable copy) -- in every case the data is on the device when the
    call returns.
    """
    keep: Any = buffer
    if isinstance(buffer, CPUBuffer):
        ptr, shape, ec, depth = buffer.data_ptr, buffer.shape, buffer.elem_class, buffer.depth
        pinned = buffer.is_pinned()
    else:
        pinned = False
        if hasattr(buffer, "is_cuda") and hasattr(buffer, "numpy"):  # torch tensor
            if buffer.is_cuda:
                raise RuntimeError("transfer_buffer expects a CPU tensor.")
            pinned = bool(buffer.is_pinned()) and buffer.is_contiguous()
            arr = buffer.contiguous().numpy()
        else:
            arr = np.ascontiguousarray(buffer)
        if arr.dtype.kind not in _NP_CLASS:
            raise RuntimeError(f"Unsupported dtype: {arr.dtype}")
        keep = arr
        ptr, shape = arr.ctypes.data, arr.shape
        ec, depth = _NP_CLASS[arr.dtype.kind], arr.dtype.itemsize
    if pinned and device_config.stream == 0:
        # as the reference does once per process (src/libspdl/cuda/transfer.cpp:28-35,48-52)
        _warn_legacy_stream_once()
    out = cuda_buffer(shape, device_config, ec, depth)
    with _tracing.trace_event("b2::transfer_h2d"):
        if not pinned and out.nbytes >= _STAGED_MIN_BYTES:
            # a large pageable source: through this thread's page-locked staging buffer, the
            # staging copy (several host threads) of one half under the upload of the other
            arena = _staging_arena()
            _lib.check(_lib.lib().b2_transfer_h2d_staged(
                out.data_ptr, ptr, out.nbytes, arena.reserve(_STAGING_BYTES), _STAGING_BYTES,
                device_config.device_index, device_config.stream))
        else:
            _lib.check(_lib.lib().b2_transfer_h2d(out.data_ptr, ptr, out.nbytes, int(pinned),
                                                  device_config.device_index,
                                                  device_config.stream))
    _tracing.record("transfer_buffer", 1, out.nbytes, out.nbytes)
    del keep
    return out


def transfer_buffer_cpu(buffer: Any) -> CPUBuffer:
    """Move a CUDA array (anything with ``__cuda_array_interface__``) to host memory."""
    ptr, shape, typestr = _cai(buffer)
    ec, depth = typestr[1], int(typestr[2:])
    dev = getattr(buffer, "device_index", None)
    if dev is None:
        dev = getattr(getattr(buffer, "device", None), "index", 0) or 0
    out = CPUBuffer(shape, _NP_CLASS.get(ec, "u"), depth)
    if out.nbytes >= _STAGED_MIN_BYTES:
        # through this thread's page-locked staging buffer, downloads under the copies out
        arena = _staging_arena()
        _lib.check(_lib.lib().b2_transfer_d2h_staged(
            out.data_ptr, ptr, out.nbytes, arena.reserve(_STAGING_BYTES), _STAGING_BYTES, dev,
            _PER_THREAD_STREAM))
    else:
        _lib.check(_lib.lib().b2_transfer_d2h(out.data_ptr, ptr, out.nbytes, dev))
    return out


# ---- frame batching ----------------------------------------------------------------------------


class FrameBatcher:
    """Batches pitched NV12 decoder surfaces into packed ``[num_frames, H*3/2, W]`` buffers.

    Same observable behaviour as the reference's ``FrameBuffer`` -- ``push`` a surface, full
    batches queue up, ``flush`` emits a short last batch whose ``shape[0]`` is the number of
    frames pushed -- but surfaces are only recorded on ``push``; one gather kernel copies the
    whole batch when it completes, with no per-frame stream synchronisation.  Surfaces must stay
    valid until their batch has been emitted.
    """

    def __init__(self, num_frames: int, width: int, height: int, device_config: CUDAConfig):
        if num_frames < 1:
            raise RuntimeError("num_frames must be positive")
        if width < 1 or height < 1 or height % 2:
            raise RuntimeError(f"Invalid NV12 frame size: {width}x{height}")
        self._n, self._w, self._h, self._cfg = int(num_frames), int(width), int(height), \
            device_config
        self._pending: list[tuple[int, int]] = []
        self._queue: list[CUDABuffer] = []
        self._tables = None  # pinned ring for the pointer/pitch tables, made on first use
        self._slot = 0

    def empty(self) -> bool:
        return not self._queue

    def push(self, surface_ptr: int, pitch: int) -> None:
        if pitch < self._w:
            raise RuntimeError(f"pitch {pitch} is smaller than the width {self._w}")
        self._pending.append((int(surface_ptr), int(pitch)))
        if len(self._pending) == self._n:
            self._emit()

    def flush(self) -> None:
        if self._pending:
            self._emit()

    def pop(self) -> CUDABuffer:
        if not self._queue:
            raise RuntimeError("There is no buffer available.")
        return self._queue.pop(0)

    _TABLE_SLOTS = 8  # pinned copies of the pointer/pitch table in flight at most

    def _table_slot(self) -> tuple[int, np.ndarray]:
        """Host address and int64 view of the next pinned table slot.  The slots form a ring; the
        stream is synchronised once per lap, so a slot is never rewritten while its upload may
        still be reading it, and a steady stream of batches costs one wait per eight."""
        from ._types import CPUStorage

        if self._tables is None:
            self._tables = CPUStorage(self._TABLE_SLOTS * 16 * self._n, pin_memory=True)
            self._slot = 0
        if self._slot == self._TABLE_SLOTS:
            synchronize_stream(self._cfg)
            self._slot = 0
        off = self._slot * 16 * self._n
        self._slot += 1
        view = self._tables.as_array()[off:off + 16 * self._n].view(np.int64)
        return self._tables.data_ptr + off, view

    def _emit(self) -> None:
        k = len(self._pending)
        h2 = self._h + self._h // 2
        out = cuda_buffer((k, h2, self._w), self._cfg)
        host_ptr, table = self._table_slot()
        table[:k] = [p for p, _ in self._pending]
        table[k:2 * k] = [q for _, q in self._pending]
        dtab = cuda_buffer((2 * k,), self._cfg, "i", 8)
        # asynchronous upload from pinned memory, then the gather on the same stream: no host wait
        _lib.check(_lib.lib().b2_transfer_h2d_async(dtab.data_ptr, host_ptr, 16 * k,
                                                    self._cfg.device_index, self._cfg.stream))
        _lib.check(_lib.lib().b2_gather_surfaces(
            dtab.data_ptr, dtab.data_ptr + 8 * k, k, self._w, self._h, out.data_ptr,
            self._cfg.device_index, self._cfg.stream))
        out._owner = dtab
        self._pending = []
        self._queue.append(out)


def frame_checksum(buffer: Any, *, device_config: CUDAConfig) -> np.ndarray:
    """Per-frame 64-bit checksum of a CUDA array, first dimension = frames (blocking)."""
    ptr, shape, typestr = _cai(buffer)
    n = shape[0] if shape else 0
    frame_bytes = int(np.prod(shape[1:], dtype=np.int64)) * int(typestr[2:]) if n else 0
    if n == 0:
        return np.zeros(0, np.uint64)
    out = cuda_buffer((n,), device_config, "u", 8)
    _lib.check(_lib.lib().b2_frame_checksum(ptr, frame_bytes, n, out.data_ptr,
                                            device_config.device_index, device_config.stream))
    synchronize_stream(device_config)
    host = transfer_buffer_cpu(out)
    return np.array(host, copy=True).reshape(n)
