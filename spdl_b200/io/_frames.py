"""Decoded frames on the host and their batching into one contiguous buffer.

``convert_frames`` mirrors ``spdl.io.convert_frames`` (``src/spdl/io/_core.py:1013-1042``;
C++ ``src/libspdl/core/detail/ffmpeg/conversion.cpp:171-303, 410-454``): every frame's planes
are copied row by row (dropping line padding) into one C-contiguous buffer whose shape depends
on the pixel format.  The decoder itself is outside this package, so frames are described by
:class:`Frames` -- plane arrays with a line size, as a decoder hands them over.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np

from ._types import CPUBuffer, CPUStorage

__all__ = ["Frames", "convert_frames", "convert_array"]

# pix_fmt -> (kind, channels/planes)
_INTERLEAVED = {"rgb24": 3, "bgr24": 3, "rgba": 4, "bgra": 4, "gray8": 1, "gray": 1}
_PLANAR = {"yuv444p": 3, "yuvj444p": 3}
_YUV420 = {"yuv420p", "yuvj420p"}
_YUV422 = {"yuv422p", "yuvj422p"}


@dataclass
class Frames:
    """A run of decoded frames of one size and pixel format.

    ``planes[i][p]`` is plane ``p`` of frame ``i`` as a 2-D ``uint8`` array whose row stride may
    exceed the visible row (line padding).  ``media`` is ``"video"`` or ``"image"``; an image
    holds exactly one frame and its batch dimension is dropped by ``convert_frames``.
    """

    pix_fmt: str
    width: int
    height: int
    planes: list[list[np.ndarray]] = field(default_factory=list)
    media: str = "video"

    @property
    def num_frames(self) -> int:
        return len(self.planes)

    def _plane_shapes(self) -> list[tuple[int, int]]:
        w, h = self.width, self.height
        f = self.pix_fmt
        if f in _INTERLEAVED:
            return [(h, w * _INTERLEAVED[f])]
        if f in _PLANAR:
            return [(h, w)] * 3
        if f in _YUV420:
            return [(h, w), (h // 2, w // 2), (h // 2, w // 2)]
        if f in _YUV422:
            return [(h, w), (h, w // 2), (h, w // 2)]
        if f == "nv12":
            return [(h, w), (h // 2, w)]
        raise RuntimeError(f"Unsupported pixel format: {f}")

    def validate(self) -> None:
        shapes = self._plane_shapes()
        if self.media == "image" and self.num_frames != 1:
            raise RuntimeError("An image holds exactly one frame.")
        for i, fr in enumerate(self.planes):
            if len(fr) != len(shapes):
                raise RuntimeError(
                    f"Frame {i} has {len(fr)} planes; {self.pix_fmt} needs {len(shapes)}.")
            for p, (arr, (rows, cols)) in enumerate(zip(fr, shapes)):
                if arr.dtype != np.uint8 or arr.ndim != 2 or arr.shape[0] < rows \
                        or arr.shape[1] < cols:
                    raise RuntimeError(
                        f"Frame {i} plane {p}: expected uint8 [{rows}, >={cols}], "
                        f"found {arr.dtype} {arr.shape}.")

    def frame_bytes(self) -> int:
        return sum(r * c for r, c in self._plane_shapes())


def _frame_shape(fr: Frames) -> tuple[int, ...]:
    w, h, f = fr.width, fr.height, fr.pix_fmt
    if f in _INTERLEAVED:
        return (h, w, _INTERLEAVED[f])
    if f in _PLANAR:
        return (3, h, w)
    if f in _YUV420 or f == "nv12":
        if h % 2 or w % 2:
            raise RuntimeError(f"Width and height must be even for {f}. Found: {w}x{h}")
        return (1, h + h // 2, w)
    if f in _YUV422:
        return (1, h + h, w)
    raise RuntimeError(f"Unsupported pixel format: {f}")


def convert_frames(frames: Frames | Sequence[Frames],
                   storage: CPUStorage | None = None) -> CPUBuffer:
    """Copy decoded frames into one contiguous host buffer.

    Shapes (``B`` = number of ``Frames`` objects when a list is given, ``N`` = frames per
    object; images drop ``N``; a single non-list argument drops ``B``):

    * ``rgb24``/``bgr24``/``rgba``/``gray8``: ``[B, N, H, W, C]``
    * ``yuv444p``: ``[B, N, 3, H, W]``
    * ``yuv420p``, ``nv12``: ``[B, N, 1, H + H/2, W]``
    * ``yuv422p``: ``[B, N, 1, 2H, W]``

    All frames must agree in size and format, else ``RuntimeError``; ``storage`` (for example
    pinned memory from ``cpu_storage``) must be large enough, else ``RuntimeError``.
    """
    single = isinstance(frames, Frames)
    batch = [frames] if single else list(frames)
    if not batch:
        raise RuntimeError("No frame to convert.")
    ref = batch[0]
    for fr in batch:
        if not isinstance(fr, Frames):
            raise TypeError("convert_frames takes Frames or a list of Frames")
        fr.validate()
        if (fr.pix_fmt, fr.width, fr.height, fr.media) != (ref.pix_fmt, ref.width, ref.height,
                                                           ref.media):
            raise RuntimeError(
                "Cannot convert the frames as the frames do not have the same size/format. "
                f"Reference {ref.pix_fmt} {ref.width}x{ref.height}, "
                f"found {fr.pix_fmt} {fr.width}x{fr.height}.")
        if fr.num_frames != ref.num_frames:
            raise RuntimeError("All the frame sequences must have the same number of frames.")
    inner = _frame_shape(ref)
    full = (len(batch), ref.num_frames, *inner)
    buf = CPUBuffer(full, "u", 1, storage)
    flat = np.frombuffer((__import__("ctypes").c_uint8 * max(buf.nbytes, 1)).from_address(
        buf.data_ptr), np.uint8, count=buf.nbytes)
    # Planes whose rows lie back to back are packed by one call of the library's host helper,
    # which deals them out to several threads when the batch is several MiB long (the reference
    # copies frame by frame on one thread: av_image_copy_to_buffer in
    # src/libspdl/core/detail/ffmpeg/conversion.cpp:171-216); pitched planes row by row here.
    pos = 0
    shapes = ref._plane_shapes()
    srcs, sizes, offsets = [], [], []
    for fr in batch:
        for planes in fr.planes:
            for arr, (rows, cols) in zip(planes, shapes):
                n = rows * cols
                view = arr[:rows, :cols]
                if view.dtype == np.uint8 and view.flags.c_contiguous:
                    srcs.append(view.ctypes.data)
                    sizes.append(n)
                    offsets.append(pos)
                else:
                    flat[pos:pos + n].reshape(rows, cols)[...] = view
                pos += n
    if srcs:
        from .. import _lib

        s_arr, z_arr, o_arr = (np.array(v, t) for v, t in ((srcs, np.uint64), (sizes, np.int64),
                                                           (offsets, np.int64)))
        _lib.check(_lib.lib().b2_pack_host(buf.data_ptr, s_arr.ctypes.data, z_arr.ctypes.data,
                                           o_arr.ctypes.data, len(srcs)))
    shape = full
    if ref.media == "image":
        shape = (shape[0], *shape[2:])
    if single:
        shape = shape[1:]
    buf.shape = tuple(shape)
    return buf


def convert_array(vals: np.ndarray, storage: CPUStorage | None = None) -> CPUBuffer:
    """Copy an int64 array (class labels and the like) into a ``CPUBuffer``, optionally backed by
    pinned ``storage`` so that its upload can overlap kernels
    (``src/spdl/io/_core.py:1045-1062``, ``src/spdl/io/lib/core/conversion.cpp:70-93``).
    An empty array is an error; other element types are rejected as the binding does."""
    arr = np.asarray(vals)
    if arr.dtype != np.int64:
        raise TypeError(f"convert_array takes an int64 array, got {arr.dtype}")
    if arr.size == 0:
        raise RuntimeError("The array be empty.")
    arr = np.ascontiguousarray(arr)
    buf = CPUBuffer(arr.shape, "i", 8, storage)
    np.array(buf, copy=False)[...] = arr
    return buf
