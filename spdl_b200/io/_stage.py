"""A pipeline stage: decoded frames on the host in, model-ready tensor on the GPU out.

The reference composes ``convert_frames -> transfer_buffer -> to_torch`` in a worker thread and
leaves colour conversion to the CPU filter graph and normalisation to user code
(``src/spdl/io/_composite.py:55-69``, ``examples/video_dataloading.py:156-177``).  This stage
uploads the frames in their native YUV layout -- half the bytes of rgb24 over PCIe -- and does
conversion, resize, crop and normalise in one kernel on the GPU.

Like ``transfer_tensor`` (``src/spdl/io/_transfer.py:91-126``) it is meant to be called from a
pool of worker threads: every thread gets its own CUDA stream on ``cuda:{LOCAL_RANK}``, the call
returns after that stream has finished, and the last ``num_caches`` results are kept alive so the
caching allocator cannot recycle their memory for another stream while a consumer still reads it.
"""

from __future__ import annotations

import os
import threading
from typing import Any

import numpy as np

from .. import _lib
from ._convert import to_torch
from ._core import (convert_nv12, convert_resize, make_image_descs, touched_rows,
                    transfer_buffer)
from ._types import CPUBuffer, CPUStorage, CUDAConfig, cuda_buffer, cuda_config

__all__ = ["FrameStage"]


class FrameStage:
    """Callable ``stage(frames) -> torch.Tensor`` for ``[N, H*3/2, W]`` NV12/I420 host frames.

    ``frames`` is a :class:`CPUBuffer` from ``convert_frames`` (a leading batch/plane dimension
    of size 1 is squeezed) or a ``uint8`` NumPy array.  Without ``resize``/``resize_shorter`` the
    frames are converted at full size; otherwise they are resized (and centre-cropped with
    ``crop``, or letterboxed / cover-cropped with ``scale_mode`` as the reference's filter
    strings do) in the same kernel.  ``clip_frames=T`` stacks every ``T`` frames as a clip in the
    channel-first video layout ``[N/T, 3, T, h, w]``.  ``arith="swscale"`` reproduces the pixels
    of the reference's CPU route (libswscale) instead of those of its CUDA kernel.
    ``dtype="bfloat16"`` returns a ``torch.bfloat16`` tensor.

    ``sparse_upload=True`` (resizing stages only) copies into the page-locked staging buffer, and
    over PCIe, only the source rows the geometry reads -- a quarter of a 4K frame that becomes
    224x224, four fifths of a 720p frame that becomes 256x256 -- instead of whole frames; the
    kernel finds the rows through the maps of :func:`touched_rows`.  The result is identical.
    ``sparse_upload="auto"`` does so when the geometry reads less than 85 % of a frame's bytes.
    Frames in pageable memory are first copied into the page-locked staging buffer by several
    host threads with streaming stores (``b2_copy_host`` for whole frames, ``b2_copy_rows`` for
    the touched rows) and uploaded from there asynchronously; that copy, at about 45 GB/s, is what
    bounds the stage (measured on a B200 host, 16 cores, two worker threads: 4K -> 224x224 3.5 k
    frames/s whole, 11 k sparse; 720p -> 256x256 33 k whole, 36 k sparse; the driver's own
    staging of pageable sources gave 0.8 k and 7 k).
    """

    def __init__(self, *, src_format: str = "i420", layout: str = "NCHW", dtype: str = "float32",
                 order: str = "rgb", coeff: int = 1, full_range: bool = False, mean=None, std=None,
                 resize: tuple[int, int] | None = None, resize_shorter: int | None = None,
                 crop: tuple[int, int] | None = None, scale_mode: str | None = None,
                 pad_color: tuple[float, float, float] = (0.0, 0.0, 0.0),
                 clip_frames: int | None = None, arith: str = "reference",
                 sparse_upload: bool = False, num_caches: int = 4,
                 device_index: int | None = None) -> None:
        if num_caches < 0:
            raise RuntimeError("num_caches must be non-negative")
        if crop is not None and resize is None and resize_shorter is None:
            raise RuntimeError("crop needs resize or resize_shorter")
        self._opts = dict(src_format=src_format, layout=layout, dtype=dtype, order=order,
                          coeff=coeff, full_range=full_range, mean=mean, std=std, arith=arith)
        self._geom = dict(resize=resize, resize_shorter=resize_shorter, crop=crop,
                          scale_mode=scale_mode)
        self._resizing = resize is not None or resize_shorter is not None
        if clip_frames and not self._resizing:
            raise RuntimeError("clip_frames needs resize or resize_shorter")
        self._resize_opts = dict(pad_color=pad_color, clip_frames=clip_frames)
        if sparse_upload not in (False, True, "auto"):
            raise RuntimeError('sparse_upload is False, True or "auto"')
        if sparse_upload is True and not self._resizing:
            raise RuntimeError("sparse_upload needs resize or resize_shorter")
        if sparse_upload is True and src_format.lower() not in ("nv12", "i420", "yuv420p"):
            raise RuntimeError("sparse_upload takes NV12 or I420 frames")
        if sparse_upload == "auto" and not (
                self._resizing and src_format.lower() in ("nv12", "i420", "yuv420p")):
            sparse_upload = False
        self._sparse = sparse_upload
        self._num_caches = int(num_caches)
        self._device_index = device_index
        self._local = threading.local()

    # -- per-thread state ------------------------------------------------------------------------
    def _state(self):
        st = getattr(self._local, "state", None)
        if st is None:
            import torch

            index = self._device_index
            if index is None:
                index = int(os.environ.get("LOCAL_RANK", "0"))
            if index >= torch.cuda.device_count():
                raise RuntimeError(f"Local rank {index} was asked for, but this process sees only "
                                   f"{torch.cuda.device_count()} CUDA device(s).")
            stream = torch.cuda.Stream(torch.device("cuda", index))
            st = {"stream": stream, "cfg": cuda_config(index, stream=stream.cuda_stream),
                  "cache": [None] * self._num_caches, "descs": {},
                  "uploads": {"sparse": 0, "whole": 0}}  # calls of this thread by upload kind
            self._local.state = st
        return st

    def _descs_for(self, st, n: int, w: int, h: int):
        key = (n, w, h)
        hit = st["descs"].get(key)
        if hit is None:
            table, out = make_image_descs([w] * n, [h] * n, src_format=self._opts["src_format"],
                                          **self._geom)
            dev = transfer_buffer(table.view(np.uint8), device_config=st["cfg"])
            hit = st["descs"][key] = (dev, out)
        return hit

    def _sparse_plan(self, st, n: int, w: int, h: int):
        """For frames of one size: which rows to copy, the descriptor table of the compacted
        batch and the row maps on the device (built once per size and thread)."""
        key = ("sparse", n, w, h)
        plan = st["descs"].get(key)
        if plan is None:
            fmt = self._opts["src_format"].lower()
            table, out = make_image_descs([w] * n, [h] * n, src_format=fmt, **self._geom)
            luma, chroma = touched_rows(table[0], src_format=fmt, out_h=out[1])
            lrows = np.flatnonzero(luma >= 0)
            crows = np.flatnonzero(chroma >= 0)
            cw = w if fmt == "nv12" else w // 2            # bytes of a chroma row
            planes = 1 if fmt == "nv12" else 2             # chroma planes
            frame_bytes = len(lrows) * w + planes * len(crows) * cw
            table["y_off"] = np.arange(n, dtype=np.uint64) * frame_bytes
            table["u_off"] = table["y_off"] + len(lrows) * w
            if fmt != "nv12":
                table["v_off"] = table["u_off"] + len(crows) * cw
            cfg = st["cfg"]
            plan = st["descs"][key] = dict(
                out=out, lrows=lrows, crows=crows, cw=cw, frame_bytes=frame_bytes,
                fraction=frame_bytes / (h * w * 1.5),
                descs=transfer_buffer(table.view(np.uint8), device_config=cfg),
                maps=(transfer_buffer(luma, device_config=cfg),
                      transfer_buffer(chroma, device_config=cfg)))
        return plan

    def _gather_rows(self, st, frames: np.ndarray, plan, w: int, h: int) -> CPUBuffer:
        """Copy the touched rows of every frame into the thread's page-locked staging buffer."""
        n = frames.shape[0]
        need = n * plan["frame_bytes"]
        store = st.get("pinned")
        if store is None or store.size < need:
            store = st["pinned"] = CPUStorage(max(need, 1 << 20), pin_memory=True)
        nl, nc, cw = len(plan["lrows"]), len(plan["crows"]), plan["cw"]
        fb, src_fb = plan["frame_bytes"], frames.strides[0]
        src, dst = frames.ctypes.data, store.data_ptr
        copy = _lib.lib().b2_copy_rows  # plain memcpy per row, outside the GIL
        lrows = np.ascontiguousarray(plan["lrows"], np.int32)
        crows = np.ascontiguousarray(plan["crows"], np.int32)
        _lib.check(copy(dst, fb, src, src_fb, w, lrows.ctypes.data, nl, w, n))
        if cw == w:  # NV12: interleaved chroma rows follow the luma rows
            _lib.check(copy(dst + nl * w, fb, src + h * w, src_fb, w, crows.ctypes.data, nc, w, n))
        else:        # I420: a U block and a V block of half-width rows
            blk = (h // 2) * cw
            for k in range(2):
                _lib.check(copy(dst + nl * w + k * nc * cw, fb, src + h * w + k * blk, src_fb, cw,
                                crows.ctypes.data, nc, cw, n))
        return CPUBuffer((need,), "u", 1, store)

    def _stage_whole(self, st, frames: np.ndarray) -> CPUBuffer:
        """Copy a batch of pageable frames into the thread's page-locked staging buffer (several
        host threads for large batches), from where the upload runs asynchronously at the
        link's rate; the driver's own staging of a pageable source is several times slower."""
        need = frames.nbytes
        store = st.get("pinned")
        if store is None or store.size < need:
            store = st["pinned"] = CPUStorage(max(need, 1 << 20), pin_memory=True)
        _lib.check(_lib.lib().b2_copy_host(store.data_ptr, frames.ctypes.data, need))
        return CPUBuffer(frames.shape, "u", 1, store)

    @staticmethod
    def _upload(view, cfg: CUDAConfig):
        """Host frames to the device on the thread's stream.  Page-locked sources are queued
        without a wait (the conversion that follows runs on the same stream and the call waits
        once, at its end); pageable ones go through the blocking copy of ``transfer_buffer``."""
        if isinstance(view, CPUBuffer) and view.is_pinned():
            dev = cuda_buffer(view.shape, cfg, view.elem_class, view.depth)
            _lib.check(_lib.lib().b2_transfer_h2d_async(dev.data_ptr, view.data_ptr, dev.nbytes,
                                                        cfg.device_index, cfg.stream))
            dev._owner = view  # the source must outlive the queued copy
            return dev
        return transfer_buffer(view, device_config=cfg)

    # -- the call --------------------------------------------------------------------------------
    def __call__(self, frames: Any):
        import torch

        st = self._state()
        cfg: CUDAConfig = st["cfg"]
        shape = tuple(frames.shape)
        while len(shape) > 3 and 1 in shape[:-2]:
            i = shape[:-2].index(1)
            shape = shape[:i] + shape[i + 1:]
        if len(shape) != 3:
            raise RuntimeError(
                f"Expected frames of shape [N, H*1.5, W] (extra dimensions of size 1 allowed). "
                f"Found: {tuple(frames.shape)}")
        n, h2, w = shape
        if h2 % 3:
            raise RuntimeError(
                f"The height of NV12 image (h*1.5) must be divisible by 3. Found: {h2}")
        h = h2 // 3 * 2
        plan = None
        if self._sparse and not (w % 2 or h % 2):
            plan = self._sparse_plan(st, n, w, h)
            if self._sparse == "auto" and plan["fraction"] >= 0.85:
                plan = None  # nearly every row is read: one copy per frame is cheaper
        elif self._sparse is True:
            raise RuntimeError(f"sparse_upload needs even frame sizes. Found: {w}x{h}")
        if plan is not None:
            host = np.ascontiguousarray(np.asarray(frames).reshape(shape))
            st["uploads"]["sparse"] += 1
            dev = self._upload(self._gather_rows(st, host, plan, w, h), cfg)
            result = convert_resize(dev, plan["descs"], out_size=plan["out"], max_src_w=w,
                                    device_config=cfg, row_maps=plan["maps"], sync=True,
                                    **self._opts, **self._resize_opts)
            tensor = to_torch(result, torch.bfloat16
                              if self._opts["dtype"] in ("bfloat16", "bf16") else None)
            if self._num_caches:
                st["cache"].append(tensor)
                st["cache"].pop(0)
            return tensor
        if isinstance(frames, CPUBuffer):
            view = CPUBuffer(shape, frames.elem_class, frames.depth, frames.storage)
        else:
            view = np.ascontiguousarray(frames).reshape(shape)
            if view.dtype == np.uint8 and view.nbytes:
                view = self._stage_whole(st, view)
        st["uploads"]["whole"] += 1
        dev = self._upload(view, cfg)
        if self._resizing:
            descs, out = self._descs_for(st, n, w, h)
            # sync=True waits for the stream once and checks the kernel's status word
            result = convert_resize(dev, descs, out_size=out, max_src_w=w, device_config=cfg,
                                    sync=True, **self._opts, **self._resize_opts)
        else:
            result = convert_nv12(dev, device_config=cfg, sync=True, **self._opts)
        tensor = to_torch(result, torch.bfloat16 if self._opts["dtype"] in ("bfloat16", "bf16")
                          else None)
        if self._num_caches:
            st["cache"].append(tensor)
            st["cache"].pop(0)
        return tensor
