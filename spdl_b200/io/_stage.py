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

from ._convert import to_torch
from ._core import convert_nv12, convert_resize, make_image_descs, transfer_buffer
from ._types import CPUBuffer, CUDAConfig, cuda_config

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
    """

    def __init__(self, *, src_format: str = "i420", layout: str = "NCHW", dtype: str = "float32",
                 order: str = "rgb", coeff: int = 1, full_range: bool = False, mean=None, std=None,
                 resize: tuple[int, int] | None = None, resize_shorter: int | None = None,
                 crop: tuple[int, int] | None = None, scale_mode: str | None = None,
                 pad_color: tuple[float, float, float] = (0.0, 0.0, 0.0),
                 clip_frames: int | None = None, arith: str = "reference", num_caches: int = 4,
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
                  "cache": [None] * self._num_caches, "descs": {}}
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
        if isinstance(frames, CPUBuffer):
            view = CPUBuffer(shape, frames.elem_class, frames.depth, frames.storage)
        else:
            view = np.ascontiguousarray(frames).reshape(shape)
        dev = transfer_buffer(view, device_config=cfg)
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
