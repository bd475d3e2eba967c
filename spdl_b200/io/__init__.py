"""``spdl.io``-compatible surface of the post-decode frame path (colour conversion, frame
batching, buffer transfer and the fused resize/crop/normalise) on hand-written sm_100a kernels."""

from ._convert import (ArrayInterface, CUDAArrayInterface, to_jax, to_numba, to_numpy,
                       to_torch)
from ._core import (DESC_DTYPE, FrameBatcher, check_resize_status, convert_nv12, convert_resize,
                    frame_checksum, make_image_descs, nv12_to_bgr, nv12_to_rgb,
                    resize_host_images, resize_image_list, synchronize_stream, touched_rows,
                    transfer_buffer, transfer_buffer_cpu)
from ._frames import Frames, convert_array, convert_frames
from ._stage import FrameStage
from ._transfer import transfer_tensor
from ._types import (CPUBuffer, CPUStorage, CUDABuffer, CUDAConfig, cpu_storage, cuda_buffer,
                     cuda_config)

__all__ = [
    "ArrayInterface", "CPUBuffer", "CPUStorage", "CUDAArrayInterface", "CUDABuffer", "CUDAConfig",
    "DESC_DTYPE", "FrameBatcher", "FrameStage", "Frames", "check_resize_status", "convert_array",
    "convert_frames", "convert_nv12", "convert_resize", "cpu_storage", "cuda_buffer",
    "cuda_config", "frame_checksum", "make_image_descs", "nv12_to_bgr", "nv12_to_rgb",
    "resize_host_images", "resize_image_list", "synchronize_stream", "to_jax", "to_numba",
    "to_numpy", "to_torch", "touched_rows", "transfer_buffer", "transfer_buffer_cpu",
    "transfer_tensor",
]
