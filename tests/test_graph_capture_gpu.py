"""The entry points only queue work on the caller's stream (no allocation, no synchronisation),
so a sequence of them can be captured into a CUDA graph and replayed."""

import ctypes

import numpy as np
import pytest

import oracle
from tests import synth

pytestmark = pytest.mark.gpu


def test_dense_resize_checksum_inside_a_cuda_graph(cuda_cfg):
    import torch

    import spdl_b200.io as io
    from spdl_b200 import _lib

    L = _lib.lib()
    n, w, h = 3, 320, 240
    nv = synth.nv12_batch(n, w, h, config=9, index=21)
    src = torch.from_numpy(nv).cuda()
    rgb = torch.zeros((n, h, w, 3), dtype=torch.uint8, device="cuda")
    small = torch.zeros((n, 3, 64, 64), dtype=torch.float32, device="cuda")
    sums = torch.zeros(n, dtype=torch.int64, device="cuda")
    descs, out = io.make_image_descs([w] * n, [h] * n, resize=(64, 64))
    dd = torch.from_numpy(descs.view(np.uint8)).cuda()

    a = _lib.DenseArgs()
    a.struct_size = ctypes.sizeof(_lib.DenseArgs)
    a.device = cuda_cfg.device_index
    a.y, a.u = src.data_ptr(), src.data_ptr() + h * w
    a.y_pitch = a.uv_pitch = w
    a.y_frame_stride = a.uv_frame_stride = h * 3 // 2 * w
    a.src_format, a.width, a.height, a.num_frames = _lib.NV12, w, h, n
    a.matrix_coeff, a.dst = 1, rgb.data_ptr()
    a.layout, a.dtype, a.order = _lib.NHWC, _lib.U8, _lib.RGB
    a.scale = (ctypes.c_float * 3)(1, 1, 1)

    r = _lib.ResizeArgs()
    r.struct_size = ctypes.sizeof(_lib.ResizeArgs)
    r.device, r.base, r.descs = cuda_cfg.device_index, src.data_ptr(), dd.data_ptr()
    r.num_images, r.src_format = n, _lib.NV12
    r.out_w, r.out_h = out
    r.matrix_coeff, r.full_range = 1, 0
    r.layout, r.dtype, r.order = _lib.NCHW, _lib.F32, _lib.RGB
    r.max_src_w, r.dst = w, small.data_ptr()
    r.scale = (ctypes.c_float * 3)(1, 1, 1)

    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph, stream=side):
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(L.b2_convert_dense(ctypes.byref(a), s))
        _lib.check(L.b2_convert_resize(ctypes.byref(r), s))
        _lib.check(L.b2_frame_checksum(rgb.data_ptr(), h * w * 3, n, sums.data_ptr(),
                                       cuda_cfg.device_index, s))
    # nothing ran during capture
    torch.cuda.synchronize()
    assert int(rgb.sum()) == 0 and int(sums.sum()) == 0

    want_rgb = oracle.nv12_to_planar(nv).transpose(0, 2, 3, 1)
    want_small = oracle.convert_resize(nv.reshape(-1), descs, out_w=64, out_h=64, dtype=oracle.F32)
    for rep in range(2):  # replay twice, with fresh input the second time
        if rep:
            nv = synth.nv12_batch(n, w, h, config=9, index=22)
            src.copy_(torch.from_numpy(nv).cuda())
            want_rgb = oracle.nv12_to_planar(nv).transpose(0, 2, 3, 1)
            want_small = oracle.convert_resize(nv.reshape(-1), descs, out_w=64, out_h=64,
                                               dtype=oracle.F32)
        graph.replay()
        torch.cuda.synchronize()
        assert (rgb.cpu().numpy() == want_rgb).all()
        np.testing.assert_allclose(small.cpu().numpy(), want_small, rtol=1e-6, atol=1e-5)
        assert sums.cpu().numpy().tolist() == [oracle.checksum(want_rgb[i]) for i in range(n)]
