"""Frames whose rows start on arbitrary byte boundaries (widths that are not a multiple of 16,
sources and destinations at odd offsets): the kernel for packed frames of any even width and the
any-alignment kernel against the oracle, at real-world sizes and at sizes of a chunk or two."""

import numpy as np
import pytest

import oracle
from tests import synth

pytestmark = pytest.mark.gpu

MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)


@pytest.mark.parametrize("w,h", [(854, 480), (426, 240), (1918, 20), (1366, 18), (30, 6), (16, 2),
                                 (18, 4), (22, 12), (46, 6), (130, 10), (8, 4), (4, 2), (46, 64),
                                 (18, 160), (130, 40)])
@pytest.mark.parametrize("fmt", ["nv12", "i420"])
@pytest.mark.parametrize("layout,dtype", [("NCHW", "uint8"), ("NHWC", "uint8"),
                                          ("NHWC", "bfloat16"), ("NCHW", "float32")])
def test_unaligned_widths(cuda_cfg, w, h, fmt, layout, dtype):
    import torch

    import spdl_b200.io as io

    n = 2
    nv = synth.nv12_batch(n, w, h, config=9, index=w, full_range=True)
    norm = dict(mean=MEAN, std=STD) if dtype != "uint8" else {}
    # one byte of offset in front makes even the first row start on an odd address
    raw = torch.zeros(nv.size + 1, dtype=torch.uint8, device="cuda")
    raw[1:] = torch.from_numpy(nv.reshape(-1)).cuda()
    dev = raw[1:].view(n, h * 3 // 2, w)
    got = io.to_torch(io.convert_nv12(dev, device_config=cuda_cfg, src_format=fmt, layout=layout,
                                      dtype=dtype, order="bgr", sync=True, **norm)).cpu().numpy()
    flat = nv.reshape(-1)
    h2 = h * 3 // 2
    if fmt == "nv12":
        u, v, up = flat[h * w:], None, w
    else:
        u, v, up = flat[h * w:], flat[h * w + (h // 2) * (w // 2):], w // 2
    want = oracle.convert_dense(
        nv, u, v, width=w, height=h, num_frames=n, y_pitch=w, uv_pitch=up, y_frame_stride=h2 * w,
        uv_frame_stride=h2 * w, src_format=oracle.NV12 if fmt == "nv12" else oracle.I420,
        layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC,
        dtype={"uint8": oracle.U8, "float32": oracle.F32, "bfloat16": oracle.BF16}[dtype],
        order=oracle.BGR, sb=oracle.scale_bias(MEAN, STD) if norm else None)
    if dtype == "uint8":
        assert (got == want).all()
    elif dtype == "float32":
        np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)
    else:
        assert (got.view(np.uint16) == want).all()


@pytest.mark.parametrize("w,h", [(31, 6), (854, 10), (1918, 4), (50, 8)])
@pytest.mark.parametrize("layout", ["NCHW", "NHWC"])
@pytest.mark.parametrize("dtype", ["uint8", "bfloat16", "float32"])
@pytest.mark.parametrize("dst_off", [1, 2, 6])
def test_destination_on_odd_elements(cuda_cfg, w, h, layout, dtype, dst_off):
    """Through the C ABI with a destination that starts ``dst_off`` elements into its buffer
    (odd offsets and odd widths: the any-alignment kernel; even ones: the kernel for packed
    frames).  The bytes around the output and the trailing odd column keep their sentinel value."""
    import ctypes

    import torch

    from spdl_b200 import _lib

    n = 2
    esz = {"uint8": 1, "bfloat16": 2, "float32": 4}[dtype]
    tdt = {"uint8": torch.uint8, "bfloat16": torch.int16, "float32": torch.int32}[dtype]
    nv = synth.nv12_batch(n, w, h, config=9, index=w + dst_off, full_range=True)
    src = torch.from_numpy(nv).cuda()
    total = n * 3 * h * w
    sentinel = {1: 0xA5, 2: 0x5A5A, 4: 0x5A5A5A5A}[esz]
    buf = torch.full((total + 8,), sentinel, dtype=tdt, device="cuda")
    a = _lib.DenseArgs()
    a.struct_size = ctypes.sizeof(_lib.DenseArgs)
    a.device = cuda_cfg.device_index
    a.y, a.u = src.data_ptr(), src.data_ptr() + h * w
    a.y_pitch = a.uv_pitch = w
    a.y_frame_stride = a.uv_frame_stride = h * 3 // 2 * w
    a.src_format, a.width, a.height, a.num_frames = _lib.NV12, w, h, n
    a.matrix_coeff, a.full_range = 6, 1
    a.dst = buf.data_ptr() + dst_off * esz
    a.layout = _lib.NCHW if layout == "NCHW" else _lib.NHWC
    a.dtype = {"uint8": _lib.U8, "bfloat16": _lib.BF16, "float32": _lib.F32}[dtype]
    a.order = _lib.RGB
    sb = oracle.scale_bias(MEAN, STD) if dtype != "uint8" else oracle.scale_bias()
    a.scale = (ctypes.c_float * 3)(*[float(x) for x in sb[:3]])
    a.bias = (ctypes.c_float * 3)(*[float(x) for x in sb[3:]])
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib().b2_convert_dense(ctypes.byref(a), stream))
    torch.cuda.synchronize()
    got = buf.cpu().numpy()
    want = oracle.convert_dense(
        nv, nv.reshape(-1)[h * w:], None, width=w, height=h, num_frames=n, y_pitch=w, uv_pitch=w,
        y_frame_stride=h * 3 // 2 * w, uv_frame_stride=h * 3 // 2 * w, src_format=oracle.NV12,
        layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC,
        dtype={"uint8": oracle.U8, "float32": oracle.F32, "bfloat16": oracle.BF16}[dtype],
        coeff=6, full_range=True, sb=sb)
    shape = (n, 3, h, w) if layout == "NCHW" else (n, h, w, 3)
    body = got[dst_off:dst_off + total].reshape(shape)
    we = w & ~1
    cols = (slice(None),) * 3 + (slice(0, we),) if layout == "NCHW" else \
        (slice(None), slice(None), slice(0, we))
    if dtype == "uint8":
        assert (body[cols] == want[cols]).all()
    elif dtype == "bfloat16":
        assert (body[cols].view(np.uint16) == want[cols]).all()
    else:
        np.testing.assert_allclose(body[cols].view(np.float32), want[cols], rtol=1e-6, atol=1e-6)
    # nothing outside the even-width part of the frames was written
    assert (got[:dst_off] == sentinel).all() and (got[dst_off + total:] == sentinel).all()
    if w & 1:
        tail = body[..., w - 1] if layout == "NCHW" else body[:, :, w - 1, :]
        assert (tail == sentinel).all()


@pytest.mark.parametrize("w", [64, 50])
@pytest.mark.parametrize("src_pad", [0, 16, 6])
@pytest.mark.parametrize("dst_gap", [0, 16, 7])
@pytest.mark.parametrize("layout", ["NCHW", "NHWC"])
def test_pitched_source_and_strided_destination(cuda_cfg, w, src_pad, dst_gap, layout):
    """Source rows with a pitch wider than the row and frames spaced apart in the destination
    (``dst_frame_stride``), aligned and not: results equal the packed case and the padding keeps
    its sentinel value."""
    import ctypes

    import torch

    from spdl_b200 import _lib

    n, h = 3, 12
    h2 = h * 3 // 2
    pitch = w + src_pad
    nv = synth.nv12_batch(n, w, h, config=9, index=w + src_pad + dst_gap)
    pitched = np.full((n, h2, pitch), 0x77, np.uint8)
    pitched[:, :, :w] = nv
    src = torch.from_numpy(pitched).cuda()
    frame = 3 * h * w
    stride = frame + dst_gap
    buf = torch.full((n * stride + 16,), 0xA5, dtype=torch.uint8, device="cuda")
    a = _lib.DenseArgs()
    a.struct_size = ctypes.sizeof(_lib.DenseArgs)
    a.device = cuda_cfg.device_index
    a.y, a.u = src.data_ptr(), src.data_ptr() + h * pitch
    a.y_pitch = a.uv_pitch = pitch
    a.y_frame_stride = a.uv_frame_stride = h2 * pitch
    a.src_format, a.width, a.height, a.num_frames = _lib.NV12, w, h, n
    a.matrix_coeff = 1
    a.dst, a.dst_frame_stride = buf.data_ptr(), stride
    a.layout = _lib.NCHW if layout == "NCHW" else _lib.NHWC
    a.dtype, a.order = _lib.U8, _lib.BGR
    a.scale = (ctypes.c_float * 3)(1, 1, 1)
    _lib.check(_lib.lib().b2_convert_dense(ctypes.byref(a), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    got = buf.cpu().numpy()
    want = oracle.convert_dense(
        nv, nv.reshape(-1)[h * w:], None, width=w, height=h, num_frames=n, y_pitch=w, uv_pitch=w,
        y_frame_stride=h2 * w, uv_frame_stride=h2 * w, src_format=oracle.NV12,
        layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC, order=oracle.BGR)
    for i in range(n):
        assert (got[i * stride:i * stride + frame] == want[i].reshape(-1)).all()
        assert (got[i * stride + frame:(i + 1) * stride] == 0xA5).all()
    assert (got[n * stride:] == 0xA5).all()
