"""The fields of ``b2_resize_args`` a plain ``convert_resize`` call does not exercise, through the
C ABI: strided and unaligned destinations with sentinels around every image, the device status
word and its three bits, letterbox padding, the channel-first clip layout, libswscale's
arithmetic, and callers built against version 1 of the struct."""

import ctypes

import numpy as np
import pytest

import oracle
from tests import synth

pytestmark = pytest.mark.gpu

MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
_O_DT = {"uint8": oracle.U8, "float32": oracle.F32, "bfloat16": oracle.BF16}
_ESZ = {"uint8": 1, "bfloat16": 2, "float32": 4}


def _dev(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _args(cfg, base, descs_dev, n, out, dst_ptr, *, fmt, layout, dtype, max_w, sb=None,
          coeff=1, full=0):
    from spdl_b200 import _lib

    a = _lib.ResizeArgs()
    a.struct_size = ctypes.sizeof(_lib.ResizeArgs)
    a.device, a.base, a.descs = cfg.device_index, base.data_ptr(), descs_dev.data_ptr()
    a.num_images, a.src_format = n, {"nv12": 0, "i420": 1, "rgb_planar": 2, "rgb24": 3}[fmt]
    a.out_w, a.out_h = out
    a.matrix_coeff, a.full_range = coeff, full
    a.layout = _lib.NCHW if layout == "NCHW" else _lib.NHWC
    a.dtype = {"uint8": _lib.U8, "bfloat16": _lib.BF16, "float32": _lib.F32}[dtype]
    a.order, a.max_src_w, a.dst = _lib.RGB, max_w, dst_ptr
    sb = oracle.scale_bias() if sb is None else sb
    a.scale = (ctypes.c_float * 3)(*[float(x) for x in sb[:3]])
    a.bias = (ctypes.c_float * 3)(*[float(x) for x in sb[3:]])
    return a


def _launch(a):
    import torch

    from spdl_b200 import _lib

    _lib.check(_lib.lib().b2_convert_resize(ctypes.byref(a),
                                            torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()


@pytest.mark.parametrize("layout", ["NCHW", "NHWC"])
@pytest.mark.parametrize("dtype", ["uint8", "bfloat16", "float32"])
@pytest.mark.parametrize("gap,dst_off,out", [(16, 0, (32, 24)), (7, 1, (32, 24)), (3, 2, (30, 17)),
                                             (0, 3, (33, 9))])
def test_strided_destination_with_sentinels(cuda_cfg, layout, dtype, gap, dst_off, out):
    """``dst_image_stride`` larger than an image, on aligned and unaligned element offsets:
    every image lands where the stride says and nothing before, between or after the images is
    written."""
    import torch

    import spdl_b200.io as io

    n, w, h = 3, 98, 50
    nv = synth.nv12_batch(n, w, h, config=9, index=gap)
    descs, _ = io.make_image_descs([w] * n, [h] * n, resize=out)
    esz = _ESZ[dtype]
    image = 3 * out[0] * out[1]
    stride = image + gap
    tdt = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[esz]
    sentinel = {1: 0xA5, 2: 0x5A5A, 4: 0x5A5A5A5A}[esz]
    buf = torch.full((dst_off + n * stride + 8,), sentinel, dtype=tdt, device="cuda")
    sb = oracle.scale_bias(MEAN, STD) if dtype != "uint8" else None
    base, dd = _dev(nv.reshape(-1)), _dev(descs.view(np.uint8))
    a = _args(cuda_cfg, base, dd, n, out, buf.data_ptr() + dst_off * esz, fmt="nv12",
              layout=layout, dtype=dtype, max_w=w, sb=sb)
    a.dst_image_stride = stride
    _launch(a)
    got = buf.cpu().numpy()
    want = oracle.convert_resize(nv.reshape(-1), descs, out_w=out[0], out_h=out[1],
                                 layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC,
                                 dtype=_O_DT[dtype], sb=sb)
    assert (got[:dst_off] == sentinel).all()
    for i in range(n):
        lo = dst_off + i * stride
        body = got[lo:lo + image]
        if dtype == "float32":
            np.testing.assert_allclose(body.view(np.float32), want[i].reshape(-1), rtol=1e-5,
                                       atol=1e-5)
        elif dtype == "bfloat16":
            assert (body.view(np.uint16) == want[i].reshape(-1)).mean() > 0.999
        else:
            assert (body == want[i].reshape(-1)).all()
        assert (got[lo + image:lo + stride] == sentinel).all()
    assert (got[dst_off + n * stride:] == sentinel).all()


def test_status_word_reports_an_image_wider_than_max_src_w(cuda_cfg):
    """A table whose second image is wider than ``max_src_w`` says: the kernel skips that image
    (it returns before touching shared memory), sets the status bit and converts the others."""
    import torch

    import spdl_b200.io as io
    from spdl_b200 import _lib

    ws, hs = [64, 200, 64], [48, 48, 48]
    sizes = [w * h * 3 // 2 for w, h in zip(ws, hs)]
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    data = np.random.default_rng(5).integers(0, 256, int(sum(sizes)), dtype=np.uint8)
    descs, out = io.make_image_descs(ws, hs, offsets=offs, resize=(32, 24))
    dst = torch.full((3, 3, 24, 32), 0xA5, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = _args(cuda_cfg, _dev(data), _dev(descs.view(np.uint8)), 3, out, dst.data_ptr(),
              fmt="nv12", layout="NCHW", dtype="uint8", max_w=64)
    a.status = status.data_ptr()
    _launch(a)
    assert int(status.item()) == _lib.STATUS_IMAGE_TOO_WIDE
    got = dst.cpu().numpy()
    want = oracle.convert_resize(data, descs, out_w=32, out_h=24)
    assert (got[1] == 0xA5).all()
    assert (got[0] == want[0]).all() and (got[2] == want[2]).all()
    # the Python wrapper turns the word into an exception when it waits for the stream ...
    with pytest.raises(RuntimeError, match="wider than max_src_w"):
        io.convert_resize(_dev(data), _dev(descs.view(np.uint8)), out_size=out, max_src_w=64,
                          device_config=cuda_cfg, sync=True)
    # ... and the word is clear again afterwards
    io.check_resize_status(cuda_cfg)
    io.convert_resize(_dev(data), _dev(descs.view(np.uint8)), out_size=out, max_src_w=200,
                      device_config=cuda_cfg, sync=True)
    # without a status word the call behaves as before: the image is skipped silently
    a.status = None
    dst.fill_(0x11)
    _launch(a)
    assert (dst.cpu().numpy()[1] == 0x11).all()


def test_status_word_reports_nonsensical_descriptors(cuda_cfg):
    """Empty sources, zero or negative or NaN scales: skipped and reported; the oracle leaves the
    same images untouched."""
    import torch

    import spdl_b200.io as io
    from spdl_b200 import _lib

    n, w, h = 5, 64, 48
    nv = synth.nv12_batch(n, w, h, config=9, index=77)
    descs, out = io.make_image_descs([w] * n, [h] * n, resize=(32, 24))
    descs["src_w"][0] = 0
    descs["scale_x"][1] = 0.0
    descs["scale_y"][2] = -1.5
    descs["scale_x"][3] = np.float32("nan")
    dst = torch.full((n, 3, 24, 32), 0xA5, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = _args(cuda_cfg, _dev(nv.reshape(-1)), _dev(descs.view(np.uint8)), n, out, dst.data_ptr(),
              fmt="nv12", layout="NCHW", dtype="uint8", max_w=w)
    a.status = status.data_ptr()
    _launch(a)
    assert int(status.item()) == _lib.STATUS_BAD_GEOMETRY
    want = oracle.convert_resize(nv.reshape(-1), descs, out_w=32, out_h=24,
                                 out=np.full((n, 3, 24, 32), 0xA5, np.uint8))
    assert (dst.cpu().numpy() == want).all()
    assert (want[:4] == 0xA5).all() and not (want[4] == 0xA5).all()


def test_huge_scales_stay_inside_the_image(cuda_cfg):
    """Scales far beyond anything a real geometry produces must not read outside the staged rows:
    taps are clamped into the image.  The result is whatever the clamped taps give; only
    completion without a fault and an untouched neighbourhood are checked."""
    import torch

    import spdl_b200.io as io

    n, w, h = 2, 64, 48
    nv = synth.nv12_batch(n, w, h, config=9, index=78)
    descs, out = io.make_image_descs([w] * n, [h] * n, resize=(32, 24))
    descs["scale_x"][0] = 3.0e9
    descs["scale_y"][1] = 1.0e30
    descs["crop_x"][1] = -1000  # every column maps to the first pixel
    buf = torch.full((16 + n * 3 * 24 * 32 + 16,), 0xA5, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = _args(cuda_cfg, _dev(nv.reshape(-1)), _dev(descs.view(np.uint8)), n, out,
              buf.data_ptr() + 16, fmt="nv12", layout="NCHW", dtype="uint8", max_w=w)
    a.status = status.data_ptr()
    _launch(a)
    got = buf.cpu().numpy()
    assert (got[:16] == 0xA5).all() and (got[-16:] == 0xA5).all()


def test_a_wait_that_runs_out_reports_and_returns(cuda_cfg):
    """``B2_DEBUG_EXPIRE_WAIT`` makes every tile wait, with a limit of a few polls, on a barrier
    that nothing completes (after its own copies have landed): the kernel must give up, set the
    status bit, leave the output alone and return, and the context must stay usable."""
    import torch

    import spdl_b200.io as io
    from spdl_b200 import _lib

    n, w, h = 4, 128, 72
    nv = synth.nv12_batch(n, w, h, config=9, index=79)
    descs, out = io.make_image_descs([w] * n, [h] * n, resize=(32, 32))
    dst = torch.full((n, 3, 32, 32), 0xA5, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    base, dd = _dev(nv.reshape(-1)), _dev(descs.view(np.uint8))
    a = _args(cuda_cfg, base, dd, n, out, dst.data_ptr(), fmt="nv12", layout="NCHW",
              dtype="uint8", max_w=w)
    a.status, a.debug_flags = status.data_ptr(), _lib.DEBUG_EXPIRE_WAIT
    _launch(a)
    assert int(status.item()) == _lib.STATUS_WAIT_EXPIRED
    assert (dst.cpu().numpy() == 0xA5).all()
    with pytest.raises(RuntimeError, match="wait for staged source rows ran out"):
        io.convert_resize(base, dd, out_size=out, max_src_w=w, device_config=cuda_cfg, sync=True,
                          _debug_flags=_lib.DEBUG_EXPIRE_WAIT)
    # the same call without the flag works right afterwards
    status.zero_()
    a.debug_flags = 0
    _launch(a)
    assert int(status.item()) == 0
    assert (dst.cpu().numpy() == oracle.convert_resize(nv.reshape(-1), descs, out_w=32,
                                                       out_h=32)).all()


@pytest.mark.parametrize("fmt", ["nv12", "i420", "rgb24"])
@pytest.mark.parametrize("layout,dtype", [("NCHW", "uint8"), ("NHWC", "float32"),
                                          ("NCHW", "bfloat16")])
def test_letterbox(cuda_cfg, fmt, layout, dtype):
    """``scale_mode="pad"``: wide, tall and square images on one square canvas; the bars take the
    pad colour through the same rounding / normalisation as image pixels."""
    import spdl_b200.io as io

    ws, hs = np.array([128, 60, 96, 250]), np.array([72, 150, 96, 40])
    yuv = fmt != "rgb24"
    sizes = ws * hs * 3 // 2 if yuv else 3 * ws * hs
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    data = np.random.default_rng(6).integers(0, 256, int(sizes.sum()), dtype=np.uint8)
    descs, out = io.make_image_descs(ws, hs, src_format=fmt, offsets=offs, resize=(64, 64),
                                     scale_mode="pad")
    assert out == (64, 64)
    assert [int(v) for v in descs["resized_h"]] == [36, 64, 64, 10]
    assert [int(v) for v in descs["crop_y"]] == [-14, 0, 0, -26 if yuv else -27]
    pad = (10.0, 128.0, 250.0)
    norm = dict(mean=MEAN, std=STD) if dtype != "uint8" else {}
    buf = io.convert_resize(_dev(data), _dev(descs.view(np.uint8)), out_size=out, max_src_w=250,
                            device_config=cuda_cfg, src_format=fmt, layout=layout, dtype=dtype,
                            pad_color=pad, sync=True, **norm)
    got = io.to_torch(buf).cpu().numpy()
    ofmt = {"nv12": oracle.NV12, "i420": oracle.I420, "rgb24": oracle.RGBI}[fmt]
    want = oracle.convert_resize(data, descs, out_w=64, out_h=64, src_format=ofmt,
                                 layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC,
                                 dtype=_O_DT[dtype], pad_value=pad,
                                 sb=oracle.scale_bias(MEAN, STD) if norm else None)
    if dtype == "uint8":
        assert (got == want).all()
        assert (got[0, :, 0, 0] == np.array(pad, np.uint8)).all()  # top bar of the wide image
        assert (got[1, :, 32, 0] == np.array(pad, np.uint8)).all()  # left bar of the tall image
    elif dtype == "float32":
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    else:
        assert (got.view(np.uint16) == want).mean() > 0.999


def test_channel_first_clip_layout(cuda_cfg):
    """``clip_frames=T`` writes ``[N/T, 3, T, H, W]`` directly: equal to the frame-major result
    permuted, as examples/video_classification/utils/pipeline.py:137 does on the host side."""
    import spdl_b200.io as io

    clips, t, w, h = 3, 4, 128, 72
    frames = np.concatenate([synth.nv12_clip(t, w, h, config=4, index=i) for i in range(clips)])
    descs, out = io.make_image_descs([w] * clips * t, [h] * clips * t, resize=(40, 24))
    base, dd = _dev(frames.reshape(-1)), _dev(descs.view(np.uint8))
    for dtype in ("uint8", "float32"):
        flat = io.to_torch(io.convert_resize(base, dd, out_size=out, max_src_w=w, coeff=6,
                                             device_config=cuda_cfg, dtype=dtype,
                                             sync=True)).cpu().numpy()
        cthw = io.to_torch(io.convert_resize(base, dd, out_size=out, max_src_w=w, coeff=6,
                                             device_config=cuda_cfg, dtype=dtype, clip_frames=t,
                                             sync=True)).cpu().numpy()
        assert cthw.shape == (clips, 3, t, 24, 40)
        assert (cthw == flat.reshape(clips, t, 3, 24, 40).transpose(0, 2, 1, 3, 4)).all()
        want = oracle.convert_resize(frames.reshape(-1), descs, out_w=40, out_h=24, coeff=6,
                                     dtype=_O_DT[dtype], clip_frames=t)
        if dtype == "uint8":
            assert (cthw == want).all()
        else:
            np.testing.assert_allclose(cthw, want, rtol=1e-5, atol=1e-5)
    with pytest.raises(RuntimeError):
        io.convert_resize(base, dd, out_size=out, max_src_w=w, device_config=cuda_cfg,
                          clip_frames=5)
    with pytest.raises(RuntimeError):
        io.convert_resize(base, dd, out_size=out, max_src_w=w, device_config=cuda_cfg,
                          clip_frames=t, layout="NHWC")


@pytest.mark.parametrize("fmt", ["nv12", "i420"])
@pytest.mark.parametrize("coeff,full", [(1, False), (5, True)])
def test_resize_with_libswscale_arithmetic(cuda_cfg, fmt, coeff, full):
    import spdl_b200.io as io

    n, w, h = 3, 320, 180
    nv = synth.nv12_batch(n, w, h, config=9, index=coeff, full_range=full)
    descs, out = io.make_image_descs([w] * n, [h] * n, src_format=fmt, resize=(96, 64))
    buf = io.convert_resize(_dev(nv.reshape(-1)), _dev(descs.view(np.uint8)), out_size=out,
                            max_src_w=w, device_config=cuda_cfg, src_format=fmt, coeff=coeff,
                            full_range=full, arith="swscale", sync=True)
    want = oracle.convert_resize(nv.reshape(-1), descs, out_w=96, out_h=64,
                                 src_format=oracle.NV12 if fmt == "nv12" else oracle.I420,
                                 coeff=coeff, full_range=full, arith=oracle.ARITH_SWSCALE)
    assert (io.to_torch(buf).cpu().numpy() == want).all()
    ref = oracle.convert_resize(nv.reshape(-1), descs, out_w=96, out_h=64,
                                src_format=oracle.NV12 if fmt == "nv12" else oracle.I420,
                                coeff=coeff, full_range=full)
    assert not (want == ref).all()  # the two arithmetics are not the same function


def test_callers_built_against_version_1_of_the_structs(cuda_cfg):
    """``struct_size`` of the first ABI version (104 / 168 bytes) is still accepted and means
    zeros for every later field, whatever bytes follow in the caller's memory."""
    import torch

    import spdl_b200.io as io
    from spdl_b200 import _lib

    n, w, h = 2, 64, 48
    nv = synth.nv12_batch(n, w, h, config=9, index=80)
    descs, out = io.make_image_descs([w] * n, [h] * n, resize=(32, 24))
    dst = torch.zeros((n, 3, 24, 32), dtype=torch.uint8, device="cuda")
    src = _dev(nv.reshape(-1))
    a = _args(cuda_cfg, src, _dev(descs.view(np.uint8)), n, out, dst.data_ptr(),
              fmt="nv12", layout="NCHW", dtype="uint8", max_w=w)
    a.struct_size = _lib.ResizeArgs.arith.offset
    a.arith, a.frames_per_group, a.debug_flags, a.status = 77, -5, 99, 0xDEAD0000  # never read
    _launch(a)
    assert (dst.cpu().numpy() == oracle.convert_resize(nv.reshape(-1), descs, out_w=32,
                                                       out_h=24)).all()
    a.struct_size = 50
    assert _lib.lib().b2_convert_resize(ctypes.byref(a), None) == 1

    d = _lib.DenseArgs()
    d.struct_size = _lib.DenseArgs.arith.offset
    d.device = cuda_cfg.device_index
    d.y, d.u = src.data_ptr(), src.data_ptr() + h * w
    d.y_pitch = d.uv_pitch = w
    d.y_frame_stride = d.uv_frame_stride = h * 3 // 2 * w
    d.src_format, d.width, d.height, d.num_frames = _lib.NV12, w, h, n
    d.matrix_coeff = 1
    full = torch.zeros((n, 3, h, w), dtype=torch.uint8, device="cuda")
    d.dst, d.layout, d.dtype, d.order = full.data_ptr(), _lib.NCHW, _lib.U8, _lib.RGB
    d.scale = (ctypes.c_float * 3)(1, 1, 1)
    d.reserved0, d.arith = 12345, 1  # bytes past the version-1 struct
    _lib.check(_lib.lib().b2_convert_dense(ctypes.byref(d),
                                           torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert (full.cpu().numpy() == oracle.nv12_to_planar(nv)).all()


@pytest.mark.parametrize("fmt", ["nv12", "i420"])
@pytest.mark.parametrize("src,geom", [((1280, 720), dict(resize=(256, 256))),
                                      ((640, 360), dict(resize_shorter=96, crop=(80, 80))),
                                      ((320, 180), dict(resize=(64, 64), scale_mode="pad")),
                                      ((96, 64), dict(resize=(200, 150)))])
def test_row_sparse_sources_equal_whole_frames(cuda_cfg, fmt, src, geom):
    """Only the rows a geometry reads are stored (back to back) and found through the row maps:
    the result equals the conversion of the whole frames, bit for bit."""
    import spdl_b200.io as io

    n, (w, h) = 3, src
    frames = synth.nv12_batch(n, w, h, config=9, index=w + h)
    table, out = io.make_image_descs([w] * n, [h] * n, src_format=fmt, **geom)
    dense = io.to_torch(io.convert_resize(_dev(frames.reshape(-1)), _dev(table.view(np.uint8)),
                                          out_size=out, max_src_w=w, device_config=cuda_cfg,
                                          src_format=fmt, pad_color=(9, 99, 199),
                                          sync=True)).cpu().numpy()
    luma, chroma = io.touched_rows(table[0], src_format=fmt, out_h=out[1])
    lrows, crows = np.flatnonzero(luma >= 0), np.flatnonzero(chroma >= 0)
    cw = w if fmt == "nv12" else w // 2
    packed = []
    for f in frames:
        parts = [f[:h][lrows].reshape(-1)]
        if fmt == "nv12":
            parts.append(f[h:][crows].reshape(-1))
        else:
            flat, blk = f.reshape(-1), (h // 2) * cw
            for k in range(2):
                plane = flat[h * w + k * blk:h * w + (k + 1) * blk].reshape(h // 2, cw)
                parts.append(plane[crows].reshape(-1))
        packed.append(np.concatenate(parts))
    fb = packed[0].size
    assert fb < h * w * 3 // 2 or w == 96  # the upscaling case reads every row
    sparse_table = table.copy()
    sparse_table["y_off"] = np.arange(n, dtype=np.uint64) * fb
    sparse_table["u_off"] = sparse_table["y_off"] + len(lrows) * w
    if fmt == "i420":
        sparse_table["v_off"] = sparse_table["u_off"] + len(crows) * cw
    got = io.to_torch(io.convert_resize(
        _dev(np.concatenate(packed)), _dev(sparse_table.view(np.uint8)), out_size=out, max_src_w=w,
        device_config=cuda_cfg, src_format=fmt, pad_color=(9, 99, 199),
        row_maps=(_dev(luma), _dev(chroma)), sync=True)).cpu().numpy()
    assert (got == dense).all()


def test_a_row_map_with_a_hole_is_reported_not_followed(cuda_cfg):
    import spdl_b200.io as io

    n, w, h = 2, 128, 72
    frames = synth.nv12_batch(n, w, h, config=9, index=3)
    table, out = io.make_image_descs([w] * n, [h] * n, resize=(32, 32))
    luma, chroma = io.touched_rows(table[0], src_format="nv12", out_h=32)
    luma = np.arange(h, dtype=np.int32)      # whole frames are on the device ...
    chroma = np.arange(h // 2, dtype=np.int32)
    luma[int(np.flatnonzero(io.touched_rows(table[0], src_format="nv12", out_h=32)[0] >= 0)[5])] = -1
    with pytest.raises(RuntimeError, match="descriptor"):  # ... but the map denies a needed row
        io.convert_resize(_dev(frames.reshape(-1)), _dev(table.view(np.uint8)), out_size=out,
                          max_src_w=w, device_config=cuda_cfg, row_maps=(_dev(luma), _dev(chroma)),
                          sync=True)
    io.check_resize_status(cuda_cfg)  # the word is clear again


def test_frame_stage_sparse_upload_equals_whole_frames():
    import torch

    import spdl_b200.io as io

    for fmt, (w, h) in (("nv12", (640, 360)), ("i420", (320, 240))):
        frames = synth.nv12_batch(4, w, h, config=9, index=w)
        kw = dict(src_format=fmt, dtype="float32", mean=MEAN, std=STD, resize_shorter=96,
                  crop=(80, 80))
        whole = io.FrameStage(**kw)(frames)
        sparse = io.FrameStage(sparse_upload=True, **kw)
        a = sparse(frames)
        b = sparse(frames[:2])  # another batch size: a second plan
        assert torch.equal(a, whole) and torch.equal(b, whole[:2])
    with pytest.raises(RuntimeError):
        io.FrameStage(sparse_upload=True)
    # "auto": sparse for a geometry that reads a small part of the frame, whole frames otherwise
    frames = synth.nv12_batch(2, 640, 360, config=9, index=5)
    for geom, expect_sparse in ((dict(resize=(64, 40)), True), (dict(resize=(320, 300)), False)):
        auto = io.FrameStage(src_format="nv12", dtype="uint8", sparse_upload="auto", **geom)
        whole = io.FrameStage(src_format="nv12", dtype="uint8", **geom)
        assert torch.equal(auto(frames), whole(frames))
        assert auto._state()["uploads"] == ({"sparse": 1, "whole": 0} if expect_sparse
                                            else {"sparse": 0, "whole": 1})
