"""Seeded random sweeps over shapes and options, CUDA path against the oracle.

The fixed cases elsewhere pin known shapes; these walk the option space (format, layout, dtype,
channel order, matrix, range, odd and unaligned sizes, up- and down-scaling, crops) with one seed
per case so a failure can be replayed.
"""

import os

import numpy as np
import pytest

import oracle
from tests import synth

pytestmark = pytest.mark.gpu

MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
_O_DT = {"uint8": oracle.U8, "float32": oracle.F32, "bfloat16": oracle.BF16}
_O_FMT = {"nv12": oracle.NV12, "i420": oracle.I420, "rgb_planar": oracle.RGBP, "rgb24": oracle.RGBI}
_O_ARITH = {"reference": oracle.ARITH_REFERENCE, "swscale": oracle.ARITH_SWSCALE}


def _dev(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _check(got, want, dtype):
    assert got.shape == want.shape
    if dtype == "uint8":
        assert (got == want).all()
    elif dtype == "float32":
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    else:
        assert (got.view(np.uint16) == want).mean() > 0.999
        np.testing.assert_allclose(oracle.bf16_to_f32(got.view(np.uint16)),
                                   oracle.bf16_to_f32(want), rtol=2 ** -7, atol=1e-6)


@pytest.mark.parametrize("seed", range(64))
def test_dense_random_cases(cuda_cfg, seed):
    import spdl_b200.io as io

    r = np.random.default_rng(7000 + seed)
    fmt = str(r.choice(["nv12", "i420"]))
    layout = str(r.choice(["NCHW", "NHWC"]))
    dtype = str(r.choice(["uint8", "float32", "bfloat16"]))
    order = str(r.choice(["rgb", "bgr"]))
    coeff = int(r.choice([1, 4, 5, 6, 7, 9, 10]))
    full = bool(r.integers(0, 2))
    n = int(r.integers(1, 5))
    # widths that hit the vector path (multiples of 16/8/4) and the any-shape path
    w = int(r.choice([16, 32, 48, 64, 200, 328, 1000, 18, 22, 50, 2, 854, 426, 130])) \
        if fmt == "nv12" else int(r.choice([16, 32, 64, 200, 328, 18, 50, 2, 854, 426, 130]))
    h = int(r.integers(1, 20)) * 2
    nv = synth.nv12_batch(n, w, h, config=9, index=seed, full_range=True)
    norm = dict(mean=MEAN, std=STD) if dtype != "uint8" and r.integers(0, 2) else {}
    arith = str(r.choice(["reference", "swscale"]))
    got = io.to_torch(io.convert_nv12(_dev(nv), device_config=cuda_cfg, src_format=fmt,
                                      layout=layout, dtype=dtype, order=order, coeff=coeff,
                                      full_range=full, arith=arith, sync=True,
                                      **norm)).cpu().numpy()
    flat = nv.reshape(-1)
    h2 = h * 3 // 2
    if fmt == "nv12":
        u, v, up = flat[h * w:], None, w
    else:
        u, v, up = flat[h * w:], flat[h * w + (h // 2) * (w // 2):], w // 2
    want = oracle.convert_dense(
        nv, u, v, width=w, height=h, num_frames=n, y_pitch=w, uv_pitch=up, y_frame_stride=h2 * w,
        uv_frame_stride=h2 * w, src_format=_O_FMT[fmt],
        layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC, dtype=_O_DT[dtype],
        order=oracle.RGB if order == "rgb" else oracle.BGR, coeff=coeff, full_range=full,
        sb=oracle.scale_bias(MEAN, STD) if norm else None, arith=_O_ARITH[arith])
    _check(got, want, dtype)


@pytest.mark.parametrize("seed", range(64))
def test_resize_random_cases(cuda_cfg, seed):
    import spdl_b200.io as io

    r = np.random.default_rng(9000 + seed)
    fmt = str(r.choice(["nv12", "i420", "rgb_planar", "rgb24"]))
    layout = str(r.choice(["NCHW", "NHWC"]))
    dtype = str(r.choice(["uint8", "float32", "bfloat16"]))
    order = str(r.choice(["rgb", "bgr"]))
    coeff = int(r.choice([1, 6, 9]))
    full = bool(r.integers(0, 2))
    n = int(r.integers(1, 7))
    ws = r.integers(8, 300, n)
    hs = r.integers(8, 300, n)
    if fmt in ("nv12", "i420") and r.integers(0, 2):
        ws, hs = ws & ~1, hs & ~1  # even sizes half of the time, odd ones otherwise
    yuv = fmt in ("nv12", "i420")
    sizes = ws * hs + 2 * ((ws + 1) // 2) * ((hs + 1) // 2) if yuv else 3 * ws * hs
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    data = r.integers(0, 256, int(sizes.sum()), dtype=np.uint8)
    mode = int(r.integers(0, 5))
    pad = (0.0, 0.0, 0.0)
    if mode >= 3:      # keep the aspect ratio: letterbox (3) or cover and crop (4)
        geom = dict(resize=(int(r.integers(2, 140)), int(r.integers(2, 140))),
                    scale_mode="pad" if mode == 3 else "crop")
        pad = tuple(float(v) for v in r.integers(0, 256, 3))
    elif mode == 0:    # stretch to a fixed size (up- or down-scaling)
        geom = dict(resize=(int(r.integers(1, 120)), int(r.integers(1, 120))))
    elif mode == 1:    # shorter side + centre crop
        s = int(r.integers(8, 100))
        c = int(r.integers(1, s + 1))
        geom = dict(resize_shorter=s, crop=(c, int(r.integers(1, s + 1))))
    else:              # fixed size + crop
        rw, rh = int(r.integers(8, 150)), int(r.integers(8, 150))
        geom = dict(resize=(rw, rh), crop=(int(r.integers(1, rw + 1)), int(r.integers(1, rh + 1))))
    descs, out = io.make_image_descs(ws, hs, src_format=fmt, offsets=offs, **geom)
    norm = dict(mean=MEAN, std=STD) if dtype != "uint8" and r.integers(0, 2) else {}
    arith = str(r.choice(["reference", "swscale"]))
    buf = io.convert_resize(_dev(data), _dev(descs.view(np.uint8)), out_size=out,
                            max_src_w=int(ws.max()), device_config=cuda_cfg, src_format=fmt,
                            coeff=coeff, full_range=full, layout=layout, dtype=dtype, order=order,
                            arith=arith, pad_color=pad, sync=True, **norm)
    got = io.to_torch(buf).cpu().numpy()
    want = oracle.convert_resize(
        data, descs, out_w=out[0], out_h=out[1], src_format=_O_FMT[fmt], coeff=coeff,
        full_range=full, layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC,
        dtype=_O_DT[dtype], order=oracle.RGB if order == "rgb" else oracle.BGR,
        sb=oracle.scale_bias(MEAN, STD) if norm else None, arith=_O_ARITH[arith], pad_value=pad)
    _check(got, want, dtype)


@pytest.mark.skipif(not os.environ.get("B2_FUZZ_SWEEP"),
                    reason="set B2_FUZZ_SWEEP=first:last to run the long sweep")
def test_long_sweep(cuda_cfg):
    """The two sweeps above over an arbitrary seed range, e.g. ``B2_FUZZ_SWEEP=64:30000`` (about
    0.7 ms per case on a B200)."""
    first, last = (int(v) for v in os.environ["B2_FUZZ_SWEEP"].split(":"))
    for seed in range(first, last):
        test_dense_random_cases(cuda_cfg, seed)
        test_resize_random_cases(cuda_cfg, seed)
        test_dense_random_memory_layouts(cuda_cfg, seed)
        if seed % 16 == 0:
            _dense_memory_layout_case(cuda_cfg, seed, larger=True)


@pytest.mark.parametrize("seed", range(48))
def test_dense_random_memory_layouts(cuda_cfg, seed):
    """Through the C ABI with surfaces at random byte offsets behind a pointer table or a random
    source pitch, and a destination at a random element offset with a random frame stride: every
    alignment path of the dense kernels against the oracle, with sentinel checks around the
    output."""
    _dense_memory_layout_case(cuda_cfg, seed, larger=False)


@pytest.mark.parametrize("seed", range(32))
def test_dense_random_memory_layouts_larger_frames(cuda_cfg, seed):
    """The same with frames of tens to a hundred rows and widths up to 1400: enough rows for the
    kernels' unchecked interior paths, row ends inside a warp's run of pixels, several warps per
    row."""
    _dense_memory_layout_case(cuda_cfg, 500 + seed, larger=True)


def _dense_memory_layout_case(cuda_cfg, seed, larger):
    import ctypes

    import torch

    from spdl_b200 import _lib

    r = np.random.default_rng(12000 + seed)
    n = int(r.integers(1, 4))
    if larger:
        w = int(r.integers(16, 1400))
        h = int(r.integers(9, 60)) * 2
    else:
        w = int(r.choice([16, 32, 48, 64, 100, 130, 200, 31, 854]))
        h = int(r.integers(1, 9)) * 2
    h2 = h * 3 // 2
    layout = str(r.choice(["NCHW", "NHWC"]))
    dtype = str(r.choice(["uint8", "float32", "bfloat16"]))
    esz = {"uint8": 1, "bfloat16": 2, "float32": 4}[dtype]
    table = bool(r.integers(0, 2))
    pitch = w + int(r.choice([0, 0, 16, 6, 1]))
    nv = synth.nv12_batch(n, w, h, config=9, index=seed, full_range=True)
    pitched = np.full((n, h2, pitch), 0x33, np.uint8)
    pitched[:, :, :w] = nv
    a = _lib.DenseArgs()
    a.struct_size = ctypes.sizeof(_lib.DenseArgs)
    a.device = cuda_cfg.device_index
    keep = []
    if table:
        ptrs = []
        for i in range(n):
            off = int(r.integers(0, 16))
            t = torch.zeros(h2 * pitch + 32, dtype=torch.uint8, device="cuda")
            t[off:off + h2 * pitch] = torch.from_numpy(pitched[i].reshape(-1)).cuda()
            keep.append(t)
            ptrs.append(t.data_ptr() + off)
        ytab = torch.tensor(ptrs, dtype=torch.int64, device="cuda")
        utab = ytab + h * pitch
        keep += [ytab, utab]
        a.y_table, a.u_table = ytab.data_ptr(), utab.data_ptr()
    else:
        off = int(r.integers(0, 16))
        t = torch.zeros(pitched.size + 32, dtype=torch.uint8, device="cuda")
        t[off:off + pitched.size] = torch.from_numpy(pitched.reshape(-1)).cuda()
        keep.append(t)
        a.y, a.u = t.data_ptr() + off, t.data_ptr() + off + h * pitch
        a.y_frame_stride = a.uv_frame_stride = h2 * pitch
    a.y_pitch = a.uv_pitch = pitch
    a.src_format, a.width, a.height, a.num_frames = _lib.NV12, w, h, n
    a.matrix_coeff, a.full_range = 1, int(r.integers(0, 2))
    a.arith = int(r.integers(0, 2))
    frame = 3 * h * w
    stride = frame + int(r.choice([0, 0, 16, 7, 2]))
    dst_off = int(r.integers(0, 4))
    tdt = {"uint8": torch.uint8, "bfloat16": torch.int16, "float32": torch.int32}[dtype]
    sentinel = {1: 0xA5, 2: 0x5A5A, 4: 0x5A5A5A5A}[esz]
    buf = torch.full((dst_off + n * stride + 8,), sentinel, dtype=tdt, device="cuda")
    a.dst, a.dst_frame_stride = buf.data_ptr() + dst_off * esz, stride
    a.layout = _lib.NCHW if layout == "NCHW" else _lib.NHWC
    a.dtype = {"uint8": _lib.U8, "bfloat16": _lib.BF16, "float32": _lib.F32}[dtype]
    a.order = _lib.RGB
    sb = oracle.scale_bias(MEAN, STD) if dtype != "uint8" else oracle.scale_bias()
    a.scale = (ctypes.c_float * 3)(*[float(x) for x in sb[:3]])
    a.bias = (ctypes.c_float * 3)(*[float(x) for x in sb[3:]])
    _lib.check(_lib.lib().b2_convert_dense(ctypes.byref(a), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    got = buf.cpu().numpy()
    want = oracle.convert_dense(
        nv, nv.reshape(-1)[h * w:], None, width=w, height=h, num_frames=n, y_pitch=w, uv_pitch=w,
        y_frame_stride=h2 * w, uv_frame_stride=h2 * w, src_format=oracle.NV12,
        layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC, dtype=_O_DT[dtype],
        full_range=bool(a.full_range), sb=sb, arith=int(a.arith))
    we = w & ~1
    shape = (3, h, w) if layout == "NCHW" else (h, w, 3)
    cols = (slice(None), slice(None), slice(0, we)) if layout == "NCHW" else \
        (slice(None), slice(0, we))
    assert (got[:dst_off] == sentinel).all()
    for i in range(n):
        lo = dst_off + i * stride
        body = got[lo:lo + frame].reshape(shape)
        if dtype == "float32":
            np.testing.assert_allclose(body[cols].view(np.float32), want[i][cols], rtol=1e-6,
                                       atol=1e-6)
        else:
            assert (body[cols].view(want.dtype) == want[i][cols]).all()
        if w & 1:
            tail = body[..., w - 1] if layout == "NCHW" else body[:, w - 1]
            assert (tail == sentinel).all()
        assert (got[lo + frame:lo + stride] == sentinel).all()
    assert (got[dst_off + n * stride:] == sentinel).all()
