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
    got = io.to_torch(io.convert_nv12(_dev(nv), device_config=cuda_cfg, src_format=fmt,
                                      layout=layout, dtype=dtype, order=order, coeff=coeff,
                                      full_range=full, sync=True, **norm)).cpu().numpy()
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
        sb=oracle.scale_bias(MEAN, STD) if norm else None)
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
    mode = int(r.integers(0, 3))
    if mode == 0:      # stretch to a fixed size (up- or down-scaling)
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
    buf = io.convert_resize(_dev(data), _dev(descs.view(np.uint8)), out_size=out,
                            max_src_w=int(ws.max()), device_config=cuda_cfg, src_format=fmt,
                            coeff=coeff, full_range=full, layout=layout, dtype=dtype, order=order,
                            sync=True, **norm)
    got = io.to_torch(buf).cpu().numpy()
    want = oracle.convert_resize(
        data, descs, out_w=out[0], out_h=out[1], src_format=_O_FMT[fmt], coeff=coeff,
        full_range=full, layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC,
        dtype=_O_DT[dtype], order=oracle.RGB if order == "rgb" else oracle.BGR,
        sb=oracle.scale_bias(MEAN, STD) if norm else None)
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
