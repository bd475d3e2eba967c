"""The CPU oracle against the reference's known answers and against itself."""

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import oracle
from tests import synth

GOLDEN = Path(__file__).resolve().parent / "golden"

# tests/cuda/nvdec_video_decoding_test.py:335-348 of the reference: three solid colours through
# NVDEC + nv12_to_rgb (coeff=1).  (Y,U,V) of the encoded colours -> expected (R,G,B).
KNOWN = [((81, 90, 240), (255, 22, 0)), ((145, 54, 34), (0, 217, 0)), ((41, 240, 110), (0, 14, 255))]


@pytest.mark.parametrize("yuv,rgb", KNOWN)
@pytest.mark.parametrize("mode", [oracle.FMA_NONE, oracle.FMA_LUMA_FIRST, oracle.FMA_CHROMA_FIRST,
                                  oracle.FMA_DEVICE])
def test_known_answers(yuv, rgb, mode):
    assert oracle.pixel(*yuv, coeff=1, mode=mode) == rgb
    assert oracle.pixel_exact(*yuv, coeff=1) == rgb


def test_known_answers_through_frame_path():
    # a 2x2 NV12 frame per colour, as the decoder would hand it over
    for (y, u, v), rgb in KNOWN:
        nv = np.array([[[y, y], [y, y], [u, v]]], np.uint8)
        out = oracle.nv12_to_planar(nv, coeff=1)
        assert out.shape == (1, 3, 2, 2)
        for c in range(3):
            assert (out[0, c] == rgb[c]).all()
        bgr = oracle.nv12_to_planar(nv, coeff=1, order=oracle.BGR)
        assert (bgr[:, ::-1] == out).all()


def test_out_of_range_coeff_means_bt709():
    m1, off1 = oracle.matrix(1)
    for k in (0, -3, 11, 99, 2, 3, 8):
        m, off = oracle.matrix(k)
        assert (m == m1).all() and off == off1 == 16
    assert not (oracle.matrix(6)[0] == m1).all()
    assert oracle.matrix(5)[0].tolist() == oracle.matrix(6)[0].tolist()
    assert oracle.matrix(9)[0].tolist() == oracle.matrix(10)[0].tolist()


@pytest.mark.parametrize("coeff", [1, 6, 9])
def test_fusion_orders_within_one_lsb_of_exact(coeff):
    """fp32 evaluation, fused or not, is never more than 1 away from exact rational arithmetic
    and agrees on at least 99.9 % of all 2^24 inputs (the tolerance of the conversion path)."""
    tables = [oracle.exhaustive(coeff, mode=m).astype(np.int16) for m in (0, 1, 2, 4)]
    # exact arithmetic through the oracle's integer path on a strided sample
    ys, us, vs = np.meshgrid(np.arange(0, 256, 5), np.arange(0, 256, 7), np.arange(0, 256, 3),
                             indexing="ij")
    for y, u, v in list(zip(ys.ravel(), us.ravel(), vs.ravel()))[::37]:
        e = np.array(oracle.pixel_exact(int(y), int(u), int(v), coeff), np.int16)
        for t in tables:
            assert np.abs(t[y, u, v] - e).max() <= 1
    for a in tables[1:]:
        d = np.abs(a - tables[0])
        assert d.max() <= 1
        assert (d == 0).mean() >= 0.999


def test_shape_rules():
    with pytest.raises(RuntimeError):
        oracle.nv12_to_planar(np.zeros((6, 8), np.uint8))
    with pytest.raises(RuntimeError):
        oracle.nv12_to_planar(np.zeros((1, 7, 8), np.uint8))
    assert oracle.nv12_to_planar(np.zeros((0, 6, 8), np.uint8)).shape == (0, 3, 4, 8)


def test_odd_tail_is_left_untouched():
    nv = synth.nv12_batch(1, 9, 6, config=9)
    out = oracle.nv12_to_planar(nv)
    assert (out[..., 8] == 0).all()
    full = oracle.nv12_to_planar(np.ascontiguousarray(
        np.concatenate([nv[:, :, :8]], axis=2)))
    # the first 8 columns only depend on the first 8 luma/chroma bytes of each row
    assert (out[..., :8] == full).all()


def test_i420_equals_nv12_with_same_chroma():
    n, w, h = 2, 16, 8
    nv = synth.nv12_batch(n, w, h, config=9, index=3)
    uv = nv[:, h:].reshape(n, h // 2, w // 2, 2)
    i420 = np.concatenate([nv[:, :h].reshape(n, -1), uv[..., 0].reshape(n, -1),
                           uv[..., 1].reshape(n, -1)], axis=1).reshape(n, h * 3 // 2, w)
    flat = i420.reshape(-1)
    got = oracle.convert_dense(i420, flat[h * w:], flat[h * w + (h // 2) * (w // 2):], width=w,
                               height=h, num_frames=n, y_pitch=w, uv_pitch=w // 2,
                               y_frame_stride=h * 3 // 2 * w, uv_frame_stride=h * 3 // 2 * w,
                               src_format=oracle.I420)
    assert (got == oracle.nv12_to_planar(nv)).all()


def test_layouts_dtypes_agree():
    nv = synth.nv12_batch(2, 16, 8, config=9, index=4)
    kw = dict(width=16, height=8, num_frames=2, y_pitch=16, uv_pitch=16, y_frame_stride=192,
              uv_frame_stride=192)
    u = nv.reshape(-1)[128:]
    base = oracle.convert_dense(nv, u, None, **kw)
    nhwc = oracle.convert_dense(nv, u, None, layout=oracle.NHWC, **kw)
    assert (nhwc == base.transpose(0, 2, 3, 1)).all()
    sb = oracle.scale_bias((0.485, 0.456, 0.406), (0.229, 0.224, 0.225))
    f = oracle.convert_dense(nv, u, None, dtype=oracle.F32, sb=sb, **kw)
    want = (base.astype(np.float64) / 255 - np.array([0.485, 0.456, 0.406])[None, :, None, None]) \
        / np.array([0.229, 0.224, 0.225])[None, :, None, None]
    np.testing.assert_allclose(f, want, rtol=1e-5, atol=1e-5)
    b = oracle.bf16_to_f32(oracle.convert_dense(nv, u, None, dtype=oracle.BF16, sb=sb, **kw))
    np.testing.assert_allclose(b, f, rtol=2 ** -8, atol=1e-6)


def _torch_bilinear(rgb_u8: np.ndarray, size):
    import torch

    x = torch.from_numpy(rgb_u8.astype(np.float32))
    return torch.nn.functional.interpolate(x, size=size, mode="bilinear", align_corners=False,
                                           antialias=False).numpy()


@pytest.mark.parametrize("src,dst", [((64, 48), (24, 20)), ((40, 30), (40, 30)), ((30, 20), (50, 44))])
def test_bilinear_matches_torch(src, dst):
    """The resize restatement equals torch's bilinear (align_corners=False, no antialias) applied
    to the converted 8-bit RGB, to 1e-4 in fp32."""
    import spdl_b200.io as io

    w, h = src
    nv = synth.nv12_batch(2, w, h, config=9, index=5)
    rgb = oracle.nv12_to_planar(nv)
    descs, (ow, oh) = io.make_image_descs([w, w], [h, h], resize=dst)
    got = oracle.convert_resize(nv.reshape(-1), descs, out_w=ow, out_h=oh, dtype=oracle.F32)
    want = _torch_bilinear(rgb, (dst[1], dst[0]))
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-4)
    got8 = oracle.convert_resize(nv.reshape(-1), descs, out_w=ow, out_h=oh)
    assert np.abs(got8.astype(np.int16) - np.floor(want + 0.5)).max() <= 1


def test_resize_crop_is_slice_of_uncropped():
    import spdl_b200.io as io

    w, h = 96, 64
    nv = synth.nv12_batch(1, w, h, config=9, index=6)
    full_d, _ = io.make_image_descs([w], [h], resize=(48, 40))
    full = oracle.convert_resize(nv.reshape(-1), full_d, out_w=48, out_h=40)
    crop_d, (ow, oh) = io.make_image_descs([w], [h], resize=(48, 40), crop=(20, 16))
    crop = oracle.convert_resize(nv.reshape(-1), crop_d, out_w=ow, out_h=oh)
    cx, cy = int(crop_d["crop_x"][0]), int(crop_d["crop_y"][0])
    assert (crop == full[:, :, cy:cy + 16, cx:cx + 20]).all()


def test_gather_frames():
    surfs = [np.random.default_rng(i).integers(0, 256, (12, 32), dtype=np.uint8) for i in range(3)]
    out = oracle.gather_frames(surfs, 20, 8)
    assert out.shape == (3, 12, 20)
    for i, s in enumerate(surfs):
        assert (out[i] == s[:, :20]).all()


def test_checksum_is_order_sensitive():
    a = np.arange(100, dtype=np.uint8)
    assert oracle.checksum(a) != oracle.checksum(a[::-1].copy())
    assert oracle.checksum(a) == sum((int(b) + 1) * (1 + i) for i, b in enumerate(a))


# ---- fixtures produced by the reference's own kernel (tests/golden/make_golden.py) -------------


def _golden():
    p = GOLDEN / "ref_kernel_golden.json"
    if not p.exists():
        pytest.skip("golden fixtures not generated yet")
    return json.loads(p.read_text())


@pytest.mark.parametrize("coeff", [0, 1, 4, 5, 6, 7, 9, 11])
def test_exhaustive_table_matches_reference_kernel(coeff):
    """Over all 2^24 (Y,U,V) inputs the oracle equals what the reference kernel produced on a
    B200, bit for bit (compared through the sha256 recorded by make_golden.py)."""
    g = _golden()
    ex = synth.exhaustive_nv12()
    for order, key in ((oracle.RGB, "rgb"), (oracle.BGR, "bgr")):
        out = oracle.nv12_to_planar(ex, coeff=coeff, order=order)
        assert hashlib.sha256(out.tobytes()).hexdigest() == g["exhaustive_sha256"][f"{key}_{coeff}"]
    assert oracle.DEVICE_FMA_MODE in g["oracle_mode_exact"][f"rgb_{coeff}"]


def test_small_batches_match_reference_kernel():
    p = GOLDEN / "ref_kernel_small.npz"
    if not p.exists():
        pytest.skip("golden fixtures not generated yet")
    z = np.load(p)
    names = sorted({k.split("_")[0] for k in z.files})
    assert names
    for name in names:
        nv = z[f"{name}_in"]
        for coeff in (1, 6, 9):
            assert (oracle.nv12_to_planar(nv, coeff=coeff) == z[f"{name}_rgb_{coeff}"]).all()
        assert (oracle.nv12_to_planar(nv, coeff=1, order=oracle.BGR) == z[f"{name}_bgr_1"]).all()


# ---- libswscale, the arithmetic of the reference's CPU route ------------------------------------


@pytest.mark.parametrize("colorspace,coeff", [(1, 1), (5, 6)])
@pytest.mark.parametrize("full", [False, True])
def test_swscale_computes_the_same_transform(colorspace, coeff, full):
    """The reference's CPU route (libswscale, fixed-point tables, nearest chroma) and its CUDA
    kernel (fp32) are two implementations of one transform: on in-gamut input they agree to the
    table precision of libswscale -- at most 1 apart for full-range sources, at most 4 apart and
    99 % within 2 for limited-range ones.  This is what makes libswscale a fair CPU baseline."""
    from oracle import swscale_ref

    if not swscale_ref.available():
        pytest.skip("no libswscale on this machine")
    w, h = 256, 128
    r = np.random.default_rng(11)
    i420 = np.empty((1, h * 3 // 2, w), np.uint8)
    i420[0, :h] = r.integers(16, 236, (h, w))
    i420[0, h:] = r.integers(100, 156, (h // 2, w))
    got = np.empty((h, w, 3), np.uint8)
    swscale_ref.I420ToRGB(w, h, colorspace=colorspace, full_range=full)(i420[0], got)
    flat = i420.reshape(-1)
    want = oracle.convert_dense(
        i420, flat[h * w:], flat[h * w + (h // 2) * (w // 2):], width=w, height=h, num_frames=1,
        y_pitch=w, uv_pitch=w // 2, y_frame_stride=h * 3 // 2 * w, uv_frame_stride=h * 3 // 2 * w,
        src_format=oracle.I420, layout=oracle.NHWC, coeff=coeff, full_range=full)[0]
    d = np.abs(got.astype(np.int16) - want)
    if full:
        assert d.max() <= 1
    else:
        assert d.max() <= 4 and (d <= 2).mean() > 0.99


@pytest.mark.parametrize("seed", range(12))
def test_bilinear_matches_torch_random_geometry(seed):
    """Random source and target sizes (up- and down-scaling, odd sizes), with and without a
    crop: the resize restatement equals torch's bilinear on the converted RGB, the crop being a
    slice of the uncropped result."""
    import spdl_b200.io as io

    r = np.random.default_rng(4000 + seed)
    w, h = int(r.integers(4, 40)) * 2, int(r.integers(4, 40)) * 2
    rw, rh = int(r.integers(2, 90)), int(r.integers(2, 90))
    nv = synth.nv12_batch(1, w, h, config=9, index=seed)
    rgb = oracle.nv12_to_planar(nv)
    want = _torch_bilinear(rgb, (rh, rw))
    geom = dict(resize=(rw, rh))
    if seed % 2:
        geom["crop"] = (int(r.integers(1, rw + 1)), int(r.integers(1, rh + 1)))
    descs, (ow, oh) = io.make_image_descs([w], [h], **geom)
    got = oracle.convert_resize(nv.reshape(-1), descs, out_w=ow, out_h=oh, dtype=oracle.F32)
    cx, cy = int(descs["crop_x"][0]), int(descs["crop_y"][0])
    np.testing.assert_allclose(got, want[:, :, cy:cy + oh, cx:cx + ow], rtol=0, atol=3e-4)


def test_letterbox_pads_outside_the_resized_grid():
    """Pixels outside the resized image take the pad colour through the same rounding and
    scale/bias; pixels inside equal the plain resize of the image to its fitted size."""
    import spdl_b200.io as io

    w, h = 128, 72
    nv = synth.nv12_batch(1, w, h, config=9, index=5)
    descs, out = io.make_image_descs([w], [h], resize=(64, 64), scale_mode="pad")
    assert out == (64, 64) and int(descs["resized_h"][0]) == 36 and int(descs["crop_y"][0]) == -14
    pad = (12.0, 200.0, 77.0)
    got = oracle.convert_resize(nv.reshape(-1), descs.view(oracle.DESC_DTYPE), out_w=64, out_h=64,
                                pad_value=pad)
    plain_d, plain_out = io.make_image_descs([w], [h], resize=(64, 36))
    plain = oracle.convert_resize(nv.reshape(-1), plain_d.view(oracle.DESC_DTYPE), out_w=64,
                                  out_h=36)
    assert (got[0, :, 14:50] == plain[0]).all()
    for c in range(3):
        assert (got[0, c, :14] == int(pad[c])).all() and (got[0, c, 50:] == int(pad[c])).all()
    sb = oracle.scale_bias((0.485, 0.456, 0.406), (0.229, 0.224, 0.225))
    f = oracle.convert_resize(nv.reshape(-1), descs.view(oracle.DESC_DTYPE), out_w=64, out_h=64,
                              pad_value=pad, dtype=oracle.F32, sb=sb, order=oracle.BGR)
    # BGR: output slot 0 holds blue, normalised with slot 0's scale and bias
    np.testing.assert_allclose(f[0, 0, 0, 0], np.float32(pad[2]) * sb[0] + sb[3], rtol=1e-6)


def test_clip_layout_and_untouched_bad_descriptors():
    import spdl_b200.io as io

    t, w, h = 4, 64, 36
    frames = np.concatenate([synth.nv12_clip(t, w, h, config=4, index=i) for i in range(2)])
    descs, out = io.make_image_descs([w] * 2 * t, [h] * 2 * t, resize=(16, 12))
    descs = descs.view(oracle.DESC_DTYPE)
    flat = oracle.convert_resize(frames.reshape(-1), descs, out_w=16, out_h=12)
    cthw = oracle.convert_resize(frames.reshape(-1), descs, out_w=16, out_h=12, clip_frames=t)
    assert cthw.shape == (2, 3, t, 12, 16)
    assert (cthw == flat.reshape(2, t, 3, 12, 16).transpose(0, 2, 1, 3, 4)).all()
    bad = descs.copy()
    bad["scale_x"][3] = 0.0
    bad["src_h"][5] = 0
    kept = oracle.convert_resize(frames.reshape(-1), bad, out_w=16, out_h=12,
                                 out=np.full((2 * t, 3, 12, 16), 0xA5, np.uint8))
    assert (kept[3] == 0xA5).all() and (kept[5] == 0xA5).all() and (kept[4] == flat[4]).all()
