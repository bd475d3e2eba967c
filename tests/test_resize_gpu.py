"""Parity of the fused convert -> resize -> crop -> normalise kernel with the oracle."""

import numpy as np
import pytest

import oracle
from tests import synth

pytestmark = pytest.mark.gpu

MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
_O_DT = {"uint8": oracle.U8, "float32": oracle.F32, "bfloat16": oracle.BF16}


def _dev(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _run(cfg, data, descs, out_size, fmt, layout, dtype, order="rgb", coeff=1, full_range=False,
         mean=None, std=None):
    import spdl_b200.io as io

    max_w = int(descs["src_w"].max())
    buf = io.convert_resize(_dev(data), _dev(descs.view(np.uint8)), out_size=out_size,
                            max_src_w=max_w, device_config=cfg, src_format=fmt, coeff=coeff,
                            full_range=full_range, layout=layout, dtype=dtype, order=order,
                            mean=mean, std=std, sync=True)
    got = io.to_torch(buf).cpu().numpy()
    want = oracle.convert_resize(
        data, descs, out_w=out_size[0], out_h=out_size[1],
        src_format=oracle.NV12 if fmt == "nv12" else oracle.I420, coeff=coeff,
        full_range=full_range, layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC,
        dtype=_O_DT[dtype], order=oracle.RGB if order == "rgb" else oracle.BGR,
        sb=oracle.scale_bias(mean, std) if mean is not None else None)
    return got, want


def _compare(got, want, dtype):
    assert got.shape == want.shape
    if dtype == "uint8":
        # same fp32 operations in the same order: bit-exact
        assert (got == want).all()
    elif dtype == "float32":
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    else:
        a = oracle.bf16_to_f32(got.view(np.uint16))
        b = oracle.bf16_to_f32(want)
        # identical up to one bf16 ulp where the fp32 values straddle a rounding boundary
        np.testing.assert_allclose(a, b, rtol=2 ** -7, atol=1e-6)
        assert (got.view(np.uint16) == want).mean() > 0.999


@pytest.mark.parametrize("src,dst", [((64, 48), (24, 20)), ((320, 240), (160, 120)),
                                     ((40, 30), (40, 30)), ((30, 20), (50, 44)),
                                     ((1280, 720), (256, 256)), ((98, 50), (33, 17))])
@pytest.mark.parametrize("fmt", ["nv12", "i420"])
@pytest.mark.parametrize("layout,dtype", [("NCHW", "uint8"), ("NHWC", "uint8"),
                                          ("NCHW", "float32"), ("NHWC", "bfloat16")])
def test_uniform_resize(cuda_cfg, src, dst, fmt, layout, dtype):
    import spdl_b200.io as io

    w, h = src
    n = 3
    nv = synth.nv12_batch(n, w, h, config=9, index=w)
    descs, out = io.make_image_descs([w] * n, [h] * n, src_format=fmt, resize=dst)
    norm = dict(mean=MEAN, std=STD) if dtype != "uint8" else {}
    got, want = _run(cuda_cfg, nv.reshape(-1), descs, out, fmt, layout, dtype, **norm)
    _compare(got, want, dtype)


def test_crop_equals_slice_of_uncropped(cuda_cfg):
    """tests/cuda/nvdec_video_decoding_test.py:257-284 of the reference checks the same property
    for the decoder's crop."""
    import spdl_b200.io as io

    w, h = 320, 240
    nv = synth.nv12_batch(2, w, h, config=9, index=8)
    full_d, fo = io.make_image_descs([w, w], [h, h], resize=(200, 150))
    crop_d, co = io.make_image_descs([w, w], [h, h], resize=(200, 150), crop=(64, 48))
    full, _ = _run(cuda_cfg, nv.reshape(-1), full_d, fo, "nv12", "NCHW", "uint8")
    crop, want = _run(cuda_cfg, nv.reshape(-1), crop_d, co, "nv12", "NCHW", "uint8")
    cx, cy = int(crop_d["crop_x"][0]), int(crop_d["crop_y"][0])
    assert (crop == full[:, :, cy:cy + 48, cx:cx + 64]).all()
    assert (crop == want).all()


@pytest.mark.parametrize("dtype", ["uint8", "float32"])
def test_ragged_i420_shorter_side_centre_crop(cuda_cfg, dtype):
    """Ragged batch: per-image sizes and offsets, shorter side to 64, centre crop 56x56,
    full-range BT.601 (JPEG-style)."""
    import spdl_b200.io as io

    data, ws, hs, offs = synth.ragged_i420(24, lo=64, hi=200, config=5, index=1)
    descs, out = io.make_image_descs(ws, hs, src_format="i420", offsets=offs, resize_shorter=64,
                                     crop=(56, 56))
    assert out == (56, 56)
    norm = dict(mean=MEAN, std=STD) if dtype != "uint8" else {}
    got, want = _run(cuda_cfg, data, descs, out, "i420", "NCHW", dtype, coeff=6, full_range=True,
                     **norm)
    _compare(got, want, dtype)


def test_odd_sizes_and_upscale(cuda_cfg):
    import spdl_b200.io as io

    data, ws, hs, offs = synth.ragged_i420(6, lo=20, hi=60, config=5, index=2)
    ws, hs = ws + 1, hs - 1  # odd sizes: chroma planes are ceil(w/2) x ceil(h/2)
    sizes = ws * hs + 2 * ((ws + 1) // 2) * ((hs + 1) // 2)
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    data = np.random.default_rng(3).integers(0, 256, int(sizes.sum()), dtype=np.uint8)
    descs, out = io.make_image_descs(ws, hs, src_format="i420", offsets=offs, resize=(80, 72))
    got, want = _run(cuda_cfg, data, descs, out, "i420", "NHWC", "uint8", order="bgr")
    _compare(got, want, "uint8")


def test_clip_stacking_layout(cuda_cfg):
    """Clips stack as N x T x C x H x W: frames of clip n are images n*T .. n*T+T-1."""
    import spdl_b200.io as io

    clips, t, w, h = 2, 4, 128, 72
    frames = np.concatenate([synth.nv12_clip(t, w, h, config=4, index=i) for i in range(clips)])
    descs, out = io.make_image_descs([w] * clips * t, [h] * clips * t, resize=(32, 32))
    got, want = _run(cuda_cfg, frames.reshape(-1), descs, out, "nv12", "NCHW", "uint8", coeff=6)
    assert (got == want).all()
    stacked = got.reshape(clips, t, 3, 32, 32)
    assert (stacked[1, 2] == want[1 * t + 2]).all()


def test_4k_to_224_bf16(cuda_cfg):
    """One 3840x2160 frame -> 224x224 bf16 NCHW normalised (the large-downscale workload)."""
    import spdl_b200.io as io

    w, h = 3840, 2160
    nv = synth.nv12_batch(1, w, h, config=3)
    descs, out = io.make_image_descs([w], [h], resize=(224, 224))
    got, want = _run(cuda_cfg, nv.reshape(-1), descs, out, "nv12", "NCHW", "bfloat16", order="bgr",
                     mean=MEAN[::-1], std=STD[::-1])
    _compare(got, want, "bfloat16")


def test_validation(cuda_cfg):
    import torch

    import spdl_b200.io as io

    base = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    bad = torch.zeros(65, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        io.convert_resize(base, bad, out_size=(8, 8), max_src_w=16, device_config=cuda_cfg)
    d, o = io.make_image_descs([16], [16], resize=(8, 8))
    with pytest.raises(RuntimeError):  # staging limit
        io.convert_resize(base, _dev(d.view(np.uint8)), out_size=o, max_src_w=1 << 20,
                          device_config=cuda_cfg)
    with pytest.raises(RuntimeError):
        io.convert_resize(base, _dev(d.view(np.uint8)), out_size=o, max_src_w=16,
                          device_config=cuda_cfg, layout="CHWN")


@pytest.mark.parametrize("fmt", ["rgb_planar", "rgb24"])
@pytest.mark.parametrize("layout,dtype", [("NCHW", "uint8"), ("NHWC", "float32"),
                                          ("NCHW", "bfloat16")])
def test_rgb_sources_ragged(cuda_cfg, fmt, layout, dtype):
    """Already-decoded RGB of different sizes (what a JPEG decoder hands over), planar or
    interleaved -> shorter side 64, centre crop 48x48, normalise."""
    import spdl_b200.io as io

    rng = np.random.default_rng(21)
    ws = rng.integers(50, 180, 9)
    hs = rng.integers(50, 180, 9)
    sizes = 3 * ws * hs
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    data = rng.integers(0, 256, int(sizes.sum()), dtype=np.uint8)
    descs, out = io.make_image_descs(ws, hs, src_format=fmt, offsets=offs, resize_shorter=64,
                                     crop=(48, 48))
    norm = dict(mean=MEAN, std=STD) if dtype != "uint8" else {}
    max_w = int(descs["src_w"].max())
    buf = io.convert_resize(_dev(data), _dev(descs.view(np.uint8)), out_size=out, max_src_w=max_w,
                            device_config=cuda_cfg, src_format=fmt, layout=layout, dtype=dtype,
                            order="bgr", sync=True, **norm)
    got = io.to_torch(buf).cpu().numpy()
    want = oracle.convert_resize(
        data, descs, out_w=out[0], out_h=out[1],
        src_format=oracle.RGBP if fmt == "rgb_planar" else oracle.RGBI,
        layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC, dtype=_O_DT[dtype],
        order=oracle.BGR, sb=oracle.scale_bias(MEAN, STD) if norm else None)
    _compare(got, want, dtype)


@pytest.mark.parametrize("fmt", ["rgb_planar", "rgb24"])
@pytest.mark.parametrize("out_w,mode", [(97, None), (160, "pad"), (300, "crop")])
def test_wide_rgb_sources_take_two_row_tiles(cuda_cfg, fmt, out_w, mode):
    """RGB sources wide enough for two-row tiles (two warps share an output row and take
    alternate blocks of 128 columns), with output widths that end inside a block, letterbox bars
    and a cover crop."""
    import spdl_b200.io as io

    rng = np.random.default_rng(77 + out_w)
    ws, hs = np.array([4000, 3600, 2200]), np.array([12, 30, 21])
    sizes = 3 * ws * hs
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    data = rng.integers(0, 256, int(sizes.sum()), dtype=np.uint8)
    kw = dict(scale_mode=mode) if mode else {}
    descs, out = io.make_image_descs(ws, hs, src_format=fmt, offsets=offs, resize=(out_w, 11), **kw)
    for layout, dtype in (("NCHW", "uint8"), ("NHWC", "float32")):
        norm = dict(mean=MEAN, std=STD) if dtype != "uint8" else {}
        buf = io.convert_resize(_dev(data), _dev(descs.view(np.uint8)), out_size=out,
                                max_src_w=int(ws.max()), device_config=cuda_cfg, src_format=fmt,
                                layout=layout, dtype=dtype, pad_color=(12.0, 200.0, 77.0),
                                sync=True, **norm)
        want = oracle.convert_resize(
            data, descs, out_w=out[0], out_h=out[1],
            src_format=oracle.RGBP if fmt == "rgb_planar" else oracle.RGBI,
            layout=oracle.NCHW if layout == "NCHW" else oracle.NHWC, dtype=_O_DT[dtype],
            pad_value=(12.0, 200.0, 77.0), sb=oracle.scale_bias(MEAN, STD) if norm else None)
        _compare(io.to_torch(buf).cpu().numpy(), want, dtype)


def test_unaligned_output_width(cuda_cfg):
    """out_w not a multiple of 4 takes the element-store path."""
    import spdl_b200.io as io

    w, h = 96, 64
    nv = synth.nv12_batch(2, w, h, config=9, index=31)
    descs, out = io.make_image_descs([w, w], [h, h], resize=(37, 23))
    for layout, dtype in (("NCHW", "uint8"), ("NHWC", "uint8"), ("NHWC", "float32")):
        got, want = _run(cuda_cfg, nv.reshape(-1), descs, out, "nv12", layout, dtype)
        _compare(got, want, dtype)


@pytest.mark.parametrize("out_w", [1, 2, 3, 4, 5, 8, 9, 28, 33, 100, 124, 132, 224, 236])
def test_output_widths_around_the_lane_mappings(cuda_cfg, out_w):
    """One group of four columns, groups that fill part of a warp, whole warps and a little more:
    every way the kernel spreads a tile's columns over its lanes, with a last tile of odd height."""
    import spdl_b200.io as io

    w, h = 150, 90
    nv = synth.nv12_batch(2, w, h, config=9, index=out_w)
    descs, out = io.make_image_descs([w, w], [h, h], resize=(out_w, 21))
    for layout, dtype in (("NCHW", "uint8"), ("NHWC", "float32")):
        got, want = _run(cuda_cfg, nv.reshape(-1), descs, out, "nv12", layout, dtype)
        _compare(got, want, dtype)


@pytest.mark.parametrize("world", [2, 8])
def test_sharded_ragged_batch_equals_whole(cuda_cfg, world):
    """The ragged batch split over ``world`` ranks in contiguous blocks (descriptor table sliced,
    offsets still relative to the shared buffer): the ranks' outputs, concatenated, are the
    whole-batch output.  Ranks run one after the other on this GPU."""
    import spdl_b200.io as io
    from spdl_b200.sharding import shard_range

    n = 24
    data, ws, hs, offs = synth.ragged_i420(n, lo=64, hi=160, config=5, index=7)
    descs, out = io.make_image_descs(ws, hs, src_format="i420", offsets=offs, resize_shorter=48,
                                     crop=(40, 40))
    whole, want = _run(cuda_cfg, data, descs, out, "i420", "NCHW", "float32", coeff=6,
                       full_range=True, mean=MEAN, std=STD)
    _compare(whole, want, "float32")
    parts = []
    for r in range(world):
        lo, hi = shard_range(n, r, world)
        got, _ = _run(cuda_cfg, data, descs[lo:hi].copy(), out, "i420", "NCHW", "float32", coeff=6,
                      full_range=True, mean=MEAN, std=STD)
        parts.append(got)
    assert (np.concatenate(parts) == whole).all()


def test_sharded_clips_equal_whole(cuda_cfg):
    """Clips split over 4 ranks (whole clips per rank): N x T x C x H x W of the ranks,
    concatenated along N, is the whole batch."""
    import spdl_b200.io as io
    from spdl_b200.sharding import shard_range

    clips, t, w, h, world = 8, 4, 128, 72, 4
    frames = np.concatenate([synth.nv12_clip(t, w, h, config=4, index=i) for i in range(clips)])
    descs, out = io.make_image_descs([w] * clips * t, [h] * clips * t, resize=(32, 32))
    whole, want = _run(cuda_cfg, frames.reshape(-1), descs, out, "nv12", "NCHW", "uint8", coeff=6)
    assert (whole == want).all()
    parts = []
    for r in range(world):
        lo, hi = shard_range(clips, r, world)
        mine = frames[lo * t:hi * t]  # this rank's clips, resident on its own GPU
        d, _ = io.make_image_descs([w] * (hi - lo) * t, [h] * (hi - lo) * t, resize=(32, 32))
        got, _ = _run(cuda_cfg, mine.reshape(-1), d, out, "nv12", "NCHW", "uint8", coeff=6)
        parts.append(got.reshape(hi - lo, t, 3, 32, 32))
    assert (np.concatenate(parts) == whole.reshape(clips, t, 3, 32, 32)).all()


@pytest.mark.parametrize("fmt", ["rgb24", "rgb_planar"])
def test_resize_image_list_reads_images_where_they_lie(cuda_cfg, fmt):
    """Separately allocated device images of different sizes (a decoder's output list) go through
    one launch without being packed; the result equals the oracle on a packed copy."""
    import torch

    import spdl_b200.io as io

    rng = np.random.default_rng(33)
    ws, hs = rng.integers(40, 160, 7), rng.integers(40, 160, 7)
    host = [rng.integers(0, 256, (h, w, 3) if fmt == "rgb24" else (3, h, w), dtype=np.uint8)
            for w, h in zip(ws, hs)]
    images = [torch.from_numpy(a).cuda() for a in host]
    got = io.to_torch(io.resize_image_list(images, device_config=cuda_cfg, src_format=fmt,
                                           resize_shorter=48, crop=(40, 32), dtype="float32",
                                           mean=MEAN, std=STD, sync=True)).cpu().numpy()
    packed = np.concatenate([a.reshape(-1) for a in host])
    descs, out = io.make_image_descs(ws, hs, src_format=fmt, resize_shorter=48, crop=(40, 32))
    want = oracle.convert_resize(packed, descs, out_w=out[0], out_h=out[1],
                                 src_format=oracle.RGBI if fmt == "rgb24" else oracle.RGBP,
                                 dtype=oracle.F32, sb=oracle.scale_bias(MEAN, STD))
    _compare(got, want, "float32")
    with pytest.raises(RuntimeError):
        io.resize_image_list([], device_config=cuda_cfg, resize=(8, 8))
    with pytest.raises(RuntimeError):
        io.resize_image_list([images[0][..., :2].contiguous()], device_config=cuda_cfg,
                             resize=(8, 8))


@pytest.mark.parametrize("fmt", ["rgb24", "rgb_planar", "i420", "nv12"])
def test_resize_host_images_packs_uploads_and_resizes_in_one_go(cuda_cfg, fmt):
    """Host images of different sizes (a CPU decoder's output list): packed into page-locked
    staging, one upload, one launch; the result equals the oracle on the same images packed back
    to back."""
    import torch

    import spdl_b200.io as io

    rng = np.random.default_rng(35)
    ws, hs = 2 * rng.integers(20, 90, 9), 2 * rng.integers(20, 90, 9)
    shape = {"rgb24": lambda w, h: (h, w, 3), "rgb_planar": lambda w, h: (3, h, w),
             "i420": lambda w, h: (h * 3 // 2, w), "nv12": lambda w, h: (h * 3 // 2, w)}[fmt]
    host = [rng.integers(0, 256, shape(w, h), dtype=np.uint8) for w, h in zip(ws, hs)]
    images = [torch.from_numpy(a) if i % 2 else a for i, a in enumerate(host)]
    kw = dict(resize_shorter=48, crop=(40, 32))
    got = io.to_torch(io.resize_host_images(images, device_config=cuda_cfg, src_format=fmt,
                                            dtype="float32", mean=MEAN, std=STD, coeff=6,
                                            **kw)).cpu().numpy()
    sizes = np.array([a.nbytes for a in host])
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    packed = np.concatenate([a.reshape(-1) for a in host])
    descs, out = io.make_image_descs(ws, hs, src_format=fmt, offsets=offs, **kw)
    ofmt = {"rgb24": oracle.RGBI, "rgb_planar": oracle.RGBP, "i420": oracle.I420,
            "nv12": oracle.NV12}[fmt]
    want = oracle.convert_resize(packed, descs, out_w=out[0], out_h=out[1], src_format=ofmt,
                                 coeff=6, dtype=oracle.F32, sb=oracle.scale_bias(MEAN, STD))
    _compare(got, want, "float32")
    # a second call of the same thread reuses the staging buffer
    again = io.to_torch(io.resize_host_images(images[:3], device_config=cuda_cfg, src_format=fmt,
                                              dtype="float32", mean=MEAN, std=STD, coeff=6,
                                              **kw)).cpu().numpy()
    _compare(again, want[:3], "float32")
    with pytest.raises(RuntimeError):
        io.resize_host_images([], device_config=cuda_cfg, resize=(8, 8))
    with pytest.raises(RuntimeError):
        io.resize_host_images([host[0].astype(np.float32)], device_config=cuda_cfg,
                              src_format=fmt, resize=(8, 8))


def _sample_against_oracle(got, base_host, descs, picks, out, fmt, dtype, **kw):
    """Oracle on a few images of a large batch: their descriptors still point into the shared
    buffer, so the oracle reads exactly the bytes the kernel read."""
    sub = descs[picks].copy()
    want = oracle.convert_resize(
        base_host, sub, out_w=out[0], out_h=out[1],
        src_format={"nv12": oracle.NV12, "i420": oracle.I420}[fmt], dtype=_O_DT[dtype], **kw)
    _compare(got[picks], want, dtype)


def test_full_size_ragged_i420_batch(cuda_cfg):
    """2048 ragged I420 images (256..1024, full-range BT.601) -> shorter side 256, centre crop
    224x224, fp32 normalised: a sample of images against the oracle, and the whole batch against
    itself run as 8 contiguous shards."""
    import spdl_b200.io as io
    from spdl_b200.sharding import shard_range

    n = 2048
    data, ws, hs, offs = synth.ragged_i420(n)
    descs, out = io.make_image_descs(ws, hs, src_format="i420", offsets=offs,
                                     resize_shorter=256, crop=(224, 224))
    assert out == (224, 224)
    base = _dev(data)
    kw = dict(out_size=out, max_src_w=int(ws.max()), device_config=cuda_cfg, src_format="i420",
              coeff=6, full_range=True, dtype="float32", mean=MEAN, std=STD, sync=True)
    whole = io.to_torch(io.convert_resize(base, _dev(descs.view(np.uint8)), **kw))
    picks = np.array([0, 1, 511, 1024, 2047, int(np.argmax(ws)), int(np.argmin(hs))])
    _sample_against_oracle(whole.cpu().numpy(), data, descs, picks, out, "i420", "float32",
                           coeff=6, full_range=True, sb=oracle.scale_bias(MEAN, STD))
    for r in range(8):
        lo, hi = shard_range(n, r, 8)
        part = io.to_torch(io.convert_resize(base, _dev(descs[lo:hi].copy().view(np.uint8)), **kw))
        assert bool((part == whole[lo:hi]).all())


def test_full_size_clip_batch(cuda_cfg):
    """64 clips x 16 frames of 1280x720 NV12 -> 256x256 u8, BT.601, stacked N x T x C x H x W:
    sampled frames against the oracle (bit-exact) and clip 8r..8r+8 of rank r against the whole."""
    import torch

    import spdl_b200.io as io

    clips, t, w, h = 64, 16, 1280, 720
    g = torch.Generator(device="cuda").manual_seed(4000)
    src = torch.randint(16, 236, (clips * t, h * 3 // 2, w), dtype=torch.uint8, device="cuda",
                        generator=g)
    descs, out = io.make_image_descs([w] * clips * t, [h] * clips * t, resize=(256, 256))
    kw = dict(out_size=out, max_src_w=w, device_config=cuda_cfg, src_format="nv12", coeff=6,
              sync=True)
    whole = io.to_torch(io.convert_resize(src, _dev(descs.view(np.uint8)), **kw))
    assert tuple(whole.reshape(clips, t, 3, 256, 256).shape) == (clips, t, 3, 256, 256)
    picks = np.array([0, 17, 500, 1023])
    frames = src[torch.from_numpy(picks).cuda()].cpu().numpy()
    d4, _ = io.make_image_descs([w] * 4, [h] * 4, resize=(256, 256))
    want = oracle.convert_resize(frames.reshape(-1), d4, out_w=256, out_h=256, coeff=6)
    assert (whole[torch.from_numpy(picks).cuda()].cpu().numpy() == want).all()
    per = clips // 8 * t  # frames per rank
    d_rank, _ = io.make_image_descs([w] * per, [h] * per, resize=(256, 256))
    d_rank_dev = _dev(d_rank.view(np.uint8))
    for r in (0, 3, 7):
        part = io.to_torch(io.convert_resize(src[r * per:(r + 1) * per], d_rank_dev, **kw))
        assert bool((part == whole[r * per:(r + 1) * per]).all())


def test_full_size_4k_batch(cuda_cfg):
    """16 x 3840x2160 NV12 -> 224x224 bf16 NCHW normalised (BGR planes): every image against the
    oracle."""
    import spdl_b200.io as io

    n, w, h = 16, 3840, 2160
    nv = synth.nv12_batch(n, w, h, config=3)
    descs, out = io.make_image_descs([w] * n, [h] * n, resize=(224, 224))
    got, want = _run(cuda_cfg, nv.reshape(-1), descs, out, "nv12", "NCHW", "bfloat16", order="bgr",
                     mean=MEAN[::-1], std=STD[::-1])
    _compare(got, want, "bfloat16")


@pytest.mark.parametrize("fmt", ["nv12", "i420", "rgb24", "rgb_planar"])
def test_source_window_then_resize(cuda_cfg, fmt):
    """Crop the source, then scale (the decoder's order): kernel against the oracle through the
    same descriptors."""
    import spdl_b200.io as io

    rng = np.random.default_rng(44)
    n = 5
    ws, hs = rng.integers(30, 100, n) * 2, rng.integers(30, 100, n) * 2
    yuv = fmt in ("nv12", "i420")
    sizes = ws * hs * 3 // 2 if yuv else 3 * ws * hs
    data = rng.integers(0, 256, int(sizes.sum()), dtype=np.uint8)
    descs, out = io.make_image_descs(ws, hs, src_format=fmt, resize=(48, 36),
                                     src_crop=(6, 2, 10, 4), crop=(40, 30))
    buf = io.convert_resize(_dev(data), _dev(descs.view(np.uint8)), out_size=out,
                            max_src_w=int(ws.max()), device_config=cuda_cfg, src_format=fmt,
                            layout="NHWC", sync=True)
    got = io.to_torch(buf).cpu().numpy()
    want = oracle.convert_resize(
        data, descs, out_w=out[0], out_h=out[1], layout=oracle.NHWC,
        src_format={"nv12": oracle.NV12, "i420": oracle.I420, "rgb24": oracle.RGBI,
                    "rgb_planar": oracle.RGBP}[fmt])
    assert (got == want).all()
