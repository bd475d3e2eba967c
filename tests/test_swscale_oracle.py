"""The oracle's restatement of libswscale's integer yuv420p -> rgb24 arithmetic -- the
arithmetic of the reference's CPU route ("format=pix_fmts=rgb24" in the filter graph of
src/libspdl/core/detail/ffmpeg/filter_graph.cpp:50-65) -- against fixtures produced by the
library itself (tests/golden/make_sws_golden.py) and, where it can be loaded, the library."""

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import oracle
from oracle import swscale_ref
from tests import synth

GOLD = json.loads((Path(__file__).parent / "golden" / "sws_golden.json").read_text())
SMALL = np.load(Path(__file__).parent / "golden" / "sws_small.npz")


@pytest.mark.parametrize("key", sorted(GOLD["tables_sha256"]))
def test_every_triple_matches_the_library_fixture(key):
    cs, full = (int(v) for v in key.split("_"))
    table = oracle.exhaustive(cs, bool(full), arith=oracle.ARITH_SWSCALE)
    assert hashlib.sha256(table.tobytes()).hexdigest() == GOLD["tables_sha256"][key]


def test_known_triplets_as_libswscale_converts_them():
    # the colours of tests/cuda/nvdec_video_decoding_test.py:335-348; libswscale's answers are
    # up to 2 LSB from the CUDA kernel's (255,22,0), (0,217,0), (0,14,255)
    for key, rgb in GOLD["triplets"].items():
        y, u, v = (int(t) for t in key.split(","))
        assert list(oracle.sws_pixel(y, u, v, 1, False)) == rgb


def test_colourspace_numbers_follow_the_library_table():
    # unknown numbers and 8 fall back to BT.601, as sws_getCoefficients does
    for cs in (-3, 0, 2, 3, 8, 11, 42):
        assert oracle.sws_coeffs(cs) == oracle.sws_coeffs(5)
    assert oracle.sws_coeffs(6) == oracle.sws_coeffs(5)
    assert oracle.sws_coeffs(10) == oracle.sws_coeffs(9)
    assert oracle.sws_coeffs(1) == {"yc": 9539, "vr": 14686, "ug": -1747, "vg": -4366,
                                    "ub": 17305, "yo": 128}
    distinct = {tuple(v) for v in GOLD["coefficients"].values()}
    assert len(distinct) == 5  # 601, 709, FCC, 240M, 2020


@pytest.mark.parametrize("name,cs,full", [("bt709_limited", 1, False), ("bt601_full", 5, True)])
@pytest.mark.parametrize("layout", [oracle.NCHW, oracle.NHWC])
def test_small_frames_through_the_frame_path(name, cs, full, layout):
    frame, want = SMALL[name + "_i420"], SMALL[name + "_rgb"]
    h2, w = frame.shape
    h = h2 * 2 // 3
    flat = frame.reshape(-1)
    got = oracle.convert_dense(frame, flat[h * w:], flat[h * w + (h // 2) * (w // 2):], width=w,
                               height=h, num_frames=1, y_pitch=w, uv_pitch=w // 2,
                               y_frame_stride=h2 * w, uv_frame_stride=h2 * w,
                               src_format=oracle.I420, coeff=cs, full_range=full, layout=layout,
                               arith=oracle.ARITH_SWSCALE)[0]
    assert (got == (want.transpose(2, 0, 1) if layout == oracle.NCHW else want)).all()


@pytest.mark.skipif(not swscale_ref.available(), reason="libswscale is not on this machine")
@pytest.mark.parametrize("cs,full", [(1, False), (5, True), (4, False)])
def test_live_library_on_the_cpu_runnable_configuration(cs, full):
    """Frames of the CPU-runnable benchmark configuration (1920x1080 I420, smooth gradient plus
    noise) converted by the loaded library and by the oracle: identical bytes."""
    w, h, n = 1920, 1080, 2
    batch = synth.i420_batch_gradient(n, w, h, config=1, index=cs)
    want = np.empty((n, h, w, 3), np.uint8)
    conv = swscale_ref.I420ToRGB(w, h, cs, full_range=full)
    for i in range(n):
        conv(batch[i], want[i])
    flat = batch.reshape(-1)
    got = oracle.convert_dense(batch, flat[h * w:], flat[h * w + (h // 2) * (w // 2):], width=w,
                               height=h, num_frames=n, y_pitch=w, uv_pitch=w // 2,
                               y_frame_stride=h * 3 // 2 * w, uv_frame_stride=h * 3 // 2 * w,
                               src_format=oracle.I420, coeff=cs, full_range=full,
                               layout=oracle.NHWC, arith=oracle.ARITH_SWSCALE)
    assert (got == want).all()


def test_the_two_arithmetics_differ_as_documented():
    """libswscale's BT.709 against the CUDA kernel's table: the same transform, but only about
    half of all pixels agree exactly (the table scales chroma by 255/219)."""
    a = oracle.exhaustive(1, False)[16:236, 16:241, 16:241].astype(np.int16)
    b = oracle.exhaustive(1, False, arith=oracle.ARITH_SWSCALE)[16:236, 16:241, 16:241]
    d = np.abs(a - b)
    assert d.max() <= 9 and 0.3 < (d == 0).mean() < 0.7


@pytest.mark.skipif(not swscale_ref.available(), reason="libswscale is not on this machine")
def test_widths_that_are_not_multiples_of_eight():
    """The library's SIMD loop converts groups of 8 pixels.  Given a destination stride with room
    it converts up to the next multiple of 8 with the same arithmetic, so every column of a
    50-wide frame equals the restatement; given a tight stride it leaves the last two columns of
    that frame unwritten (a property of the library, not a second arithmetic)."""
    import ctypes

    w, h = 50, 22
    frame = np.random.default_rng(1).integers(0, 256, (h * 3 // 2, w), dtype=np.uint8)
    flat = frame.reshape(-1)
    want = oracle.convert_dense(frame[None], flat[h * w:], flat[h * w + (h // 2) * (w // 2):],
                                width=w, height=h, num_frames=1, y_pitch=w, uv_pitch=w // 2,
                                y_frame_stride=h * 3 // 2 * w, uv_frame_stride=h * 3 // 2 * w,
                                src_format=oracle.I420, layout=oracle.NHWC,
                                arith=oracle.ARITH_SWSCALE)[0]
    conv = swscale_ref.I420ToRGB(w, h, 1)
    tight = np.full((h, w, 3), 77, np.uint8)
    conv(frame, tight)
    assert (tight[:, :48] == want[:, :48]).all() and (tight[:, 48:] == 77).all()
    roomy = np.full((h, 64, 3), 77, np.uint8)
    base = frame.ctypes.data
    src = (ctypes.c_void_p * 4)(base, base + w * h, base + w * h + (w // 2) * (h // 2), None)
    stride = (ctypes.c_int * 4)(w, w // 2, w // 2, 0)
    dst = (ctypes.c_void_p * 4)(roomy.ctypes.data, None, None, None)
    dstride = (ctypes.c_int * 4)(64 * 3, 0, 0, 0)
    assert swscale_ref.load().sws_scale(conv.ctx, src, stride, 0, h, dst, dstride) == h
    assert (roomy[:, :w] == want).all()
