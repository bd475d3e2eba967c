"""Host-side logic that needs no GPU: configuration, storage, frame batching on the CPU,
descriptor tables, the library's exported symbols and the transfer helper's traversal."""

import ctypes
import dataclasses
import re
from collections import namedtuple
from pathlib import Path
from unittest import mock

import numpy as np
import pytest

import spdl_b200.io as io
from spdl_b200 import _build, _lib

ROOT = Path(__file__).resolve().parents[1]


def test_library_exports_every_declared_symbol():
    """Every function include/b2frames.h declares is exported by the built library (no compute
    call is made)."""
    _build.build()
    header = (ROOT / "include" / "b2frames.h").read_text()
    declared = set(re.findall(r"B2_API\s+[\w\s\*]+?\b(b2_\w+)\s*\(", header))
    assert declared == set(_lib.EXPORTS)
    handle = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared:
        assert hasattr(handle, name), name
    assert _lib.lib().b2_abi_version() == 2
    assert _lib.lib().b2_last_error() == b""


def test_struct_layouts_match_header_sizes():
    assert ctypes.sizeof(_lib.ImageDesc) == 64 == io.DESC_DTYPE.itemsize
    # field order of the ctypes mirrors follows the header; offsets that matter to the kernels
    assert _lib.DenseArgs.y.offset == 8 and _lib.DenseArgs.y_pitch.offset == 56
    assert _lib.ResizeArgs.base.offset == 8 and _lib.ResizeArgs.dst.offset == 64
    # version 1 of the structs ended at these offsets; the later fields start there
    assert _lib.DenseArgs.arith.offset == 168 and ctypes.sizeof(_lib.DenseArgs) == 176
    assert _lib.ResizeArgs.arith.offset == 104 and ctypes.sizeof(_lib.ResizeArgs) == 168
    assert _lib.ResizeArgs.status.offset == 144
    header = (ROOT / "include" / "b2frames.h").read_text()
    assert "version 1 (168)" in header and "version 1 (104)" in header


def test_status_and_message_without_a_gpu():
    L = _lib.lib()
    assert L.b2_convert_dense(None, None) != 0
    assert b"null" in L.b2_last_error()
    a = _lib.DenseArgs()
    a.struct_size = 4
    assert L.b2_convert_dense(ctypes.byref(a), None) == 1
    assert b"struct_size" in L.b2_last_error()
    a.struct_size = ctypes.sizeof(_lib.DenseArgs)
    a.layout = 7
    assert L.b2_convert_dense(ctypes.byref(a), None) == 1
    a.layout = 0
    a.width = -1
    assert L.b2_convert_dense(ctypes.byref(a), None) == 1
    a.width, a.height, a.num_frames = 16, 8, 0
    assert L.b2_convert_dense(ctypes.byref(a), None) == 0  # nothing to do
    assert L.b2_last_error() == b""
    with pytest.raises(RuntimeError, match="struct_size"):
        a.struct_size = 3
        _lib.check(L.b2_convert_dense(ctypes.byref(a), None))
    assert L.b2_nv12_to_planar_rgb(None, None, 8, None, 8, 8, 4, 0, 1) == 0
    assert L.b2_nv12_to_planar_rgb(None, None, 8, None, 8, 8, 4, 1, 1) == 1
    assert L.b2_gather_surfaces(None, None, 1, 8, 3, None, 0, None) == 1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()


def test_cuda_config():
    cfg = io.cuda_config(device_index=1)
    assert (cfg.device_index, cfg.stream, cfg.allocator) == (1, 0x2, None)
    cfg = io.cuda_config(0, stream=0, allocator=(lambda s, d, st: 0, lambda p: None))
    assert cfg.stream == 0 and callable(cfg.allocator[0])
    with pytest.raises(TypeError):
        io.cuda_config("0")
    with pytest.raises(TypeError):
        io.cuda_config(0, allocator=(1, 2))
    with pytest.raises(dataclasses.FrozenInstanceError):
        cfg.stream = 5


def test_cpu_storage_errors():
    # tests/cuda/pin_memory_test.py:69-75 of the reference
    with pytest.raises(RuntimeError):
        io.cpu_storage(0, pin_memory=False)
    with pytest.raises(TypeError):
        io.cpu_storage(-1, pin_memory=False)
    s = io.cpu_storage(128, pin_memory=False)
    assert s.size == 128 and not s.is_pinned() and s.as_array().shape == (128,)


def _yuv420(n, w, h, pad=3):
    rng = np.random.default_rng(0)
    return io.Frames("yuv420p", w, h, [[rng.integers(0, 256, (h, w + pad), dtype=np.uint8),
                                        rng.integers(0, 256, (h // 2, w // 2 + pad), dtype=np.uint8),
                                        rng.integers(0, 256, (h // 2, w // 2 + pad), dtype=np.uint8)]
                                       for _ in range(n)])


def test_convert_frames_shapes():
    f = _yuv420(5, 16, 8)
    b = io.convert_frames(f)
    assert b.shape == (5, 1, 12, 16)
    a = io.to_numpy(b)
    assert (a[3, 0, :8] == f.planes[3][0][:, :16]).all()
    assert (a[3, 0, 8:].reshape(-1)[:32].reshape(4, 8) == f.planes[3][1][:, :8]).all()
    assert (a[3, 0, 8:].reshape(-1)[32:].reshape(4, 8) == f.planes[3][2][:, :8]).all()
    assert io.convert_frames([f, f]).shape == (2, 5, 1, 12, 16)

    rng = np.random.default_rng(1)
    rgb = io.Frames("rgb24", 8, 4, [[rng.integers(0, 256, (4, 30), dtype=np.uint8)] for _ in range(3)])
    assert io.convert_frames(rgb).shape == (3, 4, 8, 3)
    img = io.Frames("rgb24", 8, 4, rgb.planes[:1], media="image")
    assert io.convert_frames(img).shape == (4, 8, 3)
    assert io.convert_frames([img, img]).shape == (2, 4, 8, 3)
    p444 = io.Frames("yuv444p", 8, 4, [[rng.integers(0, 256, (4, 8), dtype=np.uint8)] * 3])
    assert io.convert_frames(p444).shape == (1, 3, 4, 8)
    nv = io.Frames("nv12", 8, 4, [[rng.integers(0, 256, (4, 8), dtype=np.uint8),
                                   rng.integers(0, 256, (2, 8), dtype=np.uint8)]])
    assert io.convert_frames(nv).shape == (1, 1, 6, 8)
    p422 = io.Frames("yuv422p", 8, 4, [[rng.integers(0, 256, (4, 8), dtype=np.uint8),
                                        rng.integers(0, 256, (4, 4), dtype=np.uint8),
                                        rng.integers(0, 256, (4, 4), dtype=np.uint8)]])
    assert io.convert_frames(p422).shape == (1, 1, 8, 8)
    gray = io.Frames("gray8", 8, 4, [[rng.integers(0, 256, (4, 8), dtype=np.uint8)]])
    assert io.convert_frames(gray).shape == (1, 4, 8, 1)


def test_convert_frames_rgb24_round_trip():
    # tests/io/reference_frames_test.py:120-135 of the reference: (5,128,128,3) survives bit-exactly
    src = np.random.default_rng(2).integers(0, 256, (5, 128, 128, 3), dtype=np.uint8)
    f = io.Frames("rgb24", 128, 128, [[src[i].reshape(128, 384)] for i in range(5)])
    assert (io.to_numpy(io.convert_frames(f)) == src).all()


def test_convert_frames_errors():
    a, b = _yuv420(2, 16, 8), _yuv420(2, 32, 8)
    with pytest.raises(RuntimeError):
        io.convert_frames([a, b])
    with pytest.raises(RuntimeError):
        io.convert_frames([])
    with pytest.raises(RuntimeError):
        io.convert_frames(a, storage=io.cpu_storage(10, pin_memory=False))
    with pytest.raises(RuntimeError):
        io.convert_frames(io.Frames("yuv420p", 15, 8, a.planes))
    with pytest.raises(RuntimeError):
        io.convert_frames(io.Frames("p010", 16, 8, a.planes))


def test_buffer_keeps_storage_alive():
    b = io.convert_frames(_yuv420(1, 16, 8))
    arr = io.to_numpy(b)
    want = arr.copy()
    del b
    assert (arr == want).all()


def test_make_image_descs_geometry():
    d, out = io.make_image_descs([640, 480, 256], [480, 640, 256], src_format="i420",
                                 resize_shorter=256, crop=(224, 224))
    assert out == (224, 224)
    # shorter side 256, longer int(256*long/short) = 341; centre offsets round((dim-224)/2)
    assert [int(x) for x in d["crop_x"]] == [round((341 - 224) / 2), 16, 16]
    assert [int(x) for x in d["crop_y"]] == [16, round((341 - 224) / 2), 16]
    assert np.float32(d["scale_x"][0]) == np.float32(640) / np.float32(341)
    assert np.float32(d["scale_y"][2]) == np.float32(1.0)
    assert [int(x) for x in d["y_off"]] == [0, 460800, 921600]
    assert int(d["u_off"][1]) == 460800 + 480 * 640
    assert int(d["v_off"][1]) == 460800 + 480 * 640 + 240 * 320
    assert int(d["uv_pitch"][0]) == 320
    d, out = io.make_image_descs([1280], [720], resize=(256, 256))
    assert out == (256, 256) and int(d["uv_pitch"][0]) == 1280 and int(d["v_off"][0]) == 0
    with pytest.raises(RuntimeError):
        io.make_image_descs([100], [100], resize=(50, 50), crop=(64, 64))
    with pytest.raises(RuntimeError):
        io.make_image_descs([100, 200], [100, 200])
    with pytest.raises(RuntimeError):
        io.make_image_descs([100], [100], resize=(50, 50), resize_shorter=10)


def test_build_flags():
    from spdl_b200.io import utils

    assert utils.built_with_cuda() is True
    assert utils.built_with_nvcodec() is False and utils.built_with_nvjpeg() is False


# ---- transfer_tensor: traversal and call order with torch.cuda mocked (no GPU needed) -----------

Pair = namedtuple("Pair", ["a", "b"])


@dataclasses.dataclass
class Sample:
    x: object
    tag: str
    derived: object = dataclasses.field(init=False, default=None)


def test_recursive_apply_over_containers():
    from spdl_b200.io._transfer import _recursive_apply

    fn = lambda v: v * 2 if isinstance(v, int) else v  # noqa: E731
    s = Sample(3, "t")
    s.derived = 5
    out = _recursive_apply(fn, {"l": [1, (2, "s")], "p": Pair(4, [5]), "d": s})
    assert out["l"] == [2, (4, "s")]
    assert out["p"] == Pair(8, [10]) and isinstance(out["p"], Pair)
    assert out["d"].x == 6 and out["d"].tag == "t" and out["d"].derived == 10


def test_leaves_follow_the_order_of_the_container_walk():
    from spdl_b200.io._transfer import _leaves, _recursive_apply

    s = Sample(3, "t")
    s.derived = 5
    batch = {"l": [1, (2, "s")], "p": Pair(4, [5]), "d": s, "n": None}
    seen = []
    _recursive_apply(lambda v: seen.append(v) or v, batch)
    assert list(_leaves(batch)) == seen == [1, 2, "s", 4, 5, 3, "t", 5, None]


def test_transfer_tensor_stages_copies_and_synchronises_once(monkeypatch):
    """The host side of ``transfer_tensor`` without a GPU: pageable tensors are packed into one
    staging block at aligned offsets, pinned ones are copied from where they are, every copy is
    queued before the single synchronise, and the last ``num_caches`` results stay referenced."""
    import torch

    from spdl_b200.io import _transfer

    events = []

    class Fake(_transfer._ThreadTransfer):
        def __init__(self, num_caches):  # no CUDA stream, no device
            from collections import deque

            self.index, self.arena = 0, _transfer._StagingArena()
            self.recent = deque([None] * num_caches, maxlen=num_caches) if num_caches else None

        def _empty_like_on_device(self, t):
            return torch.empty_like(t)  # stands in for device memory

        def _copy_async(self, dst, host, nbytes):
            events.append(("copy", host, nbytes))
            ctypes.memmove(dst, host, nbytes)

        def _synchronize(self):
            events.append(("sync",))

    block = (ctypes.c_char * (1 << 20))()
    base = ctypes.addressof(block)
    monkeypatch.setattr(_transfer._StagingArena, "reserve",
                        lambda self, n: events.append(("reserve", n)) or base)
    a = torch.arange(100, dtype=torch.int32)           # 400 bytes -> 512 in the arena
    b = torch.arange(24, dtype=torch.float32).reshape(4, 6).t()  # not contiguous, 96 bytes
    empty = torch.zeros(0)
    tr = Fake(num_caches=2)
    out = tr({"a": a, "rest": [b, "label", empty]})
    assert torch.equal(out["a"], a) and torch.equal(out["rest"][0], b)
    assert out["rest"][1] == "label" and out["rest"][2].numel() == 0
    assert out["a"].data_ptr() != a.data_ptr()
    assert events == [("reserve", 512 + 256), ("copy", base, 400), ("copy", base + 512, 96),
                      ("sync",)]
    assert list(tr.recent) == [None, out]
    second = tr(a)
    third = tr(a)
    assert list(tr.recent) == [second, third]          # `out` has left the window
    # a tensor that reports itself page-locked is copied from its own memory
    events.clear()
    monkeypatch.setattr(torch.Tensor, "is_pinned", lambda self, *a: True)
    tr(a)
    assert events == [("copy", a.data_ptr(), 400), ("sync",)]


def test_transfer_tensor_rejects_bad_local_rank(monkeypatch):
    import torch

    from spdl_b200.io import _transfer

    monkeypatch.setenv("LOCAL_RANK", "3")
    _transfer._THREAD_LOCAL.__dict__.pop("transfer", None)
    with mock.patch.object(torch.cuda, "device_count", return_value=1):
        with pytest.raises(RuntimeError, match="LOCAL_RANK is 3"):
            _transfer.transfer_tensor(torch.zeros(1))


def test_call_counters_and_tracing_switch():
    from spdl_b200.io import utils
    from spdl_b200.io.utils import _tracing

    utils.reset_call_stats()
    _tracing.record("convert_nv12", 4, 100, 200)
    _tracing.record("convert_nv12", 2, 50, 100)
    assert utils.call_stats() == {"convert_nv12": {"calls": 2, "units": 6, "bytes_in": 150,
                                                   "bytes_out": 300}}
    utils.reset_call_stats()
    assert utils.call_stats() == {}
    with utils.tracing(False):
        with utils.trace_event("off"):  # no NVTX (and no torch.cuda) involved when off
            pass
    pushed = []
    fake = mock.MagicMock()
    fake.range_push.side_effect = pushed.append
    with mock.patch.object(_tracing, "_nvtx", return_value=fake), utils.tracing(True):
        with utils.trace_event("b2::convert_dense"):
            pass
    assert pushed == ["b2::convert_dense"] and fake.range_pop.call_count == 1


def test_convert_array_and_protocols():
    """convert_array copies int64 labels into a (pinned, when storage is given) CPUBuffer; the
    protocol classes recognise the buffers (the reference's tests/cuda/pin_memory_test.py:77-98
    checks the pinned round trip and the too-small storage)."""
    import spdl_b200.io as io

    vals = np.arange(-5, 19, dtype=np.int64).reshape(4, 6)
    buf = io.convert_array(vals)
    assert buf.shape == (4, 6) and isinstance(buf, io.ArrayInterface)
    assert not isinstance(buf, io.CUDAArrayInterface)
    out = io.to_numpy(buf)
    assert out.dtype == np.int64 and (out == vals).all()
    assert io.to_numba(buf).tolist() == vals.tolist()  # host buffers need no Numba
    # non-contiguous input is copied in C order
    assert (io.to_numpy(io.convert_array(vals.T)) == vals.T).all()
    with pytest.raises(RuntimeError):
        io.convert_array(np.zeros((0,), np.int64))
    with pytest.raises(TypeError):
        io.convert_array(np.zeros((3,), np.int32))
    with pytest.raises(RuntimeError):  # storage too small
        io.convert_array(vals, storage=io.cpu_storage(8, pin_memory=False))


def test_source_window_of_make_image_descs():
    """``src_crop`` cuts the source first (the decoder's crop-then-scale order): through the oracle
    the result equals resizing a cropped copy; odd values are refused for YUV sources."""
    import oracle
    import spdl_b200.io as io
    from tests import synth

    w, h, crop = 96, 64, (8, 4, 12, 6)
    nv = synth.nv12_batch(2, w, h, config=9, index=3)
    d, out = io.make_image_descs([w, w], [h, h], resize=(40, 30), src_crop=crop)
    assert out == (40, 30) and d["src_w"].tolist() == [76, 76] and d["src_h"].tolist() == [54, 54]
    assert d["y_pitch"].tolist() == [w, w]
    got = oracle.convert_resize(nv.reshape(-1), d, out_w=40, out_h=30)
    cropped = np.concatenate([np.concatenate([f[:h][4:h - 6, 8:w - 12].reshape(-1),
                                              f[h:][2:(h - 6) // 2, 8:w - 12].reshape(-1)])
                              for f in nv])
    d2, _ = io.make_image_descs([76, 76], [54, 54], resize=(40, 30))
    assert (got == oracle.convert_resize(cropped, d2, out_w=40, out_h=30)).all()
    with pytest.raises(RuntimeError):
        io.make_image_descs([w], [h], resize=(8, 8), src_crop=(1, 0, 0, 0))
    with pytest.raises(RuntimeError):
        io.make_image_descs([w], [h], resize=(8, 8), src_crop=(48, 0, 48, 0))
    # RGB sources take any window
    d3, _ = io.make_image_descs([w], [h], src_format="rgb24", resize=(8, 8), src_crop=(1, 3, 5, 7))
    assert int(d3["y_off"][0]) == 3 * 3 * w + 3 and int(d3["src_w"][0]) == w - 6


# ---- contiguity check of device arrays (no GPU needed: a fake __cuda_array_interface__) -----------


class _FakeCuda:
    def __init__(self, shape, strides, typestr="|u1"):
        self.__cuda_array_interface__ = {"version": 2, "shape": shape, "typestr": typestr,
                                         "data": (0x7F0000000000, False), "strides": strides}


def test_contiguity_check_ignores_only_size_one_dimensions():
    from spdl_b200.io._core import _cai

    # packed, with and without explicit strides
    assert _cai(_FakeCuda((2, 1620, 1920), None))[1] == (2, 1620, 1920)
    assert _cai(_FakeCuda((2, 1620, 1920), (1620 * 1920, 1920, 1)))[1] == (2, 1620, 1920)
    # a single pitched surface (row pitch 2048 > width): rejected although N == 1
    with pytest.raises(RuntimeError, match="C-contiguous"):
        _cai(_FakeCuda((1, 1620, 1920), (1620 * 2048, 2048, 1)))
    with pytest.raises(RuntimeError, match="C-contiguous"):
        _cai(_FakeCuda((2, 1620, 1920), (1620 * 2048, 2048, 1)))
    # a transposed single image
    with pytest.raises(RuntimeError, match="C-contiguous"):
        _cai(_FakeCuda((1, 48, 64), (48 * 64, 1, 48)))
    # the stride of a size-1 dimension is meaningless and may be anything
    assert _cai(_FakeCuda((1, 1620, 1920), (12345, 1920, 1)))[1] == (1, 1620, 1920)
    assert _cai(_FakeCuda((4, 1, 1920), (1920, 999, 1)))[1] == (4, 1, 1920)
    # wider elements, empty arrays
    assert _cai(_FakeCuda((3, 5), (20, 4), "<f4"))[2] == "<f4"
    with pytest.raises(RuntimeError, match="C-contiguous"):
        _cai(_FakeCuda((3, 5), (40, 8), "<f4"))
    assert _cai(_FakeCuda((0, 10, 10), (1, 1, 1)))[1] == (0, 10, 10)


def test_aspect_preserving_geometry_follows_the_reference_filter_strings():
    """``scale_mode`` mirrors ``force_original_aspect_ratio=decrease`` + ``pad=...:x=-1:y=-1`` and
    ``increase`` + ``crop`` (src/spdl/io/_preprocessing.py:214-229)."""
    ws, hs = [1280, 640, 100], [720, 480, 300]
    d, out = io.make_image_descs(ws, hs, resize=(256, 256), scale_mode="pad")
    assert out == (256, 256)
    # the fitted side is min(round(other * aspect), target)
    assert [int(v) for v in d["resized_w"]] == [256, 256, 85]
    assert [int(v) for v in d["resized_h"]] == [144, 192, 256]
    # centred with (canvas - image) // 2, on the chroma grid for 4:2:0 sources
    assert [int(v) for v in d["crop_y"]] == [-56, -32, 0]
    assert [int(v) for v in d["crop_x"]] == [0, 0, -84]
    assert np.float32(d["scale_x"][2]) == np.float32(100) / np.float32(85)
    d24, _ = io.make_image_descs(ws, hs, src_format="rgb24", resize=(256, 256), scale_mode="pad")
    assert [int(v) for v in d24["crop_x"]] == [0, 0, -85]  # (256 - 85) // 2, no chroma grid
    d, out = io.make_image_descs(ws, hs, resize=(256, 256), scale_mode="crop")
    assert out == (256, 256)
    assert [int(v) for v in d["resized_w"]] == [0, 0, 0]  # nothing lies outside the image
    assert [int(v) for v in d["crop_x"]] == [98, 42, 0]   # (455 - 256) // 2 = 99 -> even
    assert [int(v) for v in d["crop_y"]] == [0, 0, 256]   # (768 - 256) // 2
    assert np.float32(d["scale_x"][0]) == np.float32(1280) / np.float32(455)
    # a centre crop after the letterbox refers to the canvas
    d, out = io.make_image_descs(ws, hs, resize=(256, 256), scale_mode="pad", crop=(224, 224))
    assert out == (224, 224) and [int(v) for v in d["crop_y"]] == [16 - 56, 16 - 32, 16]
    with pytest.raises(ValueError):
        io.make_image_descs(ws, hs, resize=(256, 256), scale_mode="fit")
    with pytest.raises(RuntimeError):
        io.make_image_descs(ws, hs, resize_shorter=256, scale_mode="pad")


def test_touched_rows_of_the_benchmark_geometries():
    """The host helper that says which source rows a geometry reads (for row-sparse uploads)."""
    d, out = io.make_image_descs([3840], [2160], resize=(224, 224))
    luma, chroma = io.touched_rows(d[0], src_format="nv12", out_h=out[1])
    assert luma.shape == (2160,) and chroma.shape == (1080,)
    # 224 output rows read two luma rows each; the scale (9.64) keeps all pairs apart
    assert (luma >= 0).sum() == 448 and (chroma >= 0).sum() == 336
    kept = luma[luma >= 0]
    assert (kept == np.arange(448)).all()  # positions in a compacted copy, in row order
    # 0.24 of the frame's bytes
    assert abs(((luma >= 0).sum() + (chroma >= 0).sum()) / (2160 * 1.5) - 0.242) < 0.001
    d, out = io.make_image_descs([1280], [720], resize=(256, 256))
    luma, chroma = io.touched_rows(d[0], src_format="nv12", out_h=256)
    assert (luma >= 0).sum() == 512 and (chroma >= 0).sum() == 360
    # no resize: every row is read; upscaling too
    d, out = io.make_image_descs([64], [48], resize=(64, 48))
    luma, chroma = io.touched_rows(d[0], src_format="i420", out_h=48)
    assert (luma == np.arange(48)).all() and (chroma == np.arange(24)).all()
    # letterbox: rows of padding read nothing
    d, out = io.make_image_descs([1280], [720], resize=(64, 64), scale_mode="pad")
    luma, _ = io.touched_rows(d[0], src_format="nv12", out_h=64)
    assert (luma >= 0).sum() <= 2 * int(d["resized_h"][0])
    # RGB sources have no half-height planes
    d, out = io.make_image_descs([100], [80], src_format="rgb24", resize=(20, 10))
    luma, chroma = io.touched_rows(d[0], src_format="rgb24", out_h=10)
    assert chroma.size == 0 and (luma >= 0).sum() == 20
    bad = d.copy()
    bad["scale_y"] = 0.0
    with pytest.raises(RuntimeError):
        io.touched_rows(bad[0], src_format="rgb24", out_h=10)


@pytest.mark.parametrize("threads", ["1", "3", "8"])
@pytest.mark.parametrize("pitch_pad", [0, 48])
def test_copy_rows_large_batches_over_several_threads(monkeypatch, threads, pitch_pad):
    """Batches of more than a few MiB are cut into ranges for several host threads, and runs of
    consecutive rows of a tightly pitched source go as one copy: same bytes either way."""
    monkeypatch.setenv("B2_HOST_COPY_THREADS", threads)
    L = _lib.lib()
    rng = np.random.default_rng(11)
    n, rows_total, row_bytes = 5, 400, 4096
    pitch = row_bytes + pitch_pad
    src = rng.integers(0, 256, (n, rows_total, pitch), dtype=np.uint8)
    rows = np.sort(rng.choice(rows_total, 300, replace=False)).astype(np.int32)  # runs and gaps
    dst = np.full((n, len(rows) * row_bytes + 7), 0xA5, np.uint8)
    assert L.b2_copy_rows(dst.ctypes.data, dst.strides[0], src.ctypes.data, src.strides[0], pitch,
                          rows.ctypes.data, len(rows), row_bytes, n) == 0
    want = src[:, rows, :row_bytes].reshape(n, -1)
    assert (dst[:, :len(rows) * row_bytes] == want).all()
    assert (dst[:, len(rows) * row_bytes:] == 0xA5).all()
    # whole frames as one "row" each: the staging copy of a batch of frames
    frame = rows_total * pitch
    whole = np.zeros((n, frame), np.uint8)
    zero = np.zeros(1, np.int32)
    assert L.b2_copy_rows(whole.ctypes.data, frame, src.ctypes.data, frame, frame,
                          zero.ctypes.data, 1, frame, n) == 0
    assert (whole == src.reshape(n, -1)).all()


@pytest.mark.parametrize("threads", ["1", "5"])
def test_copy_host_and_the_arguments_of_the_staged_transfer(monkeypatch, threads):
    """``b2_copy_host`` moves every byte whatever the number of host threads;
    ``b2_transfer_h2d_staged`` rejects null pointers and a staging buffer without room for two
    halves before it makes any CUDA call."""
    monkeypatch.setenv("B2_HOST_COPY_THREADS", threads)
    L = _lib.lib()
    n = (9 << 20) + 4321
    src = np.random.default_rng(5).integers(0, 256, n, dtype=np.uint8)
    dst = np.zeros(n + 3, np.uint8)
    assert L.b2_copy_host(dst.ctypes.data, src.ctypes.data, n) == 0
    assert (dst[:n] == src).all() and (dst[n:] == 0).all()
    assert L.b2_copy_host(None, None, 0) == 0
    assert L.b2_copy_host(None, src.ctypes.data, 8) == 1
    assert L.b2_transfer_h2d_staged(None, None, 0, None, 0, 0, None) == 0  # nothing to do
    assert L.b2_transfer_h2d_staged(None, src.ctypes.data, 8, dst.ctypes.data, 1024, 0, None) == 1
    assert L.b2_transfer_h2d_staged(dst.ctypes.data, src.ctypes.data, 8, dst.ctypes.data, 300, 0,
                                    None) == 1
    assert b"staging" in L.b2_last_error()


@pytest.mark.parametrize("threads", ["1", "4"])
def test_pack_host_packs_items_of_different_sizes(monkeypatch, threads):
    """``b2_pack_host``: every item lands at its offset, nothing else is touched, whatever the
    number of host threads the items are dealt out to."""
    monkeypatch.setenv("B2_HOST_COPY_THREADS", threads)
    L = _lib.lib()
    rng = np.random.default_rng(8)
    items = [rng.integers(0, 256, int(k), dtype=np.uint8)
             for k in rng.integers(0, 3 << 20, 11)] + [np.zeros(0, np.uint8)]
    sizes = np.array([a.size for a in items], np.int64)
    offsets = np.zeros(len(items), np.int64)
    np.cumsum((sizes[:-1] + 15) & ~15, out=offsets[1:])
    total = int(offsets[-1] + sizes[-1])
    dst = np.full(total + 9, 0xA5, np.uint8)
    srcs = np.array([a.ctypes.data for a in items], np.uint64)
    assert L.b2_pack_host(dst.ctypes.data, srcs.ctypes.data, sizes.ctypes.data,
                          offsets.ctypes.data, len(items)) == 0
    covered = np.zeros(dst.size, bool)
    for a, o in zip(items, offsets):
        assert (dst[o:o + a.size] == a).all()
        covered[o:o + a.size] = True
    assert (dst[~covered] == 0xA5).all()
    assert L.b2_pack_host(None, None, None, None, 0) == 0
    sizes[2] = -1
    assert L.b2_pack_host(dst.ctypes.data, srcs.ctypes.data, sizes.ctypes.data,
                          offsets.ctypes.data, len(items)) == 1


def test_resize_host_images_rejects_what_it_cannot_batch():
    """Argument checks of ``resize_host_images`` come before any CUDA call."""
    import spdl_b200.io as io

    cfg = io.cuda_config(0)
    rgb = np.zeros((8, 6, 3), np.uint8)
    for images, kw in (([], {}),                                          # nothing to do
                       ([rgb], dict(src_format="gray8")),                # unknown format
                       ([rgb.astype(np.float32)], {}),                    # not bytes
                       ([rgb[..., :2]], {}),                              # two channels
                       ([np.zeros((9, 6), np.uint8)], dict(src_format="i420")),   # odd height
                       ([np.zeros((12, 7), np.uint8)], dict(src_format="nv12")),  # odd width
                       ([rgb], dict(src_format="i420"))):                # planes expected
        with pytest.raises(RuntimeError):
            io.resize_host_images(images, device_config=cfg, resize=(4, 4), **kw)


def test_copy_rows_packs_selected_rows_of_every_frame():
    """``b2_copy_rows``: the host-side packing step of a row-sparse upload (no CUDA call)."""
    L = _lib.lib()
    rng = np.random.default_rng(4)
    n, rows_total, pitch, row_bytes = 3, 20, 70, 64
    src = rng.integers(0, 256, (n, rows_total, pitch), dtype=np.uint8)
    rows = np.array([1, 2, 7, 19], np.int32)
    dst = np.full((n, len(rows) * row_bytes + 5), 0xA5, np.uint8)
    assert L.b2_copy_rows(dst.ctypes.data, dst.strides[0], src.ctypes.data, src.strides[0], pitch,
                          rows.ctypes.data, len(rows), row_bytes, n) == 0
    for f in range(n):
        assert (dst[f, :len(rows) * row_bytes].reshape(len(rows), row_bytes) ==
                src[f, rows, :row_bytes]).all()
        assert (dst[f, len(rows) * row_bytes:] == 0xA5).all()
    assert L.b2_copy_rows(None, 0, None, 0, 0, None, 0, 16, 2) == 0  # nothing to do
    assert L.b2_copy_rows(None, 0, src.ctypes.data, 0, 0, rows.ctypes.data, 4, 16, 2) == 1
    rows[1] = -3
    assert L.b2_copy_rows(dst.ctypes.data, dst.strides[0], src.ctypes.data, src.strides[0], pitch,
                          rows.ctypes.data, len(rows), row_bytes, n) == 1
    assert b"negative" in L.b2_last_error()
