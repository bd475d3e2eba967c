"""Buffer transfer, storage, allocator accounting and array-interface contracts on a GPU.

Modelled on the reference's tests/cuda/buffer_transfer_test.py, tests/cuda/pin_memory_test.py,
tests/cuda/transfer_test.py and tests/io/buffer_conversion_refcount_test.py.
"""

import gc
import sys

import numpy as np
import pytest

import oracle
from tests import synth

pytestmark = pytest.mark.gpu


def _frames(n=4, w=32, h=16):
    import spdl_b200.io as io

    rng = np.random.default_rng(0)
    planes = [[rng.integers(0, 256, (h, w * 3 + 5), dtype=np.uint8)] for _ in range(n)]
    return io.Frames("rgb24", w, h, planes), planes


def test_h2d_of_converted_frames_equals_cpu(cuda_cfg):
    import spdl_b200.io as io

    frames, planes = _frames()
    cpu = io.convert_frames(frames)
    dev = io.transfer_buffer(cpu, device_config=cuda_cfg)
    t = io.to_torch(dev)
    assert t.is_cuda and tuple(t.shape) == (4, 16, 32, 3)
    assert (t.cpu().numpy() == io.to_numpy(cpu)).all()
    assert (io.to_numpy(cpu)[2] == planes[2][0][:, :96].reshape(16, 32, 3)).all()


def test_custom_allocator_is_called_and_deleter_runs_on_gc():
    import torch

    import spdl_b200.io as io

    calls = {"alloc": 0, "free": 0}

    def alloc(size, device, stream):
        calls["alloc"] += 1
        assert device == 0 and size > 0
        return torch.cuda.caching_allocator_alloc(size, device, stream)

    def free(ptr):
        calls["free"] += 1
        torch.cuda.caching_allocator_delete(ptr)

    cfg = io.cuda_config(0, stream=torch.cuda.current_stream().cuda_stream,
                         allocator=(alloc, free))
    buf = io.transfer_buffer(np.arange(100, dtype=np.int32), device_config=cfg)
    assert calls == {"alloc": 1, "free": 0}
    nv = torch.zeros((2, 6, 8), dtype=torch.uint8, device="cuda")
    out = io.nv12_to_rgb(nv, device_config=cfg, sync=True)
    assert calls == {"alloc": 2, "free": 0}
    del buf
    gc.collect()
    assert calls["free"] == 1
    t = io.to_torch(out)
    del out
    gc.collect()
    assert calls["free"] == 1  # the tensor keeps the buffer alive
    del t
    gc.collect()
    assert calls["free"] == 2


def test_allocator_that_raises_propagates():
    import spdl_b200.io as io

    def alloc(size, device, stream):
        raise MemoryError("no memory today")

    cfg = io.cuda_config(0, allocator=(alloc, lambda p: None))
    with pytest.raises(MemoryError):
        io.transfer_buffer(np.zeros(4, np.uint8), device_config=cfg)


@pytest.mark.parametrize("dtype", [np.uint8, np.int32, np.int64, np.float32])
def test_array_round_trip(cuda_cfg, dtype):
    import torch

    import spdl_b200.io as io

    a = (np.arange(2 * 3 * 5) * 7 % 251).astype(dtype).reshape(2, 3, 5)
    for src in (a, torch.from_numpy(a)):
        dev = io.transfer_buffer(src, device_config=cuda_cfg)
        assert dev.device_index == 0
        iface = dev.__cuda_array_interface__
        assert iface["version"] == 2 and iface["shape"] == (2, 3, 5)
        assert iface["strides"] is None and iface["data"][1] is False
        assert iface["stream"] == cuda_cfg.stream
        assert iface["typestr"] == f"|{np.dtype(dtype).kind}{np.dtype(dtype).itemsize}"
        t = io.to_torch(dev)
        assert t.data_ptr() == iface["data"][0]
        assert t.dtype == torch.from_numpy(a).dtype
        assert (t.cpu().numpy() == a).all()
        back = io.to_numpy(io.transfer_buffer_cpu(dev))
        assert back.dtype == a.dtype and (back == a).all()


@pytest.mark.parametrize("nbytes", [8 << 20, (40 << 20) + 12345])
def test_large_pageable_arrays_go_through_the_staging_buffer(cuda_cfg, nbytes):
    """From 8 MiB on a pageable source is staged in halves of this thread's page-locked buffer
    under the uploads of the other half; the data arrives unchanged."""
    import torch

    import spdl_b200.io as io

    a = np.random.default_rng(nbytes & 0xFFFF).integers(0, 256, nbytes, dtype=np.uint8)
    dev = io.transfer_buffer(a, device_config=cuda_cfg)
    assert (io.to_torch(dev).cpu().numpy() == a).all()
    if nbytes % 4 == 0:  # a pageable torch tensor of another element type takes the same route
        t = torch.from_numpy(a.view(np.int32))
        assert torch.equal(io.to_torch(io.transfer_buffer(t, device_config=cuda_cfg)).cpu(), t)


def test_staged_transfer_with_a_tiny_staging_buffer(cuda_cfg):
    """``b2_transfer_h2d_staged`` through the C ABI with halves of 512 bytes: many chunks, a
    ragged last one, both halves reused."""
    import ctypes

    import torch

    from spdl_b200 import _lib

    L = _lib.lib()
    a = np.random.default_rng(3).integers(0, 256, 5000, dtype=np.uint8)
    staging = ctypes.c_void_p()
    _lib.check(L.b2_alloc_pinned(ctypes.byref(staging), 1100))
    try:
        dst = torch.zeros(5000 + 16, dtype=torch.uint8, device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(L.b2_transfer_h2d_staged(dst.data_ptr(), a.ctypes.data, a.size, staging, 1100, 0,
                                            stream))
        got = dst.cpu().numpy()
        assert (got[:5000] == a).all() and (got[5000:] == 0).all()
    finally:
        _lib.check(L.b2_free_pinned(staging))


def test_large_device_arrays_come_back_through_the_staging_buffer(cuda_cfg):
    """``transfer_buffer_cpu`` of 8 MiB and more downloads in halves of this thread's
    page-locked buffer under the copies out; and the C entry point with halves of 512 bytes."""
    import ctypes

    import torch

    import spdl_b200.io as io
    from spdl_b200 import _lib

    n = (24 << 20) + 777
    t = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    back = io.to_numpy(io.transfer_buffer_cpu(t))
    assert back.shape == (n,) and (back == t.cpu().numpy()).all()

    L = _lib.lib()
    staging = ctypes.c_void_p()
    _lib.check(L.b2_alloc_pinned(ctypes.byref(staging), 1100))
    try:
        host = np.full(5000 + 16, 0xA5, np.uint8)
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(L.b2_transfer_d2h_staged(host.ctypes.data, t.data_ptr(), 5000, staging, 1100,
                                            0, stream))
        assert (host[:5000] == back[:5000]).all() and (host[5000:] == 0xA5).all()
        assert L.b2_transfer_d2h_staged(host.ctypes.data, t.data_ptr(), 8, staging, 100, 0,
                                        stream) == 1
    finally:
        _lib.check(L.b2_free_pinned(staging))


def test_non_contiguous_inputs(cuda_cfg):
    import torch

    import spdl_b200.io as io

    a = np.arange(4 * 6 * 8, dtype=np.int32).reshape(4, 6, 8)
    for view in (a[:, ::2], a.transpose(2, 0, 1), a[1:3, 1:5, ::3]):
        dev = io.transfer_buffer(view, device_config=cuda_cfg)
        assert (io.to_torch(dev).cpu().numpy() == view).all()
        dev = io.transfer_buffer(torch.from_numpy(a)[:, ::2], device_config=cuda_cfg)
        assert (io.to_torch(dev).cpu().numpy() == a[:, ::2]).all()


def test_many_transfers(cuda_cfg):
    import spdl_b200.io as io

    a = np.random.default_rng(1).integers(0, 255, (64, 64), dtype=np.uint8)
    for _ in range(100):
        assert (io.to_torch(io.transfer_buffer(a, device_config=cuda_cfg)).cpu().numpy() == a).all()


@pytest.mark.parametrize("pin", [True, False])
def test_storage_convert_transfer_on_torch_stream(pin):
    import torch

    import spdl_b200.io as io

    frames, _ = _frames(3, 40, 20)
    want = io.to_numpy(io.convert_frames(frames)).copy()
    storage = io.cpu_storage(3 * 20 * 40 * 3, pin_memory=pin)
    cpu = io.convert_frames(frames, storage=storage)
    assert cpu.is_pinned() == pin
    stream = torch.cuda.Stream(device=0)
    cfg = io.cuda_config(0, stream=stream.cuda_stream)
    dev = io.transfer_buffer(cpu, device_config=cfg)
    assert (io.to_torch(dev).cpu().numpy() == want).all()
    with pytest.raises(RuntimeError):
        io.convert_frames(frames, storage=io.cpu_storage(100, pin_memory=pin))


def test_buffer_outlives_its_variable(cuda_cfg):
    import spdl_b200.io as io

    a = np.arange(64, dtype=np.int64)
    dev = io.transfer_buffer(a, device_config=cuda_cfg)
    before = sys.getrefcount(dev)
    t = io.to_torch(dev)
    assert sys.getrefcount(dev) == before + 1
    del dev
    gc.collect()
    assert (t.cpu().numpy() == a).all()


def test_zero_element_buffers(cuda_cfg):
    import spdl_b200.io as io

    with pytest.raises(RuntimeError):
        io.transfer_buffer(np.zeros((0, 3), np.uint8), device_config=cuda_cfg)

    class Empty:
        device_index = 0
        __cuda_array_interface__ = {"version": 2, "shape": (0, 4), "typestr": "|u1",
                                    "data": (0, False), "strides": None}

    with pytest.raises(ValueError):
        io.to_torch(Empty())


def test_transfer_tensor_large(cuda_cfg):
    """tests/cuda/transfer_test.py of the reference, at a smaller but still multi-MB size."""
    import torch

    import spdl_b200.io as io

    x = torch.randint(0, 256, (4, 3, 1152, 1332), dtype=torch.uint8)
    out = io.transfer_tensor({"a": x, "b": [x[:1], "label"]})
    assert out["a"].is_cuda and torch.equal(out["a"].cpu(), x)
    assert out["b"][1] == "label" and torch.equal(out["b"][0].cpu(), x[:1])


def test_frame_batcher_matches_gather_oracle(cuda_cfg):
    """Pitched surfaces -> packed batches of 3, with a short last batch, then conversion."""
    import torch

    import spdl_b200.io as io

    w, h, pitch, total = 100, 36, 256, 8
    h2 = h * 3 // 2
    rng = np.random.default_rng(9)
    host = [rng.integers(0, 256, (h2, pitch), dtype=np.uint8) for _ in range(total)]
    dev = [torch.from_numpy(s).cuda() for s in host]
    fb = io.FrameBatcher(3, w, h, cuda_cfg)
    assert fb.empty()
    with pytest.raises(RuntimeError):
        fb.pop()
    for d in dev:
        fb.push(d.data_ptr(), pitch)
    fb.flush()
    shapes, got = [], []
    while not fb.empty():
        b = fb.pop()
        shapes.append(b.shape)
        got.append(io.to_torch(b).cpu().numpy())
    assert shapes == [(3, h2, w), (3, h2, w), (2, h2, w)]
    want = oracle.gather_frames(host, w, h)
    assert (np.concatenate(got) == want).all()
    rgb = io.nv12_to_rgb(torch.from_numpy(np.concatenate(got)).cuda(), device_config=cuda_cfg,
                         sync=True)
    assert (io.to_torch(rgb).cpu().numpy() == oracle.nv12_to_planar(want)).all()


def test_checksum_kernel_matches_oracle(cuda_cfg):
    import torch

    import spdl_b200.io as io

    a = np.random.default_rng(4).integers(0, 256, (5, 70001), dtype=np.uint8)
    got = io.frame_checksum(torch.from_numpy(a).cuda(), device_config=cuda_cfg)
    assert [int(x) for x in got] == [oracle.checksum(a[i]) for i in range(5)]


def test_frame_stage_from_worker_threads():
    """The pipeline stage: host yuv420p frames (as convert_frames lays them out) -> normalised
    tensor, called concurrently from four threads; dense and resizing variants."""
    import threading

    import torch

    import spdl_b200.io as io

    mean, std = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
    n, w, h = 3, 64, 48
    i420 = synth.i420_batch_gradient(n, w, h, config=1, index=2)
    flat = i420.reshape(-1)
    kw = dict(width=w, height=h, num_frames=n, y_pitch=w, uv_pitch=w // 2,
              y_frame_stride=h * 3 // 2 * w, uv_frame_stride=h * 3 // 2 * w,
              src_format=oracle.I420)
    u, v = flat[h * w:], flat[h * w + (h // 2) * (w // 2):]
    want_dense = oracle.convert_dense(i420, u, v, dtype=oracle.F32,
                                      sb=oracle.scale_bias(mean, std), **kw)
    descs, out = io.make_image_descs([w] * n, [h] * n, src_format="i420", resize_shorter=32,
                                     crop=(24, 24))
    want_small = oracle.convert_resize(flat, descs, out_w=24, out_h=24, src_format=oracle.I420,
                                       dtype=oracle.BF16, sb=oracle.scale_bias(mean, std))
    dense = io.FrameStage(mean=mean, std=std)
    small = io.FrameStage(dtype="bfloat16", mean=mean, std=std, resize_shorter=32, crop=(24, 24))
    # a CPUBuffer shaped like convert_frames' yuv420p output: [N, 1, H*1.5, W], pinned
    frames = io.Frames("yuv420p", w, h, [[i420[i, :h], i420[i, h:].reshape(-1)[:(h // 2) * (w // 2)]
                                          .reshape(h // 2, w // 2),
                                          i420[i, h:].reshape(-1)[(h // 2) * (w // 2):]
                                          .reshape(h // 2, w // 2)] for i in range(n)])
    host = io.convert_frames(frames, storage=io.cpu_storage(i420.nbytes))
    assert host.shape == (n, 1, h * 3 // 2, w)
    errors = []

    def work():
        try:
            for _ in range(5):
                a = dense(host)
                b = small(i420)
                assert a.dtype == torch.float32 and tuple(a.shape) == (n, 3, h, w)
                np.testing.assert_allclose(a.cpu().numpy(), want_dense, rtol=1e-6, atol=1e-6)
                assert b.dtype == torch.bfloat16 and tuple(b.shape) == (n, 3, 24, 24)
                got = b.view(torch.uint16).cpu().numpy()
                assert (got == want_small).mean() > 0.999
        except Exception as e:  # pragma: no cover
            errors.append(e)

    threads = [threading.Thread(target=work) for _ in range(4)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert not errors, errors
    with pytest.raises(RuntimeError):
        dense(np.zeros((2, 7, 8), np.uint8))
    with pytest.raises(RuntimeError):
        io.FrameStage(crop=(8, 8))


def test_convert_array_through_pinned_storage_to_the_gpu(cuda_cfg):
    """tests/cuda/pin_memory_test.py:77-98 of the reference: int64 labels -> pinned CPUBuffer ->
    transfer_buffer -> tensor on the device; a storage that is too small is an error."""
    import torch

    import spdl_b200.io as io

    vals = np.arange(0, 10)
    storage = io.cpu_storage(vals.nbytes, pin_memory=True)
    buffer = io.convert_array(vals, storage=storage)
    assert buffer.is_pinned()
    tensor = io.to_torch(io.transfer_buffer(buffer, device_config=cuda_cfg))
    assert tensor.shape == (10,) and tensor.dtype == torch.int64
    assert tensor.device == torch.device(f"cuda:{cuda_cfg.device_index}")
    assert (vals == tensor.cpu().numpy()).all()
    with pytest.raises(RuntimeError):
        io.convert_array(vals, storage=io.cpu_storage(vals.nbytes // 2, pin_memory=True))
