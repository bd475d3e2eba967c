"""``FrameStage`` as a stage of the reference's own ``spdl.pipeline.PipelineBuilder``
(src/spdl/pipeline/_builder.py; the shape of examples/video_classification/utils/pipeline.py):
``.pipe(stage, concurrency=2)`` on a pool of worker threads.

``spdl.pipeline`` is pure Python and is imported from the reference tree where that tree exists
(the ``REFERENCE_ROOT`` environment variable names it); the tests are skipped elsewhere.  The CPU test
replaces the three device calls of the stage with host stand-ins built on the oracle, so that the
packaging -- one object shared by all workers, per-thread state, ordered results, the keep-alive
window -- runs under the reference's executor without a GPU; the GPU test runs the real stage.
"""

import os
import sys
import threading
from pathlib import Path

import numpy as np
import pytest

import oracle
from tests import synth

_REF_SRC = Path(os.environ.get("REFERENCE_ROOT", "/root/reference")) / "src"


def _pipeline_builder():
    if not (_REF_SRC / "spdl" / "pipeline" / "__init__.py").exists():
        pytest.skip("the reference's spdl.pipeline is not on this machine")
    if str(_REF_SRC) not in sys.path:
        sys.path.append(str(_REF_SRC))  # after the repository root: only `spdl` comes from there
    from spdl.pipeline import PipelineBuilder

    return PipelineBuilder


MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)


def _batches(count, n, w, h):
    return [synth.i420_batch_gradient(n, w, h, config=1, index=i) for i in range(count)]


def _want(batch, resize, crop):
    import spdl_b200.io as io

    n, h2, w = batch.shape
    h = h2 * 2 // 3
    descs, out = io.make_image_descs([w] * n, [h] * n, src_format="i420", resize_shorter=resize,
                                     crop=crop)
    return oracle.convert_resize(batch.reshape(-1), descs.view(oracle.DESC_DTYPE), out_w=out[0],
                                 out_h=out[1], src_format=oracle.I420, dtype=oracle.F32,
                                 sb=oracle.scale_bias(MEAN, STD))


def test_stage_under_the_reference_pipeline_builder_host_stand_ins(monkeypatch):
    import torch

    import spdl_b200.io as io
    from spdl_b200.io import _stage

    PipelineBuilder = _pipeline_builder()
    threads_seen, streams_made = set(), []

    class HostBuffer:  # what the stand-in "device" hands around
        def __init__(self, array):
            self.array = np.ascontiguousarray(array)
            self.shape = self.array.shape

    def fake_transfer(buffer, *, device_config):
        threads_seen.add(threading.get_ident())
        return HostBuffer(np.array(buffer, copy=True))

    def fake_resize(base, descs, *, out_size, max_src_w, device_config, src_format, mean, std,
                    dtype, **kw):
        assert kw["sync"] is True and src_format == "i420" and dtype == "float32"
        table = descs.array.view(oracle.DESC_DTYPE).reshape(-1)
        return HostBuffer(oracle.convert_resize(
            base.array.reshape(-1), table, out_w=out_size[0], out_h=out_size[1],
            src_format=oracle.I420, dtype=oracle.F32, sb=oracle.scale_bias(mean, std)))

    class FakeStream:
        def __init__(self, device):
            streams_made.append(threading.get_ident())
            self.cuda_stream = 0x1000 + len(streams_made)

    monkeypatch.setattr(_stage, "transfer_buffer", fake_transfer)
    # no page-locked memory without a driver: the staging copy hands the frames through
    monkeypatch.setattr(_stage.FrameStage, "_stage_whole", lambda self, st, frames: frames)
    monkeypatch.setattr(_stage, "convert_resize", fake_resize)
    monkeypatch.setattr(_stage, "to_torch", lambda buf, dtype=None: torch.from_numpy(buf.array))
    monkeypatch.setattr(torch.cuda, "Stream", FakeStream)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 1)

    stage = io.FrameStage(src_format="i420", dtype="float32", mean=MEAN, std=STD,
                          resize_shorter=24, crop=(20, 20), num_caches=2)
    batches = _batches(64, 2, 64, 36)
    pipeline = (PipelineBuilder()
                .add_source(range(len(batches)))
                .pipe(lambda i: batches[i])            # stands in for decode + convert_frames
                .pipe(stage, concurrency=2, output_order="input")
                .add_sink(3)
                .build(num_threads=4))
    with pipeline.auto_stop():
        results = list(pipeline.get_iterator())
    assert len(results) == 64
    for i, got in enumerate(results):  # results arrive in source order
        assert tuple(got.shape) == (2, 3, 20, 20)
        np.testing.assert_array_equal(got.numpy(), _want(batches[i], 24, (20, 20)))
    # the one stage object served several worker threads, each with a stream of its own
    assert len(threads_seen) >= 2
    assert sorted(streams_made) == sorted(threads_seen)
    # every thread uploaded its descriptor table once, not per call
    assert len(streams_made) <= 4


@pytest.mark.gpu
def test_stage_under_the_reference_pipeline_builder_on_the_gpu():
    import torch

    import spdl_b200.io as io

    PipelineBuilder = _pipeline_builder()
    stage = io.FrameStage(src_format="i420", dtype="float32", mean=MEAN, std=STD,
                          resize_shorter=96, crop=(80, 80), num_caches=2)
    batches = _batches(64, 4, 320, 180)
    seen = set()

    def staged(batch):
        seen.add(threading.get_ident())
        return stage(batch)

    pipeline = (PipelineBuilder()
                .add_source(range(len(batches)))
                .pipe(lambda i: batches[i])
                .pipe(staged, concurrency=2, output_order="input")
                .add_sink(3)
                .build(num_threads=4))
    with pipeline.auto_stop():
        results = [t.cpu().numpy() for t in pipeline.get_iterator()]
    assert len(results) == 64 and len(seen) >= 2
    for i, got in enumerate(results):
        np.testing.assert_allclose(got, _want(batches[i], 96, (80, 80)), rtol=1e-5, atol=1e-5)
    torch.cuda.synchronize()
