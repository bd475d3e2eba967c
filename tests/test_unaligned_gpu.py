"""Frames whose rows start on arbitrary byte boundaries (widths that are not a multiple of 16):
the realigning rows kernel against the oracle, at real-world sizes."""

import numpy as np
import pytest

import oracle
from tests import synth

pytestmark = pytest.mark.gpu

MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)


@pytest.mark.parametrize("w,h", [(854, 480), (426, 240), (1918, 20), (1366, 18), (30, 6)])
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
