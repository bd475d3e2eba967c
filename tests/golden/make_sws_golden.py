"""Generates ``sws_golden.json`` / ``sws_small.npz``: outputs of the libswscale that ships inside
the opencv wheel (FFmpeg 8 ABI), the library the reference's CPU route converts colours with.

    python tests/golden/make_sws_golden.py

For each of BT.709 and BT.601, limited and full range, one frame that holds every (Y,U,V) triple
is converted yuv420p -> rgb24 by ``sws_scale`` and the resulting ``[256,256,256,3]`` table is
hashed; the colourspace table of ``sws_getCoefficients`` and two small raw frames are stored too.
The oracle's restatement of that arithmetic is tested against these files, so the test-suite does
not need the library to be present.
"""

from __future__ import annotations

import ctypes
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from oracle import swscale_ref  # noqa: E402
from tests import synth  # noqa: E402


def exhaustive_i420() -> tuple[np.ndarray, int, int]:
    """The all-triples NV12 frame of ``synth.exhaustive_nv12`` with planar chroma."""
    nv = synth.exhaustive_nv12()[0]
    w = nv.shape[1]
    h = nv.shape[0] * 2 // 3
    uv = nv[h:].reshape(h // 2, w // 2, 2)
    out = np.empty((h * 3 // 2, w), np.uint8)
    out[:h] = nv[:h]
    flat = out.reshape(-1)
    flat[h * w:h * w + (h // 2) * (w // 2)] = uv[:, :, 0].reshape(-1)
    flat[h * w + (h // 2) * (w // 2):] = uv[:, :, 1].reshape(-1)
    return out, w, h


def library_table(cs: int, full: bool) -> np.ndarray:
    frame, w, h = exhaustive_i420()
    conv = swscale_ref.I420ToRGB(w, h, cs, full_range=full)
    rgb = np.empty((h, w, 3), np.uint8)
    conv(frame, rgb)
    return synth.exhaustive_lookup(np.ascontiguousarray(rgb.transpose(2, 0, 1))[None])


def main() -> None:
    sws = swscale_ref.load()
    if sws is None:
        raise SystemExit("libswscale not found")
    sws.swscale_version.restype = ctypes.c_uint
    ver = sws.swscale_version()
    gold = {"library": f"libswscale {ver >> 16}.{(ver >> 8) & 255}.{ver & 255}",
            "coefficients": {}, "tables_sha256": {}, "triplets": {}}
    for cs in range(12):
        c = sws.sws_getCoefficients(cs)
        gold["coefficients"][str(cs)] = [int(c[i]) for i in range(4)]
    for cs, full in ((1, False), (5, False), (5, True), (1, True), (9, False), (7, True)):
        t = library_table(cs, full)
        gold["tables_sha256"][f"{cs}_{int(full)}"] = hashlib.sha256(t.tobytes()).hexdigest()
        if (cs, full) == (1, False):
            # the YUV triplets behind tests/cuda/nvdec_video_decoding_test.py:335-348
            for yuv in ((81, 90, 240), (145, 54, 34), (41, 240, 110)):
                gold["triplets"]["%d,%d,%d" % yuv] = [int(v) for v in t[yuv]]
    (HERE / "sws_golden.json").write_text(json.dumps(gold, indent=1) + "\n")
    small = {}
    for name, cs, full, seed in (("bt709_limited", 1, False, 7), ("bt601_full", 5, True, 8)):
        w, h = 64, 36
        frame = synth.nv12_batch(1, w, h, config=9, index=seed, full_range=full)[0]
        conv = swscale_ref.I420ToRGB(w, h, cs, full_range=full)
        rgb = np.empty((h, w, 3), np.uint8)
        conv(frame, rgb)  # the bytes are read as I420: Y rows, U block, V block
        small[name + "_i420"] = frame
        small[name + "_rgb"] = rgb
    np.savez_compressed(HERE / "sws_small.npz", **small)
    print(json.dumps(gold["tables_sha256"], indent=1))


if __name__ == "__main__":
    main()
