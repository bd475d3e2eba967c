"""Generates the golden fixtures of ``tests/golden`` by running the REFERENCE's own kernel.

Needs a GPU and ``oracle/_ref/libspdl_ref_nv12.so`` (the reference's
``src/libspdl/cuda/detail/color_conversion.cu`` compiled unmodified by ``make -C oracle ref``).

    python tests/golden/make_golden.py [OUT_DIR]

Writes
  ref_kernel_golden.json   sha256 of the reference kernel's output over the frame that holds
                           every (Y,U,V) triple once (``tests.synth.exhaustive_nv12``), for each
                           matrix index 0..11 and both channel orders; plus, for each, which of
                           the oracle's multiply-add fusion orders reproduce it exactly.
  ref_kernel_small.npz     inputs and reference-kernel outputs for small seeded batches, including
                           an odd width and a non-multiple-of-16 width.
"""

from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402
from tests import synth  # noqa: E402


def run_ref(nv12: np.ndarray, coeff: int, bgr: bool) -> np.ndarray:
    import torch

    ref = oracle.ref_kernel()
    assert ref is not None, "build oracle/_ref first (make -C oracle ref)"
    n, h2, w = nv12.shape
    h = h2 // 3 * 2
    src = torch.from_numpy(nv12).cuda()
    dst = torch.zeros((n, 3, h, w), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    fn = ref.ref_nv12_to_planar_bgr if bgr else ref.ref_nv12_to_planar_rgb
    rc = fn(stream, src.data_ptr(), w, dst.data_ptr(), w, w, h, n, coeff)
    assert rc == 0
    torch.cuda.synchronize()
    return dst.cpu().numpy()


def main() -> None:
    out_dir = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parent
    out_dir.mkdir(parents=True, exist_ok=True)
    ex = synth.exhaustive_nv12()
    meta: dict = {"exhaustive_sha256": {}, "oracle_mode_exact": {}, "mismatch_fraction": {}}
    for coeff in range(0, 12):
        for bgr in (False, True):
            got = run_ref(ex, coeff, bgr)
            key = f"{'bgr' if bgr else 'rgb'}_{coeff}"
            meta["exhaustive_sha256"][key] = hashlib.sha256(got.tobytes()).hexdigest()
            if not bgr:
                exact, frac = [], {}
                for mode in (oracle.FMA_NONE, oracle.FMA_LUMA_FIRST, oracle.FMA_CHROMA_FIRST,
                             oracle.FMA_DEVICE):
                    want = oracle.nv12_to_planar(ex, coeff=coeff, mode=mode)
                    bad = float((want != got).mean())
                    frac[str(mode)] = bad
                    if bad == 0.0:
                        exact.append(mode)
                meta["oracle_mode_exact"][key] = exact
                meta["mismatch_fraction"][key] = frac
    small = {}
    for name, (n, w, h) in {"a": (3, 64, 36), "b": (2, 50, 22), "c": (1, 33, 10),
                            "d": (2, 1920, 8)}.items():
        nv = synth.nv12_batch(n, w, h, config=9, index=len(small), full_range=True)
        small[f"{name}_in"] = nv
        for coeff in (1, 6, 9):
            small[f"{name}_rgb_{coeff}"] = run_ref(nv, coeff, False)
        small[f"{name}_bgr_1"] = run_ref(nv, 1, True)
    np.savez_compressed(out_dir / "ref_kernel_small.npz", **small)
    (out_dir / "ref_kernel_golden.json").write_text(json.dumps(meta, indent=1, sort_keys=True))
    print(json.dumps(meta["oracle_mode_exact"]))


if __name__ == "__main__":
    main()
