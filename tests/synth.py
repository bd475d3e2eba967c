"""Seeded synthetic inputs with the shapes and value distributions of the benchmark workloads.

No dataset is involved anywhere: every workload is generated from
``numpy.random.default_rng(1000 * config + index)``.  Used by the tests, by ``bench.py`` and by
``tests/golden/make_golden.py``.
"""

from __future__ import annotations

import numpy as np


def rng_for(config: int, index: int = 0) -> np.random.Generator:
    return np.random.default_rng(1000 * config + index)


def nv12_batch(n: int, w: int, h: int, *, config: int = 2, index: int = 0,
               full_range: bool = False) -> np.ndarray:
    """``[n, h*3/2, w]`` u8: Y uniform in [16,235], interleaved UV uniform in [16,240]
    (or 0..255 for both when ``full_range``)."""
    r = rng_for(config, index)
    out = np.empty((n, h + h // 2, w), np.uint8)
    ylo, yhi, clo, chi = (0, 256, 0, 256) if full_range else (16, 236, 16, 241)
    out[:, :h] = r.integers(ylo, yhi, (n, h, w), dtype=np.uint8)
    out[:, h:] = r.integers(clo, chi, (n, h // 2, w), dtype=np.uint8)
    return out


def i420_batch_gradient(n: int, w: int, h: int, *, config: int = 1, index: int = 0) -> np.ndarray:
    """``[n, h*3/2, w]`` u8 in I420 order (Y rows, U block, V block).  Y is a smooth diagonal
    gradient plus uniform noise in [-8, 8] clipped to [16,235]; U, V uniform in [16,240]."""
    r = rng_for(config, index)
    yy, xx = np.mgrid[0:h, 0:w]
    grad = 16.0 + 219.0 * (xx + yy) / float(w + h - 2)
    out = np.empty((n, h + h // 2, w), np.uint8)
    noise = r.integers(-8, 9, (n, h, w))
    out[:, :h] = np.clip(np.rint(grad)[None] + noise, 16, 235).astype(np.uint8)
    out[:, h:] = r.integers(16, 241, (n, h // 2, w), dtype=np.uint8)
    return out


def nv12_clip(t: int, w: int, h: int, *, config: int = 4, index: int = 0) -> np.ndarray:
    """``[t, h*3/2, w]`` u8: frame 0 as :func:`nv12_batch`; each later frame is the previous
    one plus rounded Gaussian noise (sigma 4), clipped to [16,235] (Y) / [16,240] (UV)."""
    r = rng_for(config, index)
    out = np.empty((t, h + h // 2, w), np.uint8)
    out[0, :h] = r.integers(16, 236, (h, w), dtype=np.uint8)
    out[0, h:] = r.integers(16, 241, (h // 2, w), dtype=np.uint8)
    for i in range(1, t):
        step = np.rint(r.normal(0.0, 4.0, (h + h // 2, w))).astype(np.int16)
        nxt = out[i - 1].astype(np.int16) + step
        out[i, :h] = np.clip(nxt[:h], 16, 235)
        out[i, h:] = np.clip(nxt[h:], 16, 240)
    return out


def ragged_i420(n: int, *, lo: int = 256, hi: int = 1024, config: int = 5,
                index: int = 0) -> tuple[np.ndarray, np.ndarray, np.ndarray, np.ndarray]:
    """``n`` I420 images with even width/height uniform in [lo, hi], values uniform in 0..255,
    packed back to back.  Returns ``(bytes, widths, heights, offsets)``."""
    r = rng_for(config, index)
    ws = r.integers(lo // 2, hi // 2 + 1, n) * 2
    hs = r.integers(lo // 2, hi // 2 + 1, n) * 2
    sizes = ws * hs * 3 // 2
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int64)
    data = r.integers(0, 256, int(sizes.sum()), dtype=np.uint8)
    return data, ws.astype(np.int64), hs.astype(np.int64), offs


def exhaustive_nv12() -> np.ndarray:
    """One NV12 frame ``[1, 24576, 1024]`` that contains every (Y,U,V) triple exactly once.

    Quad ``q = (u*256 + v)*64 + k`` sits at quad column ``q % 512``, quad row ``q // 512``; its
    four luma samples (row-major inside the quad) are ``4k .. 4k+3`` and its chroma is (u, v).
    """
    W, QW = 1024, 512
    nq = 256 * 256 * 64
    H = 2 * (nq // QW)
    q = np.arange(nq, dtype=np.int64)
    k = (q % 64).astype(np.uint8)
    uv = q // 64
    u, v = (uv // 256).astype(np.uint8), (uv % 256).astype(np.uint8)
    frame = np.empty((H + H // 2, W), np.uint8)
    yq = frame[:H].reshape(H // 2, 2, QW, 2)
    kk = (4 * k).reshape(H // 2, QW)
    yq[:, 0, :, 0] = kk
    yq[:, 0, :, 1] = kk + 1
    yq[:, 1, :, 0] = kk + 2
    yq[:, 1, :, 1] = kk + 3
    c = frame[H:].reshape(H // 2, QW, 2)
    c[:, :, 0] = u.reshape(H // 2, QW)
    c[:, :, 1] = v.reshape(H // 2, QW)
    return frame[None]


def exhaustive_lookup(planar: np.ndarray) -> np.ndarray:
    """Rearrange the ``[1,3,16384,1024]`` conversion of :func:`exhaustive_nv12` into the
    ``[256(y),256(u),256(v),3]`` table layout of ``oracle.exhaustive``."""
    H = planar.shape[2]
    t = planar[0].reshape(3, H // 2, 2, 512, 2).transpose(1, 3, 2, 4, 0)  # [qrow,qcol,r,c,ch]
    t = t.reshape(256, 256, 64, 4, 3)  # [u, v, k, sample, ch]; y = 4k + sample
    return np.ascontiguousarray(t.reshape(256, 256, 256, 3).transpose(2, 0, 1, 3))
