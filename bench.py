"""Benchmark of the post-decode frame path: 1080p NV12 -> interleaved RGB, frames/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--scaling weak|strong] [--workload c2|c3|c4|c5|j5|aux] [--scale F]
                    [--repeats R] [--arith reference|swscale] [--kernel-only] [--no-numa]

One "step" converts one batch of 64 synthetic 1920x1080 NV12 frames (BT.709 limited range) to
interleaved RGB u8 with a single kernel launch.  Inputs are seeded synthetic frames with the
workload's value distributions (Y uniform in [16,235], UV uniform in [16,240]); no dataset is
involved.  For N > 1 launch with ``torch.distributed.run``; every rank converts its own 64
frames per step on its own GPU (weak scaling, no collective on the data path).

Prints one JSON line (rank 0).  ``value`` is frames/s with inputs resident in HBM; ``e2e`` is the
same metric through the public API from pinned host memory; ``roofline`` relates the kernel to
the measured HBM copy bandwidth; ``cpu_baseline`` times the reference's CPU arithmetic on a
bounded sample on this machine's cores.  ``--impl reference`` times only that CPU path.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_FRAMES, W, H = 64, 1920, 1080
SCALING = "weak"
FRAME_IN = W * H * 3 // 2
FRAME_OUT = W * H * 3
ALGO_BYTES_PER_FRAME = FRAME_IN + FRAME_OUT  # 9,331,200
METRIC = "1080p NV12->RGB frames/s"
WORKLOAD = "64 x 1920x1080 NV12 -> interleaved RGB u8 (NHWC), BT.709 limited range"
ROTATE = 4  # distinct input batches cycled through, so no step finds its input in L2

#: what both arms print as ``config`` (the driver compares the two dicts)
CONFIG = {"workload": WORKLOAD, "frames_per_step_per_gpu": N_FRAMES}
DENSE_PROFILE = ROOT / "profiles" / "dense_nhwc_u8_1080p_x64.md"


def ncu_traffic_bytes_per_launch() -> int:
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dense kernel on this
    workload, read from the committed ncu summary of this very workload (its
    ``traffic_bytes_per_launch:`` line), so that the figure cannot drift from the evidence."""
    import re

    m = re.search(r"^traffic_bytes_per_launch:\s*([0-9_,]+)", DENSE_PROFILE.read_text(), re.M)
    if m is None:
        raise SystemExit(f"{DENSE_PROFILE} has no traffic_bytes_per_launch line")
    return int(m.group(1).replace(",", "").replace("_", ""))


def measured_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi.  The process is started early
    (it needs a second or more to come up on a box with many GPUs); ``begin``/``end`` mark the
    timed region and ``summary`` reports the samples taken between the marks."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.proc, self.samples = index, None, []  # samples: (host time, fields)
        self.t0 = self.t1 = None
        self.extended = False

    def start(self) -> "ClockSampler":
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            f = line.strip().split(", ")
            if len(f) >= 6 and f[0].isdigit():
                self.samples.append((time.perf_counter(), f))

    def wait_ready(self, timeout: float = 20.0) -> None:
        t = time.perf_counter()
        while self.proc is not None and not self.samples and time.perf_counter() - t < timeout:
            time.sleep(0.01)

    def begin(self) -> None:
        self.t0 = time.perf_counter()

    def end(self) -> None:
        self.t1 = time.perf_counter()

    def in_window(self) -> list:
        if self.t0 is None or self.t1 is None:
            return []
        return [f for t, f in self.samples if self.t0 <= t <= self.t1]

    def stop(self) -> None:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.proc = None

    def __enter__(self):
        self.start().wait_ready()
        self.begin()
        return self

    def __exit__(self, *a):
        self.end()
        self.stop()

    def summary(self) -> dict | None:
        rows = self.in_window()
        if not rows:
            return None
        sm = sorted(int(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].strip() == "Active" for r in rows)]
        out = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(rows[0][1]), "samples": len(rows),
               "window_ms": round(1e3 * (self.t1 - self.t0), 1), "reasons": reasons}
        if self.extended:
            out["window"] = ("timed steps plus untimed repeats of the same steps (the timed region "
                             "is shorter than three sampling periods)")
        return out


# ---- the reference's CPU path -------------------------------------------------------------------


def cpu_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def make_cpu_runner(frames: int):
    """Returns (run_once, kind, description) converting ``frames`` 1080p I420 frames to rgb24 into
    one contiguous buffer with all host cores."""
    from oracle import swscale_ref
    from tests import synth

    cores = cpu_cores()
    batch = synth.i420_batch_gradient(min(frames, 8), W, H, config=1)
    reps = -(-frames // batch.shape[0])
    batch = np.concatenate([batch] * reps)[:frames]
    out = np.empty((frames, H, W, 3), np.uint8)
    if swscale_ref.available():
        conv = swscale_ref.BatchConverter(W, H, cores)
        conv(batch[:cores], out[:cores])  # first call builds swscale's tables
        return (lambda: conv(batch, out)), "reference", (
            f"libswscale (the library the reference's CPU path converts with), yuv420p->rgb24 "
            f"BT.709 limited->full into one contiguous buffer, {frames} frames 1920x1080 per step, "
            f"one SwsContext per thread")
    import oracle

    flat = batch.reshape(-1)
    h2 = H * 3 // 2

    def run():
        oracle.convert_dense(batch, flat[H * W:], flat[H * W + (H // 2) * (W // 2):], width=W,
                             height=H, num_frames=frames, y_pitch=W, uv_pitch=W // 2,
                             y_frame_stride=h2 * W, uv_frame_stride=h2 * W,
                             src_format=oracle.I420, layout=oracle.NHWC, out=out)

    return run, "port", (f"C restatement of the reference kernel arithmetic with OpenMP (swscale "
                         f"unavailable on this box), {frames} frames 1920x1080 per step")


def time_cpu(frames: int, steps: int, warmup: int, limit_s: float = 60.0) -> dict:
    """Time ``steps`` steps of the CPU path.  A step is at most ``frames`` frames; it is cut down
    (never below 8) so that all steps together take about ``limit_s`` seconds."""
    probe, _, _ = make_cpu_runner(8)
    probe()
    t0 = time.perf_counter()
    probe()
    rate = 8 / (time.perf_counter() - t0)
    frames = int(max(8, min(frames, limit_s * rate / max(steps, 1))))
    run, kind, desc = make_cpu_runner(frames)
    for _ in range(warmup):
        run()
    # the K steps are timed `repeats` times (at least 10, about `limit_s` / 4 seconds in all) and
    # the median repeat is reported: one pass of K steps lasts a fraction of a second and moves
    # by +-15 % with whatever else the host is doing
    est = steps * frames / rate
    repeats = int(max(10, min(200, (limit_s / 4) / max(est, 1e-6))))
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        for _ in range(steps):
            run()
        times.append(time.perf_counter() - t0)
    times.sort()
    dt = times[len(times) // 2]
    res = {"value": frames * steps / dt, "unit": "frames/s", "cores": cpu_cores(), "kind": kind,
           "sample": desc + f"; median of {repeats} repeats of the {steps} steps",
           "ms_per_step": 1e3 * dt / steps, "frames_per_step": frames, "repeats": repeats,
           "best": frames * steps / times[0], "worst": frames * steps / times[-1]}
    if kind == "reference":
        # The reference's filter graph runs on one thread
        # (src/libspdl/core/detail/ffmpeg/filter_graph.cpp:52); that figure, on 8 frames.
        from oracle import swscale_ref
        from tests import synth

        one = swscale_ref.BatchConverter(W, H, 1)
        b8 = synth.i420_batch_gradient(8, W, H, config=1)
        o8 = np.empty((8, H, W, 3), np.uint8)
        one(b8[:1], o8[:1])
        t0 = time.perf_counter()
        one(b8, o8)
        res["single_thread_frames_per_s"] = 8 / (time.perf_counter() - t0)
        one.close()
    return res


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = time_cpu(N_FRAMES, args.steps, max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "frames/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": dict(CONFIG),
        "notes": {"input": "the CPU path takes yuv420p (what FFmpeg decoders emit) instead of NV12",
                  "frames_per_step": r["frames_per_step"], "repeats": r["repeats"],
                  "best": r["best"], "worst": r["worst"]},
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample",
                                           "single_thread_frames_per_s") if k in r},
        "e2e": {"value": r["value"], "unit": "frames/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---- our arm ------------------------------------------------------------------------------------


def synth_batch_on_device(torch, device, seed: int):
    g = torch.Generator(device=device).manual_seed(seed)
    src = torch.empty((N_FRAMES, H * 3 // 2, W), dtype=torch.uint8, device=device)
    src[:, :H] = torch.randint(16, 236, (N_FRAMES, H, W), dtype=torch.uint8, device=device,
                               generator=g)
    src[:, H:] = torch.randint(16, 241, (N_FRAMES, H // 2, W), dtype=torch.uint8, device=device,
                               generator=g)
    return src


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    import spdl_b200.io as io
    from spdl_b200 import _lib
    from spdl_b200.sharding import ShardWorker, gather_stats, rank_info

    info = rank_info()
    multi = info.world_size > 1
    # stdout carries exactly one JSON line.  Libraries print there too (NCCL its version banner),
    # so file descriptor 1 is pointed at stderr for the run and the line goes to the saved one.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(obj) -> None:
        os.write(json_fd, (json.dumps(obj) + "\n").encode())

    if multi:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", info.local_rank))
    worker = ShardWorker(info)
    dev, stream, cfg = worker.device, worker.stream, worker.config
    L = _lib.lib()
    K, Wm = args.steps, max(args.warmup, 3)

    inputs = [synth_batch_on_device(torch, dev, 2000 + 17 * info.rank + i) for i in range(ROTATE)]
    outputs = [torch.empty((N_FRAMES, H, W, 3), dtype=torch.uint8, device=dev)
               for _ in range(ROTATE // 2)]
    torch.cuda.synchronize(dev)

    def dense_args(src, dst):
        a = _lib.DenseArgs()
        a.struct_size = ctypes.sizeof(_lib.DenseArgs)
        a.device = info.local_rank
        a.y, a.u = src.data_ptr(), src.data_ptr() + H * W
        a.y_pitch = a.uv_pitch = W
        a.y_frame_stride = a.uv_frame_stride = FRAME_IN
        a.src_format, a.width, a.height, a.num_frames = _lib.NV12, W, H, N_FRAMES
        a.matrix_coeff, a.full_range = 1, 0
        a.dst, a.dst_frame_stride = dst.data_ptr(), 0
        a.layout, a.dtype, a.order = _lib.NHWC, _lib.U8, _lib.RGB
        a.arith = _lib.ARITH_SWSCALE if args.arith == "swscale" else _lib.ARITH_REFERENCE
        a.scale = (ctypes.c_float * 3)(1, 1, 1)
        a.bias = (ctypes.c_float * 3)(0, 0, 0)
        return a

    calls = [dense_args(inputs[i % ROTATE], outputs[i % len(outputs)]) for i in range(ROTATE * 2)]
    launches = 0

    def step(i):
        nonlocal launches
        _lib.check(L.b2_convert_dense(ctypes.byref(calls[i % len(calls)]), cfg.stream))
        launches += 1

    def barrier():
        torch.cuda.synchronize(dev)
        if multi:
            dist.barrier()
            torch.cuda.synchronize(dev)

    # -- kernel-resident timing: K steps, CUDA events on the launching stream ---------------------
    # The K steps are timed R times back to back, each pass between its own pair of events, with
    # one barrier + synchronize before the first pass and one after the last.  The median pass is
    # reported (best and worst beside it), and the clock sampler's window spans all passes, so its
    # samples lie inside timed regions.
    R = max(1, args.repeats)
    clocks = ClockSampler(info.local_rank).start() if info.rank == 0 else None
    for i in range(Wm):
        step(i)
    if clocks is not None:
        clocks.wait_ready()
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(R)]
    launches = 0
    if clocks is not None:
        clocks.begin()
    for e0, e1 in ev:
        e0.record(stream)
        for i in range(K):
            step(i)
        e1.record(stream)
    barrier()
    pass_ms = [e0.elapsed_time(e1) for e0, e1 in ev]
    timed_launches = launches
    if clocks is not None:
        clocks.end()
        # a short timed region holds too few sampling periods: keep the same load running, untimed
        give_up = time.perf_counter() + 1.0
        while len(clocks.in_window()) < 3 and time.perf_counter() < give_up:
            clocks.extended = True
            for i in range(K):
                step(i)
            torch.cuda.synchronize(dev)
            clocks.end()
        clocks.stop()
    ms_total = sorted(pass_ms)[R // 2]  # this rank's median pass of K steps

    # A seconds-long run of the same launches: the board's power cap pulls the SM clock down once
    # the load lasts (the copy that defines the peak is itself a short burst), so the sustained
    # figure is reported beside the headline, with the clocks seen while it ran.
    sustained = None
    if info.world_size == 1 and not args.kernel_only and args.sustained > 0:
        probe = ClockSampler(info.local_rank).start()
        probe.wait_ready()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        probe.begin()
        s0.record(stream)
        for i in range(args.sustained):
            step(i)
        s1.record(stream)
        torch.cuda.synchronize(dev)
        probe.end()
        probe.stop()
        ms_s = s0.elapsed_time(s1) / args.sustained
        sustained = {"launches": args.sustained, "ms_per_launch": ms_s,
                     "frames_per_s": N_FRAMES / (ms_s * 1e-3),
                     "gb_per_s": N_FRAMES * ALGO_BYTES_PER_FRAME / (ms_s * 1e-3) / 1e9,
                     "clocks": probe.summary()}

    # -- end to end through the public API: pinned host NV12 -> H2D -> convert -> checksum -> D2H -
    if args.kernel_only:
        emit({"kernel_only": True, "ms_per_launch": ms_total / K,
              "gb_per_s": N_FRAMES * ALGO_BYTES_PER_FRAME / (ms_total / K * 1e-3) / 1e9})
        return
    # Pinned buffers and the worker threads that feed the GPU live on the GPU's NUMA node, so that
    # uploads do not cross the socket interconnect (it matters once several ranks upload at once).
    from spdl_b200.sharding import bind_to_gpu_node

    numa = bind_to_gpu_node(info.local_rank) if not args.no_numa else None
    host = [io.CPUBuffer((N_FRAMES, H * 3 // 2, W), "u", 1,
                         io.cpu_storage(N_FRAMES * FRAME_IN, pin_memory=True)) for _ in range(2)]
    for hb, src in zip(host, inputs):
        _lib.check(L.b2_transfer_d2h(hb.data_ptr, src.data_ptr(), hb.nbytes, info.local_rank))

    # Two worker threads, each with its own stream, as a loader pipeline would call the stage:
    # the upload of one step overlaps the conversion, checksum and read-back of the other.
    from concurrent.futures import ThreadPoolExecutor

    tls = threading.local()

    def e2e_step(i):
        if not hasattr(tls, "cfg"):
            torch.cuda.set_device(dev)
            tls.stream = torch.cuda.Stream(dev)
            tls.cfg = io.cuda_config(info.local_rank, stream=tls.stream.cuda_stream)
        d = io.transfer_buffer(host[i % 2], device_config=tls.cfg)
        rgb = io.convert_nv12(d, device_config=tls.cfg, layout="NHWC", arith=args.arith)
        return io.frame_checksum(rgb, device_config=tls.cfg)

    with ThreadPoolExecutor(2) as pool:
        list(pool.map(e2e_step, range(2 * Wm)))
        barrier()
        Ke = min(K, 50)  # each end-to-end step moves 199 MB over PCIe; 50 steps are plenty
        t0 = time.perf_counter()
        sums = list(pool.map(e2e_step, range(Ke)))[-1]
        torch.cuda.synchronize(dev)
        e2e_s = (time.perf_counter() - t0) / Ke  # seconds per end-to-end step
    assert sums.shape == (N_FRAMES,)
    # the link's own rate for the same upload (pinned host -> device, nothing else running): the
    # bound of the end-to-end figure
    try:
        t0 = time.perf_counter()
        for i in range(8):
            _lib.check(L.b2_transfer_h2d(inputs[i % ROTATE].data_ptr(), host[i % 2].data_ptr,
                                         host[i % 2].nbytes, 1, info.local_rank, cfg.stream))
        h2d_gbs = 8 * host[0].nbytes / (time.perf_counter() - t0) / 1e9
    except Exception as exc:  # informational figure: never fail the run over it
        print(f"link measurement skipped: {exc}", file=sys.stderr)
        h2d_gbs = None
    if numa is not None and numa["bound"]:
        os.sched_setaffinity(0, numa["previous"])  # the CPU legs below use every core again

    # -- max over ranks ----------------------------------------------------------------------------
    per_rank = gather_stats([e2e_s] + pass_ms, device=dev)
    e2e_max = max(r[0] for r in per_rank)
    # every pass takes as long as its slowest rank; the median pass is the reported one
    worst_rank = sorted(max(r[1 + j] for r in per_rank) for j in range(R))
    ms_max, ms_best, ms_worst = worst_rank[R // 2], worst_rank[0], worst_rank[-1]
    total_frames = N_FRAMES * K * info.world_size

    if info.rank == 0:
        peak, peak_kind = measured_peak()
        ms_launch = ms_total / K
        achieved = N_FRAMES * ALGO_BYTES_PER_FRAME / (ms_launch * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": total_frames / (ms_max * 1e-3), "unit": "frames/s",
            "n_gpus": info.world_size, "steps": K, "warmup": Wm, "ms_per_step": ms_max / K,
            "higher_is_better": True, "scaling": SCALING, "vs_baseline": None, "dtype": "u8",
            "data": "synthetic",
            "config": dict(CONFIG, frames_per_step_per_gpu=N_FRAMES) if args.arith == "reference"
            else dict(CONFIG, frames_per_step_per_gpu=N_FRAMES, arith=args.arith),
            "notes": {"l2": f"inputs ({N_FRAMES * FRAME_IN / 1e6:.0f} MB per batch) rotate over "
                            f"{ROTATE} batches, {ROTATE * N_FRAMES * FRAME_IN / 1e6:.0f} MB in "
                            f"all, more than L2",
                      "sharding": "each rank converts its own frames; no data-path collective",
                      "timing": f"median of {R} back-to-back passes of the {K} steps, each between "
                                f"its own CUDA events; every pass counted at its slowest rank",
                      "ms_per_step_best": ms_best / K, "ms_per_step_worst": ms_worst / K,
                      "sustained": sustained},
            "e2e": {"value": N_FRAMES * info.world_size / e2e_max, "unit": "frames/s",
                    "steps": min(K, 50),
                    "h2d_bytes_per_step": N_FRAMES * FRAME_IN, "d2h_bytes_per_step": N_FRAMES * 8,
                    "h2d_gb_per_s": N_FRAMES * FRAME_IN / e2e_s / 1e9,
                    "link_h2d_gb_per_s": h2d_gbs,
                    "host_binding": None if numa is None else
                    {k: numa[k] for k in ("node", "cpus", "bound")},
                    "note": "pinned NV12 -> transfer_buffer -> convert_nv12 -> frame_checksum -> "
                            "host, per step, two worker threads on private streams, host-timed; "
                            "the converted frames stay on the device by design (the model reads "
                            "them there), only their 64 checksums are copied back"},
            "gpu_launches": timed_launches,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "frac_of_nominal_8000": achieved / 8000.0,
                         "traffic": ncu_traffic_bytes_per_launch() * N_FRAMES // 64,
                         "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)"
                         if peak_kind == "measured" else "fallback 6650 GB/s",
                         "algorithmic_bytes_per_launch": N_FRAMES * ALGO_BYTES_PER_FRAME,
                         "kernel": "dense_vec_kernel<NV12,NHWC,u8>", "ms_per_launch": ms_launch},
            "clocks": clocks.summary() if clocks is not None else None,
        }
        if info.world_size == 1:
            line["cpu_baseline"] = {k: v for k, v in time_cpu(N_FRAMES, 200, 2, 20.0).items()
                                    if k not in ("ms_per_step", "frames_per_step")}
            ref = reference_kernel_fps(torch, inputs[0], cfg)
            if ref is not None:
                line["reference_gpu_kernel"] = ref
        emit(line)
    if multi:
        dist.barrier()
        dist.destroy_process_group()


# ---- the fused resize workloads (informational; the headline is the dense workload above) --------


def _tap_bytes(w, h, rw, rh, cx, cy, ow, oh, fmt) -> tuple[int, int]:
    """(tap-exact, row-granular) source bytes of one image: distinct luma taps plus distinct chroma
    samples under them, and whole touched rows."""
    def taps(n_in, n_out, off, keep):
        d = np.arange(off, off + keep, dtype=np.float64)
        s = np.maximum((d + 0.5) * (n_in / n_out) - 0.5, 0.0)
        i0 = np.minimum(np.floor(s).astype(np.int64), n_in - 1)
        return np.unique(np.concatenate([i0, np.minimum(i0 + 1, n_in - 1)]))

    xs, ys = taps(w, rw, cx, ow), taps(h, rh, cy, oh)
    if fmt in ("rgb24", "rgb_planar"):
        return 3 * len(xs) * len(ys), 3 * len(ys) * w
    ncx, ncy = len(np.unique(xs // 2)), len(np.unique(ys // 2))
    exact = len(xs) * len(ys) + 2 * ncx * ncy
    rows = len(ys) * w + ncy * (w if fmt == "nv12" else 2 * ((w + 1) // 2))
    return exact, rows


def _clips_on_device(torch, dev, clip_ids, t: int, w: int, h: int):
    """Clips of the sharded clip workload, generated on the device: frame 0 uniform in the nominal
    ranges, every later frame the previous one plus rounded Gaussian noise (sigma 4), clipped to
    [16,235] (Y) / [16,240] (UV).  Seeded per clip, so a rank's shard equals the same clips of
    the whole batch whichever GPU generates them."""
    h2 = h * 3 // 2
    out = torch.empty((len(clip_ids) * t, h2, w), dtype=torch.uint8, device=dev)
    hi = torch.full((h2, 1), 240, dtype=torch.int16, device=dev)
    hi[:h] = 235
    for k, clip in enumerate(clip_ids):
        g = torch.Generator(device=dev).manual_seed(4000 + int(clip))
        cur = torch.empty((h2, w), dtype=torch.int16, device=dev)
        cur[:h] = torch.randint(16, 236, (h, w), dtype=torch.int16, device=dev, generator=g)
        cur[h:] = torch.randint(16, 241, (h // 2, w), dtype=torch.int16, device=dev, generator=g)
        out[k * t] = cur.to(torch.uint8)
        for f in range(1, t):
            step = torch.randn((h2, w), device=dev, generator=g).mul_(4.0).round_().to(torch.int16)
            cur = torch.minimum(torch.clamp_min(cur + step, 16), hi)
            out[k * t + f] = cur.to(torch.uint8)
    return out


def run_resize_workload(args) -> None:
    """``--workload c3|c4|c5|j5``: kernel-resident timing of the fused resize kernel on the other
    benchmark configurations (j5: the images of c5 as decoded RGB), with tap-exact and
    row-granular roofline figures.  Under ``torch.distributed.run`` the units of the workload
    (clips for c4, images otherwise) are split over the ranks in contiguous blocks -- the
    configurations define c4 and c5 as sharded over 8 GPUs -- each rank holding and converting
    its own shard; after the timed steps the per-image checksums of all ranks are gathered and
    compared with the whole batch converted on rank 0's GPU."""
    import torch
    import torch.distributed as dist

    import spdl_b200.io as io
    from spdl_b200 import _lib
    from spdl_b200.sharding import ShardWorker, gather_stats, rank_info, shard_range
    from tests import synth

    info = rank_info()
    multi = info.world_size > 1
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)  # libraries print to stdout too (NCCL's banner); keep it for the JSON line
    if multi:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", info.local_rank))
    worker = ShardWorker(info)
    dev, stream, cfg = worker.device, worker.stream, worker.config
    L = _lib.lib()
    scale = float(args.scale)
    mean, std = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
    wl = args.workload
    per_unit = 1  # images per sharded unit
    if wl == "c3":
        units, w, h = max(info.world_size, int(16 * scale)), 3840, 2160
        geom = dict(resize=(224, 224))
        spec = dict(fmt="nv12", dtype="bfloat16", esz=2, coeff=1, full=False, norm=True,
                    name="{n} x 3840x2160 NV12 -> 224x224 bf16 NCHW, BT.709, normalised")
    elif wl == "c4":
        per_unit = 16
        units, w, h = max(info.world_size, int(64 * scale)), 1280, 720
        geom = dict(resize=(256, 256))
        spec = dict(fmt="nv12", dtype="uint8", esz=1, coeff=6, full=False, norm=False,
                    name="{n} frames ({u} clips x 16) 1280x720 NV12 -> 256x256 u8 "
                         "N x T x C x H x W, BT.601")
    else:
        units = max(info.world_size, int(2048 * scale))
        geom = dict(resize_shorter=256, crop=(224, 224))
        if wl == "j5":
            spec = dict(fmt="rgb24", dtype="float32", esz=4, coeff=1, full=False, norm=True,
                        name="{n} ragged interleaved RGB images (256..1024) -> shorter side 256, "
                             "centre crop 224x224 fp32 NCHW, normalised")
        else:
            spec = dict(fmt="i420", dtype="float32", esz=4, coeff=6, full=True, norm=True,
                        name="{n} ragged I420 images (256..1024) -> shorter side 256, centre crop "
                             "224x224 fp32 NCHW, full-range BT.601, normalised")
    lo, hi = shard_range(units, info.rank, info.world_size)

    # -- inputs: the rank's shard resident in its own HBM (rank 0 also builds the whole batch, after
    #    the timed steps, for the shard-equals-whole check) -------------------------------------------
    host_cache: dict = {}

    def build(first: int, last: int):
        """(device bytes, descriptor table, (out_w, out_h), widths, heights) of units [first, last)."""
        if wl in ("c3", "c4"):
            n_img = (last - first) * per_unit
            if wl == "c4":
                data = _clips_on_device(torch, dev, range(first, last), 16, w, h).reshape(-1)
            else:
                g = torch.Generator(device=dev)
                parts = []
                for i in range(first, last):
                    g.manual_seed(3000 + i)
                    f = torch.empty((h * 3 // 2, w), dtype=torch.uint8, device=dev)
                    f[:h] = torch.randint(16, 236, (h, w), dtype=torch.uint8, device=dev, generator=g)
                    f[h:] = torch.randint(16, 241, (h // 2, w), dtype=torch.uint8, device=dev,
                                          generator=g)
                    parts.append(f.reshape(-1))
                data = torch.cat(parts)
            ws_, hs_ = [w] * n_img, [h] * n_img
            descs, out = io.make_image_descs(ws_, hs_, **geom)
            return data, descs, out, np.asarray(ws_), np.asarray(hs_)
        # ragged images: sizes and bytes from the seeded host generator, the shard's bytes uploaded
        if wl == "c5":
            if "c5" not in host_cache:
                host_cache["c5"] = synth.ragged_i420(units)
            host, ws_, hs_, offs = host_cache["c5"]
            sizes = ws_ * hs_ * 3 // 2
        else:
            r = synth.rng_for(5, 0)
            ws_ = (r.integers(128, 513, units) * 2).astype(np.int64)
            hs_ = (r.integers(128, 513, units) * 2).astype(np.int64)
            sizes = 3 * ws_ * hs_
            offs = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int64)
            host = None
        b0 = int(offs[first])
        b1 = int(offs[last - 1] + sizes[last - 1])
        if host is not None:
            data = torch.from_numpy(host[b0:b1]).to(dev)
        else:
            g = torch.Generator(device=dev).manual_seed(5000)
            whole = torch.randint(0, 256, (int(sizes.sum()),), dtype=torch.uint8, device=dev,
                                  generator=g)
            data = whole[b0:b1].clone()
            del whole
        descs, out = io.make_image_descs(ws_[first:last], hs_[first:last], src_format=spec["fmt"],
                                         offsets=offs[first:last] - b0, **geom)
        return data, descs, out, ws_[first:last], hs_[first:last]

    with torch.cuda.stream(stream):
        data, descs, out, ws, hs = build(lo, hi)
        n = len(descs)
        # rotate copies of the shard so that a step does not find its source rows in L2
        copies = max(2, min(8, int(2 * 126e6 // max(int(data.numel()), 1)) + 1))
        bases = [data] + [data.clone() for _ in range(copies - 1)]
        dd = torch.from_numpy(descs.view(np.uint8)).to(dev)
        dst = torch.empty(n * 3 * out[0] * out[1] * spec["esz"], dtype=torch.uint8, device=dev)
    sc, bi = io._core._scale_bias(mean if spec["norm"] else None, std if spec["norm"] else None)

    def make_call(base, table, count, target, max_w):
        a = _lib.ResizeArgs()
        a.struct_size = ctypes.sizeof(_lib.ResizeArgs)
        a.device, a.base, a.descs = info.local_rank, base.data_ptr(), table.data_ptr()
        a.num_images, a.src_format = count, io._core._FORMATS[spec["fmt"]]
        a.out_w, a.out_h = out
        a.matrix_coeff, a.full_range = spec["coeff"], int(spec["full"])
        a.layout, a.dtype, a.order = _lib.NCHW, io._core._DTYPES[spec["dtype"]], _lib.RGB
        a.max_src_w, a.dst = int(max_w), target.data_ptr()
        a.scale = (ctypes.c_float * 3)(*sc.tolist())
        a.bias = (ctypes.c_float * 3)(*bi.tolist())
        return a

    calls = [make_call(b, dd, n, dst, max(ws)) for b in bases]
    K, Wm = args.steps, max(args.warmup, 3)

    def barrier():
        torch.cuda.synchronize(dev)
        if multi:
            dist.barrier()
            torch.cuda.synchronize(dev)

    stream.synchronize()
    for i in range(Wm):
        _lib.check(L.b2_convert_resize(ctypes.byref(calls[i % copies]), stream.cuda_stream))
    clocks = ClockSampler(info.local_rank).start() if info.rank == 0 else None
    if clocks is not None:
        clocks.wait_ready()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if clocks is not None:
        clocks.begin()
    e0.record(stream)
    for i in range(K):
        _lib.check(L.b2_convert_resize(ctypes.byref(calls[i % copies]), stream.cuda_stream))
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1) / K
    if clocks is not None:
        clocks.end()
        give_up = time.perf_counter() + 1.0
        # keep the same load running, untimed, until three samples are in
        while len(clocks.in_window()) < 3 and time.perf_counter() < give_up:
            clocks.extended = True
            for i in range(K):
                _lib.check(L.b2_convert_resize(ctypes.byref(calls[i % copies]), stream.cuda_stream))
            torch.cuda.synchronize(dev)
            clocks.end()
        clocks.stop()

    # -- the shard's bytes (tap-exact and row-granular), summed over ranks ----------------------------
    rw = np.rint(np.asarray(ws) / descs["scale_x"].astype(np.float64)).astype(np.int64)
    rh = np.rint(np.asarray(hs) / descs["scale_y"].astype(np.float64)).astype(np.int64)
    cache: dict = {}
    exact = rows = 0
    for i in range(n):
        key = (int(ws[i]), int(hs[i]), int(rw[i]), int(rh[i]), int(descs["crop_x"][i]),
               int(descs["crop_y"][i]))
        if key not in cache:
            cache[key] = _tap_bytes(*key, out[0], out[1], spec["fmt"])
        exact += cache[key][0]
        rows += cache[key][1]
    out_bytes = n * 3 * out[0] * out[1] * spec["esz"]

    # -- correctness in the same run: checksums of every rank's output against the whole batch ------
    frame_bytes = 3 * out[0] * out[1] * spec["esz"]
    sums = torch.empty(n, dtype=torch.int64, device=dev)
    _lib.check(L.b2_convert_resize(ctypes.byref(calls[0]), stream.cuda_stream))
    _lib.check(L.b2_frame_checksum(dst.data_ptr(), frame_bytes, n, sums.data_ptr(),
                                   info.local_rank, stream.cuda_stream))
    stream.synchronize()
    equal = None
    if multi:
        counts = [(shard_range(units, r, info.world_size)[1] -
                   shard_range(units, r, info.world_size)[0]) * per_unit
                  for r in range(info.world_size)]
        padded = torch.zeros(max(counts), dtype=torch.int64, device=dev)
        padded[:n] = sums
        gathered = [torch.zeros_like(padded) for _ in range(info.world_size)]
        dist.all_gather(gathered, padded)
        if info.rank == 0:
            all_sums = torch.cat([g[:c] for g, c in zip(gathered, counts)]).cpu().numpy()
    else:
        all_sums = sums.cpu().numpy()
    if info.rank == 0:
        del bases[1:], calls[1:]
        with torch.cuda.stream(stream):
            wdata, wdescs, _, wws, _ = build(0, units)
            wdd = torch.from_numpy(wdescs.view(np.uint8)).to(dev)
            wn = len(wdescs)
            wdst = torch.empty(wn * frame_bytes, dtype=torch.uint8, device=dev)
            wsums = torch.empty(wn, dtype=torch.int64, device=dev)
        whole_call = make_call(wdata, wdd, wn, wdst, max(wws))
        _lib.check(L.b2_convert_resize(ctypes.byref(whole_call), stream.cuda_stream))
        _lib.check(L.b2_frame_checksum(wdst.data_ptr(), frame_bytes, wn, wsums.data_ptr(),
                                       info.local_rank, stream.cuda_stream))
        stream.synchronize()
        equal = bool((wsums.cpu().numpy() == all_sums).all())
        if not equal:
            raise SystemExit("the ranks' outputs differ from the whole batch converted on one GPU")

    # -- end to end for the uniform-size workloads: decoded frames in pageable host memory (as a
    #    decoder leaves them) -> FrameStage (stage into pinned memory, upload, fused kernel) ->
    #    checksum of the result on the host.  Whole frames against row-sparse uploads: only the
    #    source rows the geometry reads are staged and sent.
    e2e = None
    if wl in ("c3", "c4"):
        from concurrent.futures import ThreadPoolExecutor

        n_e2e = min(n, 16 if wl == "c3" else 128)  # frames per end-to-end step
        h2 = h * 3 // 2
        host_frames = [data[:n_e2e * h2 * w].reshape(n_e2e, h2, w).cpu().numpy() for _ in range(2)]
        stage_kw = dict(src_format="nv12", dtype=spec["dtype"], coeff=spec["coeff"],
                        mean=mean if spec["norm"] else None, std=std if spec["norm"] else None,
                        device_index=info.local_rank, **geom)
        e2e = {"frames_per_step": n_e2e, "unit": "frames/s",
               "note": "pageable host frames -> FrameStage (staging copy into pinned memory by up to 8 "
                       "host threads, async H2D, fused kernel) -> frame_checksum -> host; two "
                       "worker threads on private streams, host-timed, median of 5 rounds"}
        frame_in = h2 * w
        for label, sparse in (("whole_frames", False), ("sparse_rows", True)):
            stg = io.FrameStage(sparse_upload=sparse, **stage_kw)

            def e2e_step(i, stg=stg):
                t = stg(host_frames[i % 2])
                cfg_t = stg._state()["cfg"]
                return io.frame_checksum(t.view(torch.uint8).reshape(n_e2e, -1),
                                         device_config=cfg_t)

            with ThreadPoolExecutor(2) as pool:
                list(pool.map(e2e_step, range(4)))
                barrier()
                reps, rounds = 12, []
                for _ in range(5):  # the host is shared: median of five rounds of twelve steps
                    t0 = time.perf_counter()
                    last = list(pool.map(e2e_step, range(reps)))[-1]
                    rounds.append((time.perf_counter() - t0) / reps)
                dt = sorted(rounds)[len(rounds) // 2]
            if sparse:
                lm, cm = io.touched_rows(descs[0], src_format="nv12", out_h=out[1])
                sent = int(((lm >= 0).sum() + (cm >= 0).sum()) * w)
            else:
                sent = frame_in
            e2e[label] = {"value": n_e2e / dt, "h2d_bytes_per_step": sent * n_e2e,
                          "d2h_bytes_per_step": 8 * n_e2e, "ms_per_step": 1e3 * dt,
                          "ms_per_step_rounds": [round(1e3 * r, 3) for r in rounds],
                          "checksum_of_frame_0": int(last[0])}
        assert e2e["whole_frames"]["checksum_of_frame_0"] == e2e["sparse_rows"]["checksum_of_frame_0"]

    # -- end to end for the ragged workloads: a list of decoded images in pageable host memory (a
    #    CPU decoder's output) -> resize_host_images (packed into pinned staging by several host
    #    threads, one upload, one launch) -> checksum of the result on the host.
    if wl in ("c5", "j5"):
        from concurrent.futures import ThreadPoolExecutor

        n_e2e = min(n, 256)  # images per end-to-end step
        flat = data.cpu().numpy()
        first_off = int(descs["y_off"][0])
        sizes_e = (3 * ws * hs // 2 if wl == "c5" else 3 * ws * hs)[:n_e2e]
        starts = descs["y_off"][:n_e2e].astype(np.int64) - first_off
        shape_of = (lambda w, h: (h * 3 // 2, w)) if wl == "c5" else (lambda w, h: (h, w, 3))
        images = [flat[int(b):int(b + k)].reshape(shape_of(int(w), int(h))).copy()
                  for b, k, w, h in zip(starts, sizes_e, ws[:n_e2e], hs[:n_e2e])]
        tls = threading.local()

        def cfg_of_thread():
            if not hasattr(tls, "cfg"):
                tls.stream = torch.cuda.Stream(dev)
                tls.cfg = io.cuda_config(info.local_rank, stream=tls.stream.cuda_stream)
            return tls.cfg

        def e2e_images(i):
            c = cfg_of_thread()
            o = io.resize_host_images(images, device_config=c, src_format=spec["fmt"],
                                      dtype=spec["dtype"], coeff=spec["coeff"],
                                      full_range=spec.get("full", False),
                                      mean=mean if spec["norm"] else None,
                                      std=std if spec["norm"] else None, **geom)
            t = io.to_torch(o)
            return io.frame_checksum(t.view(torch.uint8).reshape(n_e2e, -1), device_config=c)

        with ThreadPoolExecutor(2) as pool:
            list(pool.map(e2e_images, range(4)))
            barrier()
            reps, rounds = 8, []
            for _ in range(5):
                t0 = time.perf_counter()
                last = list(pool.map(e2e_images, range(reps)))[-1]
                rounds.append((time.perf_counter() - t0) / reps)
            dt = sorted(rounds)[len(rounds) // 2]
        sent = int(sizes_e.sum())
        e2e = {"value": n_e2e / dt, "unit": "images/s", "images_per_step": n_e2e,
               "h2d_bytes_per_step": sent, "d2h_bytes_per_step": 8 * n_e2e,
               "ms_per_step": 1e3 * dt,
               "ms_per_step_rounds": [round(1e3 * r, 3) for r in rounds],
               "checksum_of_image_0": int(last[0]),
               "note": "pageable host images of different sizes -> resize_host_images (packed "
                       "into pinned staging by up to 8 host threads, one async H2D, fused kernel) "
                       "-> frame_checksum -> host; two worker threads on private streams, "
                       "host-timed, median of 5 rounds"}
        del flat, images

    per_rank = gather_stats([ms, float(exact), float(rows), float(out_bytes), float(n)], device=dev)
    if info.rank == 0:
        ms_max = max(r[0] for r in per_rank)
        t_exact, t_rows, t_out = (sum(r[i] for r in per_rank) for i in (1, 2, 3))
        total_n = int(sum(r[4] for r in per_rank))
        peak, peak_kind = measured_peak()
        g = info.world_size
        per_gpu = lambda b: b / g / (ms_max * 1e-3) / 1e9  # noqa: E731
        line = {
            "metric": "fused convert+resize images/s", "value": total_n / (ms_max * 1e-3),
            "unit": "images/s", "n_gpus": g, "steps": K, "warmup": Wm, "ms_per_step": ms_max,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {1: "u8", 2: "bf16", 4: "f32"}[spec["esz"]], "data": "synthetic",
            "config": {"workload": spec["name"].format(n=total_n, u=units),
                       "images_per_step": total_n, "images_per_gpu": total_n // g,
                       "l2": f"{copies} copies of each rank's shard rotated",
                       "sharding": "contiguous blocks of clips/images per rank, each resident in "
                                   "its own GPU's memory; no data-path collective"},
            "ms_per_rank": [r[0] for r in per_rank],
            "shards_equal_whole": equal,
            "e2e": e2e,
            "gpu_launches": K,
            "roofline": {"bound": "hbm", "unit": "GB/s", "peak": peak, "peak_source": peak_kind,
                         "achieved": per_gpu(t_exact + t_out),
                         "frac": per_gpu(t_exact + t_out) / peak,
                         "algorithmic_bytes_per_launch": (t_exact + t_out) / g,
                         "row_granular_bytes_per_launch": (t_rows + t_out) / g,
                         "row_granular_gb_per_s": per_gpu(t_rows + t_out),
                         "row_granular_frac": per_gpu(t_rows + t_out) / peak,
                         "traffic": None, "kernel": "resize_kernel", "ms_per_launch": ms_max,
                         "note": "per GPU: the ranks' bytes divided by the number of GPUs and by "
                                 "the slowest rank's time"},
            "clocks": clocks.summary() if clocks is not None else None,
        }
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if multi:
        dist.barrier()
        dist.destroy_process_group()


def run_aux_workload(args) -> None:
    """``--workload aux``: the small kernels around the two main ones, one GPU, CUDA events:
    surface gather (frame batching), per-frame checksum, and the any-shape dense path."""
    import torch

    from spdl_b200 import _lib

    torch.cuda.init()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(dev)
    L = _lib.lib()
    K, Wm = args.steps, max(args.warmup, 3)
    peak, _ = measured_peak()
    n, w, h, pitch = N_FRAMES, W, H, 2048
    h2 = h * 3 // 2
    results = {}

    def timed(fn):
        for _ in range(Wm):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(K):
            fn()
        e1.record(stream)
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / K

    with torch.cuda.stream(stream):
        # 1. gather: 64 pitched 1080p NV12 surfaces (pitch 2048) -> packed batch
        surf = [torch.randint(0, 256, (2, n, h2, pitch), dtype=torch.uint8, device=dev)]
        packed = torch.empty((n, h2, w), dtype=torch.uint8, device=dev)
        tabs = []
        for c in range(2):
            ptrs = torch.tensor([surf[0][c, i].data_ptr() for i in range(n)], dtype=torch.int64,
                                device=dev)
            tabs.append((ptrs, torch.full((n,), pitch, dtype=torch.int64, device=dev)))
        stream.synchronize()
        i = [0]

        def gather():
            i[0] += 1
            p, q = tabs[i[0] % 2]
            _lib.check(L.b2_gather_surfaces(p.data_ptr(), q.data_ptr(), n, w, h, packed.data_ptr(),
                                            0, stream.cuda_stream))

        ms = timed(gather)
        b = 2 * n * h2 * w
        results["gather_kernel"] = {"ms": ms, "bytes": b, "gb_per_s": b / ms / 1e6,
                                    "frac": b / ms / 1e6 / peak,
                                    "what": "64 x 1080p NV12 surfaces, pitch 2048 -> packed"}
        # 1b. the same surfaces converted straight through the pointer table (no gather pass)
        rgb_out = torch.empty((n, h, w, 3), dtype=torch.uint8, device=dev)
        tcalls = []
        for c in range(2):
            ytab = tabs[c][0]
            utab = ytab + h * pitch
            a = _lib.DenseArgs()
            a.struct_size = ctypes.sizeof(_lib.DenseArgs)
            a.device, a.y_table, a.u_table = 0, ytab.data_ptr(), utab.data_ptr()
            a.y_pitch = a.uv_pitch = pitch
            a.src_format, a.width, a.height, a.num_frames = _lib.NV12, w, h, n
            a.matrix_coeff, a.dst = 1, rgb_out.data_ptr()
            a.layout, a.dtype, a.order = _lib.NHWC, _lib.U8, _lib.RGB
            a.scale = (ctypes.c_float * 3)(1, 1, 1)
            tcalls.append((a, ytab, utab))
        stream.synchronize()

        def table_convert():
            i[0] += 1
            _lib.check(L.b2_convert_dense(ctypes.byref(tcalls[i[0] % 2][0]), stream.cuda_stream))

        ms = timed(table_convert)
        b = n * h * w * 9 // 2
        results["dense_vec_kernel_pointer_table"] = {
            "ms": ms, "bytes": b, "gb_per_s": b / ms / 1e6, "frac": b / ms / 1e6 / peak,
            "what": "64 x 1080p NV12 surfaces, pitch 2048, through the pointer table -> NHWC u8"}
        del rgb_out
        # 1c. 256 decoder surfaces of a width that is no multiple of 16 (854x480, pitch 1024)
        #     through the pointer table into a packed batch: the flat kernel's pitched variant
        nq, wq, hq, pq = 256, 854, 480, 1024
        surf_q = torch.randint(16, 236, (2, nq, hq * 3 // 2, pq), dtype=torch.uint8, device=dev)
        out_q = torch.empty((nq, hq, wq, 3), dtype=torch.uint8, device=dev)
        qcalls = []
        for c in range(2):
            ytab = torch.tensor([surf_q[c, k].data_ptr() for k in range(nq)], dtype=torch.int64,
                                device=dev)
            utab = ytab + hq * pq
            a = _lib.DenseArgs()
            a.struct_size = ctypes.sizeof(_lib.DenseArgs)
            a.device, a.y_table, a.u_table = 0, ytab.data_ptr(), utab.data_ptr()
            a.y_pitch = a.uv_pitch = pq
            a.src_format, a.width, a.height, a.num_frames = _lib.NV12, wq, hq, nq
            a.matrix_coeff, a.dst = 1, out_q.data_ptr()
            a.layout, a.dtype, a.order = _lib.NHWC, _lib.U8, _lib.RGB
            a.scale = (ctypes.c_float * 3)(1, 1, 1)
            qcalls.append((a, ytab, utab))
        stream.synchronize()

        def table_convert_854():
            i[0] += 1
            _lib.check(L.b2_convert_dense(ctypes.byref(qcalls[i[0] % 2][0]), stream.cuda_stream))

        ms = timed(table_convert_854)
        b = nq * hq * wq * 9 // 2
        results["dense_flat_kernel_854x480_surfaces"] = {
            "ms": ms, "bytes": b, "gb_per_s": b / ms / 1e6, "frac": b / ms / 1e6 / peak,
            "what": "256 x 854x480 NV12 surfaces, pitch 1024, through the pointer table -> packed "
                    "NHWC u8"}
        del surf_q, out_q, qcalls
        # 2. checksum of a 64 x 1080p RGB batch
        rgb = [torch.randint(0, 256, (n, h, w, 3), dtype=torch.uint8, device=dev)
               for _ in range(2)]
        sums = torch.empty(n, dtype=torch.int64, device=dev)
        stream.synchronize()

        def checksum():
            i[0] += 1
            _lib.check(L.b2_frame_checksum(rgb[i[0] % 2].data_ptr(), h * w * 3, n, sums.data_ptr(),
                                           0, stream.cuda_stream))

        ms = timed(checksum)
        b = n * h * w * 3
        results["checksum_kernel"] = {"ms": ms, "bytes": b, "gb_per_s": b / ms / 1e6,
                                      "frac": b / ms / 1e6 / peak,
                                      "what": "64 x 1080p RGB frames (read only)"}
        # 3. widths that are not a multiple of 16: packed frames of width 1918, 1366x768 and 854x480
        #    (common video sizes) take the kernel for packed frames; the 1918-wide batch written to
        #    an odd address takes the any-alignment kernel
        for name, wq, hq, off, what in (
                ("dense_flat_kernel_1918x1080", 1918, 1080, 0,
                 "64 x 1918x1080 NV12 -> NHWC u8 (packed frames, rows on even, unaligned offsets)"),
                ("dense_any_kernel_odd_address", 1918, 1080, 1,
                 "the same batch written to an odd address"),
                ("dense_flat_kernel_1366x768", 1366, 768, 0,
                 "128 x 1366x768 NV12 -> NHWC u8 (packed frames)"),
                ("dense_flat_kernel_854x480", 854, 480, 0,
                 "256 x 854x480 NV12 -> NHWC u8 (packed 480p frames)")):
            nq = {1080: n, 768: 128, 480: 256}[hq]
            hq2 = hq * 3 // 2
            srcq = [torch.randint(16, 236, (nq, hq2, wq), dtype=torch.uint8, device=dev)
                    for _ in range(2)]
            dstq = torch.empty((nq * hq * wq * 3 + 16,), dtype=torch.uint8, device=dev)
            b = nq * hq * wq * 9 // 2
            calls = []
            for s in srcq:
                a = _lib.DenseArgs()
                a.struct_size = ctypes.sizeof(_lib.DenseArgs)
                a.device, a.y, a.u = 0, s.data_ptr(), s.data_ptr() + hq * wq
                a.y_pitch = a.uv_pitch = wq
                a.y_frame_stride = a.uv_frame_stride = hq2 * wq
                a.src_format, a.width, a.height, a.num_frames = _lib.NV12, wq, hq, nq
                a.matrix_coeff, a.dst = 1, dstq.data_ptr() + off
                a.layout, a.dtype, a.order = _lib.NHWC, _lib.U8, _lib.RGB
                a.scale = (ctypes.c_float * 3)(1, 1, 1)
                calls.append(a)
            stream.synchronize()

            def unaligned(calls=calls):
                i[0] += 1
                _lib.check(L.b2_convert_dense(ctypes.byref(calls[i[0] % 2]), stream.cuda_stream))

            ms = timed(unaligned)
            results[name] = {"ms": ms, "bytes": b, "gb_per_s": b / ms / 1e6,
                             "frac": b / ms / 1e6 / peak, "what": what}
            del srcq, dstq, calls
    # 4. transfer_tensor (this package's transport: reused page-locked arena filled by several host
    #    threads, async upload, one synchronise per batch) against what the reference's
    #    transfer_tensor does per call (pin every tensor anew, upload, synchronise); host-timed
    import spdl_b200.io as io

    batch = {"frames": torch.randint(0, 256, (32, 3, 720, 1280), dtype=torch.uint8),
             "labels": torch.arange(32, dtype=torch.int64)}
    nbytes = sum(t.numel() * t.element_size() for t in batch.values())

    def ours():
        return io.transfer_tensor(batch)

    side = torch.cuda.Stream(dev)

    def pin_per_call():
        with torch.cuda.stream(side):
            out = {k: v.pin_memory().to(dev, non_blocking=True) for k, v in batch.items()}
        side.synchronize()
        return out

    host_ms = {}
    for label, fn in (("transfer_tensor", ours), ("pin_memory_per_call", pin_per_call)):
        for _ in range(3):
            fn()
        times = []
        for _ in range(9):
            t0 = time.perf_counter()
            fn()
            times.append(time.perf_counter() - t0)
        host_ms[label] = 1e3 * sorted(times)[len(times) // 2]
    results["transfer_tensor"] = {
        "ms": host_ms["transfer_tensor"], "bytes": nbytes,
        "gb_per_s": nbytes / host_ms["transfer_tensor"] / 1e6,
        "pin_memory_per_call_ms": host_ms["pin_memory_per_call"],
        "what": "a batch of 32 x 3 x 720 x 1280 u8 frames + labels from pageable memory, median of "
                "9 calls, host-timed; beside it the per-call pin_memory() route of the reference's "
                "transfer_tensor (src/spdl/io/_transfer.py:82-109)"}
    print(json.dumps({"workload": "aux", "steps": K, "warmup": Wm, "peak_gb_per_s": peak,
                      "kernels": results}), flush=True)


def reference_kernel_fps(torch, src, cfg) -> dict | None:
    """The reference's own kernel (planar RGB, compiled unmodified for sm_100a) on the same input,
    as the GPU-side kernel to beat.  Informational; absent when oracle/_ref was not built."""
    import oracle

    ref = oracle.ref_kernel()
    if ref is None:
        return None
    dst = torch.empty((N_FRAMES, 3, H, W), dtype=torch.uint8, device=src.device)
    stream = torch.cuda.current_stream(src.device)

    def run():
        ref.ref_nv12_to_planar_rgb(stream.cuda_stream, src.data_ptr(), W, dst.data_ptr(), W, W, H,
                                   N_FRAMES, 1)

    for _ in range(3):
        run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(20):
        run()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 20

    # The reference's call around that kernel allocates the output with cudaMalloc every time
    # (src/libspdl/cuda/storage.cpp:44-58) and frees it when the buffer dies: the same launches
    # with that allocation pattern, host-timed.
    from spdl_b200 import _lib

    L, index = _lib.lib(), src.device.index or 0
    t0 = time.perf_counter()
    for _ in range(10):
        p = ctypes.c_void_p()
        _lib.check(L.b2_device_alloc(ctypes.byref(p), N_FRAMES * 3 * H * W, index))
        ref.ref_nv12_to_planar_rgb(stream.cuda_stream, src.data_ptr(), W, p.value, W, W, H,
                                   N_FRAMES, 1)
        stream.synchronize()
        _lib.check(L.b2_device_free(p, index))
    alloc_s = (time.perf_counter() - t0) / 10
    return {"value": N_FRAMES / (ms * 1e-3), "unit": "frames/s", "layout": "planar RGB u8",
            "gb_per_s": N_FRAMES * ALGO_BYTES_PER_FRAME / (ms * 1e-3) / 1e9,
            "with_per_call_cudaMalloc": N_FRAMES / alloc_s}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--repeats", type=int, default=25,
                    help="c2: how many times the K timed steps are run (median reported)")
    ap.add_argument("--arith", choices=["reference", "swscale"], default="reference",
                    help="c2: which colour arithmetic the kernel computes (the reference's CUDA "
                         "kernel, or libswscale's integers as on the reference's CPU route)")
    ap.add_argument("--sustained", type=int, default=4000,
                    help="c2, one GPU: launches of the extra seconds-long run reported in "
                         "notes.sustained (0 = skip)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU legs (for profiler captures)")
    ap.add_argument("--workload", choices=["c2", "c3", "c4", "c5", "j5", "aux"], default="c2",
                    help="c2 = the headline dense workload; c3/c4/c5 = fused resize workloads; "
                         "aux = gather, checksum and any-shape kernels (one GPU, informational)")
    ap.add_argument("--scale", default="1.0",
                    help="fraction of a resize workload's batch (for profiler captures)")
    ap.add_argument("--no-numa", action="store_true",
                    help="do not bind the end-to-end leg to the GPU's NUMA node")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                    help="c2 only: weak = 64 frames per GPU (default); strong = 64 frames per step "
                         "split over the GPUs")
    args = ap.parse_args()
    if args.scaling == "strong" and args.workload == "c2" and args.impl == "ours":
        global N_FRAMES, SCALING, ROTATE
        if 64 % max(args.gpus, 1):
            raise SystemExit("--scaling strong needs a GPU count that divides 64")
        N_FRAMES, SCALING = 64 // max(args.gpus, 1), "strong"
        ROTATE = 4 * 64 // N_FRAMES  # keep the rotated inputs at 796 MB per GPU, well above L2
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "aux":
        run_aux_workload(args)
    elif args.workload != "c2":
        run_resize_workload(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
