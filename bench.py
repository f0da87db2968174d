#!/usr/bin/env python
"""Benchmark of the fused transform hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scaling weak|strong]

A step is one fused launch of the batched crop -> resize -> normalise workload (64 frames of 1920x1080 uchar3,
32 random crops per frame, each resized with preserved aspect ratio to 224x224 on a (114,114,114) background, times
1/255, written as a 224x224x2048 float3 tensor).  With N > 1 (one process per GPU under torch.distributed.run) the
headline is weak scaling: every rank runs a whole 64-frame job of its own — N independent jobs, no exchange between
GPUs — and the value is the pixels of all ranks divided by the slowest rank's device time.  The same line also carries,
inside ``roofline``, the split the workload description names — ONE 64-frame batch divided by frame over the N GPUs
(``strong_split``) — and the divergent 8-plane launch with its planes dealt over the GPUs (``config5_sharded``), each
with its efficiency against one GPU of the same run.  Rank 0 prints one JSON line.

``--impl reference`` times the reference library's own CPU backend (compiled from its headers into
oracle/_ref/libfkl_ref.so; when that file is absent, the CPU restatement in oracle/) on the host cores, on a bounded
sample of the same workload per step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fused-pipeline output Gpix/s"
UNIT = "Gpix/s"
N_FRAMES, CROPS_PER_FRAME = 64, 32
FALLBACK_HBM_GBS = 6650.0
PROFILE_SUMMARY = os.path.join(ROOT, "profiles", "staged_kernel_batched_crop_resize.md")


def profiled_traffic(planes: int):
    """DRAM bytes of one staged_kernel launch, from the committed ncu summary (its line `dram_bytes_per_plane: N`, measured
    once under ncu, not in this run), scaled to `planes` planes.  Returns (bytes or None, where the figure comes from)."""
    try:
        with open(PROFILE_SUMMARY) as f:
            for line in f:
                if line.strip().startswith("dram_bytes_per_plane:"):
                    per_plane = float(line.split(":", 1)[1].split()[0])
                    return int(per_plane * planes), "profiles/staged_kernel_batched_crop_resize.md (one ncu capture, scaled by planes)"
    except OSError:
        pass
    return None, "no committed ncu summary found"


def make_workload(rank: int, n_frames: int = N_FRAMES, frame_w: int = 1920, frame_h: int = 1080):
    from fusedkernellibrary_b200 import workloads as W
    return W.batched_crop_resize(n_frames=n_frames, crops_per_frame=CROPS_PER_FRAME, w=frame_w, h=frame_h, seed=4 + rank,
                                 frame_seed_base=1000 + 64 * rank)


def shard_workload(rank: int, world: int, scaling: str, n_frames: int = N_FRAMES, frame_w: int = 1920, frame_h: int = 1080):
    """The part of the job rank `rank` of `world` processes.  Returns (workload, frames of this rank).
    weak: every rank runs the whole n_frames workload on its own seeded frames (per-GPU work fixed).
    strong: one n_frames job, rank r keeps frames [r*n/world, (r+1)*n/world) and their planes (total work fixed).
    Either way a rank reads only its own frames and writes only its own output: there is no exchange."""
    from fusedkernellibrary_b200 import workloads as W
    if scaling == "weak":
        return make_workload(rank, n_frames, frame_w, frame_h), n_frames
    shard = W.shard_by_frame(make_workload(0, n_frames, frame_w, frame_h), rank, world)
    return shard, len(shard.sources)


def workload_config(n_gpus: int, scaling: str, frames_per_gpu: int) -> dict:
    if scaling == "weak":
        sharding = (f"weak scaling: {n_gpus} independent {frames_per_gpu}-frame job(s), one per GPU, each on its own seeded frames; "
                    "no collective; the split of ONE 64-frame batch by frame is reported in roofline.strong_split")
    else:
        sharding = f"strong scaling: one {N_FRAMES}-frame batch split by frame over {n_gpus} GPU(s), {frames_per_gpu} frames each; no collective"
    return {
        "workload": "batched_crop_resize = BASELINE configs[3]: 1920x1080 uchar3 frames, 32 random crops each "
                    "(w,h in 16..512, clipped), Resize INTER_LINEAR PRESERVE_AR to 224x224 bg (114,114,114), Mul 1/255, "
                    "float3 tensor 224x224xplanes",
        "frames_per_gpu": frames_per_gpu, "crops_per_frame": CROPS_PER_FRAME, "planes_per_gpu": frames_per_gpu * CROPS_PER_FRAME,
        "sharding": sharding,
        "l2": "inputs + outputs per launch (1.6 GB per GPU at 64 frames) exceed the 126 MB L2; no flush needed",
        "timing": "W warm-up launches and 50 ms of the same launch after the barrier (clock ramp), then the K launches, captured "
                  "into one CUDA graph, replayed between two CUDA events (device time, max over ranks); --stream-launches "
                  "submits them one by one instead; roofline.sustained is the same replay after 0.6 s of continuous launches",
    }


# ---------------------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU through NVML (read-only) while the benchmark runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x2: "applications_clocks_setting", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting", 0x10: "sync_boost"}

    def __init__(self, cuda_index: int, period_s: float = 0.05):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.period = period_s
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            try:  # the CUDA ordinal is not the NVML index when CUDA_VISIBLE_DEVICES is set: go through the UUID
                self.h = pynvml.nvmlDeviceGetHandleByUUID("GPU-" + str(torch.cuda.get_device_properties(cuda_index).uuid))
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(cuda_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                self.samples.append((mhz, 0))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        mhz = sorted(m for m, _ in self.samples)
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(mhz)}


# ---------------------------------------------------------------------------------------------------------------
# the reference CPU arm
# ---------------------------------------------------------------------------------------------------------------
def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_time_sample(sample_frames: int, threads: int, repeats: int):
    """Times the CPU implementation on `sample_frames` frames of the workload.  Returns (best seconds, pixels, kind)."""
    import oracle
    wl = make_workload(0, n_frames=sample_frames)
    kind = "reference" if oracle.have_ref() else "port"
    run = (lambda: oracle.run_ref(wl, threads=threads)) if kind == "reference" else (lambda: oracle.run_oracle(wl, threads=threads))
    run()  # warm: page-faults the output
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        run()
        best = min(best, time.perf_counter() - t0)
    return best, wl.out_pixels, kind


def reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    threads = host_threads()
    sample_frames = 16
    wl = make_workload(0, n_frames=sample_frames)
    kind = "reference" if oracle.have_ref() else "port"
    run = (lambda: oracle.run_ref(wl, threads=threads)) if kind == "reference" else (lambda: oracle.run_oracle(wl, threads=threads))
    for _ in range(max(1, args.warmup)):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = (time.perf_counter() - t0) / args.steps
    value = wl.out_pixels / dt / 1e9
    sample = (f"{sample_frames} of the 64 frames ({sample_frames * CROPS_PER_FRAME} planes, {wl.out_pixels} output pixels) per step; "
              f"the reference CPU backend is single-threaded, so the planes are spread over {threads} threads as independent calls")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {**workload_config(args.gpus, args.scaling, N_FRAMES), "timing": "host wall clock around each step of the CPU backend"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------------------
def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (earlier measurement on this pool)"


def time_launches(fn, steps: int, torch) -> float:
    """Device time in seconds of `steps` calls of fn() on the current stream (CUDA events, synchronised both sides)."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / 1e3


def other_configs(torch, steps: int, peak: float, widened: bool = False) -> dict:
    """Kernel-only figures of the other four configurations on one GPU.  Their launches last a few microseconds, less
    than the host needs to submit one, so rounds over all buffer sets are captured into one CUDA graph (about two
    milliseconds of work: a replay far outlasts the host's cost of submitting it) and the graph is replayed; rotating the
    buffer sets (together larger than the L2) makes every launch read from HBM."""
    from fusedkernellibrary_b200 import abi, runtime, workloads as W
    out = {}
    cases = [("readme_crops", W.readme_crops), ("vertical_fusion", W.vertical_fusion),
             ("nv12_preprocess", W.nv12_preprocess), ("divergent_planes", W.divergent_planes)]
    if widened:
        # the chains beside the five configurations (border handling, other YCbCr sources, conditional batches, planar and
        # YCbCr destinations), each on a launch large enough to time
        cases = [
            ("uchar4_batched_crop_resize", lambda: W.batched_crop_resize(n_frames=8, crops_per_frame=32, src4=True)),
            ("four_channel_crops", lambda: W.rgba_crops(dst=(224, 224), rects=tuple((30 * i, 15 * i, 200 + 8 * i, 160 + 4 * i) for i in range(32)))),
            ("border_replicate_crops", lambda: W.border_crops(abi.BORDER_REPLICATE, w=1920, h=1080, dst=(224, 224))),
            ("nv21_limited_bt601_preprocess", lambda: W.nv12_preprocess(src_format=abi.PIX_NV21, colour=(abi.RANGE_LIMITED, abi.PRIMITIVES_BT601))),
            ("uyvy_preprocess", lambda: W.nv12_preprocess(src_format=abi.PIX_UYVY, colour=(abi.RANGE_FULL, abi.PRIMITIVES_BT709))),
            ("p010_limited_bt2020_preprocess", lambda: W.nv12_preprocess(src_format=abi.PIX_P010, colour=(abi.RANGE_LIMITED, abi.PRIMITIVES_BT2020))),
            ("bgr_to_rgba_crops", lambda: W.add_alpha_crops(swap=True, w=1920, h=1080, dst=(224, 224))),
            ("conditional_batch_resize", lambda: W.conditional_resize(used=6, w=1920, h=1080, dst=(640, 360))),
            ("tensor_t_split_resize", lambda: W.tsplit_resize(w=1920, h=1080, dst=(640, 360))),
            ("split_planes_resize", lambda: W.split_planes(w=1920, h=1080, dst=(960, 540))),
            ("rgb_to_nv12_image", lambda: W.rgb_to_yuv_image(abi.PIX_NV12, (abi.RANGE_LIMITED, abi.PRIMITIVES_BT709), w=1920, h=1080)),
        ]
    for name, factory in cases:
        wl = factory()
        alg = wl.algorithmic_bytes()
        footprint = sum(s.nbytes for s in wl.sources) + sum(wl.out_sizes)
        n_sets = max(1, min(8, int(400e6 // footprint) + 1))
        sets = [runtime.DeviceWorkload(wl, poison=None) for _ in range(n_sets)]
        for s in sets:
            s.plan()
        for _ in range(3):  # warm-up outside the capture (first launches configure the kernels)
            for s in sets:
                s.launch_plan()
        torch.cuda.synchronize()
        # A replay must last much longer than the host needs to submit it (tens of microseconds), or the figure is the
        # host's replay rate: as many rounds over the sets go into one graph as fill about two milliseconds.
        def one_round():
            for s in sets:
                s.launch_plan()
        est = time_launches(one_round, 3, torch) / 3
        inner = max(1, min(64, int(2e-3 / max(est, 1e-6)) + 1))
        side = torch.cuda.Stream()

        def capture(body):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    for _ in range(inner):
                        body()
            g.replay()
            return g
        graph = capture(one_round)
        rounds = max(10, steps // 2)  # replays per measurement; the median of five measurements is reported

        def median_time(replay):
            return sorted(time_launches(replay, rounds, torch) / (rounds * inner * n_sets) for _ in range(5))[2]
        dt = median_time(graph.replay)
        ref_us = None
        try:
            import oracle
            if oracle.have_ref_cuda():
                launchers = [oracle.ref_cuda_launcher(wl, [t.data_ptr() for t in s.src], [t.data_ptr() for t in s.out], side.cuda_stream) for s in sets]
                if launchers[0] is not None:
                    for fn in launchers:
                        fn()
                    torch.cuda.synchronize()
                    def ref_round():
                        for fn in launchers:
                            fn()
                    ref_graph = capture(ref_round)
                    ref_us = median_time(ref_graph.replay) * 1e6
                    del ref_graph
        except Exception as exc:  # the comparison is optional; the product's figures never depend on it
            ref_us = f"failed: {exc}"
        out[name] = {"us_per_launch": dt * 1e6, "reference_cuda_us_per_launch": ref_us, "gpix_s": wl.out_pixels / dt / 1e9, "alg_bytes": alg["total"],
                     "hbm_gbs": alg["total"] / dt / 1e9, "frac_of_measured_peak": alg["total"] / dt / 1e9 / peak,
                     "buffer_sets_rotated": n_sets, "kernels_per_launch": sets[0].kernel_launches(),
                     "rounds_per_graph": inner,
                     "timing": "CUDA graph of rounds_per_graph rounds over the buffer sets (about 2 ms of work), replayed; median of five measurements"}
        del graph
        for s in sets:
            s.close()
        del sets
        torch.cuda.empty_cache()
    return out


def reference_cuda_main(torch, wl, dw, steps: int, our_ms: float) -> dict:
    """The reference library's own CUDA backend (its generic templated kernel compiled for sm_100a, oracle/_ref) on the
    same resident buffers: a comparison figure beside the product's, not part of the product's path.  Its output is
    compared with ours (the reference contracts to FMA, so the last bit may differ; tolerance 1e-5 relative)."""
    import oracle
    if not oracle.have_ref_cuda():
        return {"unavailable": "oracle/_ref/libfkl_ref_cuda.so was not built (reference headers or nvcc absent at build time)"}
    from fusedkernellibrary_b200 import runtime
    ours = dw.out[0].view(torch.float32).clone()
    launch = oracle.ref_cuda_launcher(wl, [t.data_ptr() for t in dw.src], [t.data_ptr() for t in dw.out], runtime.current_stream_ptr())
    kernels = launch()
    torch.cuda.synchronize()
    theirs = dw.out[0].view(torch.float32)
    rel = ((theirs - ours).abs() / ours.abs().clamp_min(1e-30)).max().item()
    for _ in range(2):
        launch()
    dt = time_launches(launch, steps, torch) / steps
    del ours
    return {"ms_per_step": dt * 1e3, "value": wl.out_pixels / dt / 1e9, "unit": UNIT, "kernel_launches_per_step": kernels,
            "max_rel_diff_vs_ours": rel, "speedup_of_ours": dt * 1e3 / our_ms,
            "note": "reference templated kernel, nvcc 12.9 sm_100a, 256 planes per launch (kernel-parameter limit)"}


def timed_plan_launches(sets, rounds: int, torch, barrier=None, stretch_s: float = 0.05, n_streams: int = 1) -> float:
    """Seconds per launch of the plans of `sets` (DeviceWorkloads rotated so that every launch reads HBM): `rounds` rounds
    over the sets are captured into one CUDA graph; after `barrier` every rank first replays it for `stretch_s` (clocks up),
    then one replay is timed with CUDA events.  With n_streams > 1 consecutive launches (of different sets: independent
    batches) alternate between that many streams inside the graph, so one launch's ramp-up runs under the tail of the
    launch before it: the throughput of a stream of batches rather than the duration of a launch."""
    for s in sets:
        s.plan()
    for _ in range(3):
        for s in sets:
            s.launch_plan()
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    others = [torch.cuda.Stream() for _ in range(n_streams - 1)]
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for o in others:
                o.wait_stream(side)
            k = 0
            for _ in range(rounds):
                for s in sets:
                    with torch.cuda.stream(side if k % n_streams == 0 else others[k % n_streams - 1]):
                        s.launch_plan()
                    k += 1
            for o in others:
                side.wait_stream(o)
    graph.replay()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    t_end = time.perf_counter() + stretch_s
    while time.perf_counter() < t_end:
        graph.replay()
        torch.cuda.synchronize()
    dt = sorted(time_launches(graph.replay, 1, torch) for _ in range(3))[1]
    del graph
    return dt / (rounds * len(sets))


def rotating_sets(wl, runtime, target_bytes: float = 300e6, max_sets: int = 8, min_sets: int = 1):
    """Enough independent copies of a workload's buffers that one round over them moves more bytes than the L2 holds."""
    touched = max(1, wl.algorithmic_bytes()["total"])
    n = max(min_sets, min(max_sets, int(target_bytes // touched) + 1))
    return [runtime.DeviceWorkload(wl, poison=None) for _ in range(n)]


def gather_max(value: float, torch, dist, world: int):
    """(max over ranks, list by rank) of a per-rank float."""
    if world == 1:
        return value, [value]
    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    every = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(every, t)
    vals = [float(e.item()) for e in every]
    return max(vals), vals


def strong_split(rank: int, world: int, steps: int, t1_ms: float, t1_two_ms: float, torch, dist) -> dict:
    """ONE 64-frame batch divided by frame over the ranks (what the workload description asks of 2, 4 and 8 GPUs): every
    rank runs its 64 / world frames; time = the slowest rank's; efficiency against one GPU doing all 64 frames in this
    same run (t1_ms, the mean of the ranks' full-job times).  `two_streams` is the same split as a stream of batches:
    consecutive batches alternate between two CUDA streams (against t1_two_ms, one GPU doing whole batches that way)."""
    from fusedkernellibrary_b200 import runtime, workloads as W
    shard = W.shard_by_frame(make_workload(0), rank, world)
    sets = rotating_sets(shard, runtime, min_sets=2)
    sec = timed_plan_launches(sets, max(5, steps), torch, barrier=dist.barrier)
    sec2 = timed_plan_launches(sets, max(5, steps), torch, barrier=dist.barrier, n_streams=2)
    for s in sets:
        s.close()
    t_max, by_rank = gather_max(sec * 1e3, torch, dist, world)
    t2_max, _ = gather_max(sec2 * 1e3, torch, dist, world)
    total_px = N_FRAMES * CROPS_PER_FRAME * 224 * 224
    return {"what": f"one {N_FRAMES}-frame batch split by frame, {N_FRAMES // world} frames ({N_FRAMES // world * CROPS_PER_FRAME} planes) per GPU",
            "ms_per_step": t_max, "ms_per_step_by_rank": by_rank, "gpix_s": total_px / (t_max / 1e3) / 1e9,
            "one_gpu_ms_same_run": t1_ms, "speedup_vs_one_gpu": t1_ms / t_max, "efficiency": t1_ms / (world * t_max),
            "two_streams": {"what": "consecutive batches alternate between two CUDA streams (a stream of batches: one launch's "
                                    "ramp-up runs under the tail of the launch before it)",
                            "ms_per_step": t2_max, "gpix_s": total_px / (t2_max / 1e3) / 1e9, "one_gpu_ms_same_run": t1_two_ms,
                            "efficiency": t1_two_ms / (world * t2_max)},
            "buffer_sets_rotated": len(sets)}


def config5_sharded(rank: int, world: int, steps: int, peak: float, torch, dist) -> dict:
    """The divergent 8-plane launch (benchmark configuration 5) with its planes dealt over the ranks, plane z to rank z % world, so
    that resize planes and arithmetic planes are spread evenly.  Rank 0 also times the whole launch on its one GPU."""
    from fusedkernellibrary_b200 import runtime, workloads as W
    wl = W.divergent_planes()
    shard = W.shard_by_plane(wl, rank, world)
    sets = rotating_sets(shard, runtime)
    sec = timed_plan_launches(sets, max(5, steps), torch, barrier=dist.barrier)
    for s in sets:
        s.close()
    del sets
    torch.cuda.empty_cache()
    t_max, by_rank = gather_max(sec * 1e3, torch, dist, world)
    t1 = 0.0
    if rank == 0:
        whole = rotating_sets(wl, runtime)
        t1 = timed_plan_launches(whole, max(5, steps), torch) * 1e3
        for s in whole:
            s.close()
    t1, _ = gather_max(t1, torch, dist, world)
    per_plane = [W.shard_by_plane(wl, z, len(wl.planes)).algorithmic_bytes()["total"] for z in range(len(wl.planes))]
    heaviest = max(sum(per_plane[z] for z in part) for part in W.plane_partition(len(wl.planes), world))
    total = wl.algorithmic_bytes()["total"]
    return {"what": f"8 planes dealt over {world} GPUs (plane z on rank z % {world})", "ms_per_step": t_max, "ms_per_step_by_rank": by_rank,
            "gpix_s": wl.out_pixels / (t_max / 1e3) / 1e9, "one_gpu_ms_same_run": t1, "speedup_vs_one_gpu": t1 / t_max,
            "ideal_speedup_cap": total / heaviest, "fraction_of_cap": (t1 / t_max) / (total / heaviest),
            "heaviest_rank_hbm_gbs": heaviest / (t_max / 1e3) / 1e9, "heaviest_rank_frac_of_peak": heaviest / (t_max / 1e3) / 1e9 / peak}


def host_cost(dw, lib, abi, torch) -> dict:
    """Synchronous host time of one launch of the 2048-plane workload with host descriptors, the GPU idle before every
    call: fkb_launch_transform through ctypes, and fk::executeOperations through the C++ front end (bench_frontend.cpp)."""
    import subprocess
    out = {}
    stream = torch.cuda.current_stream().cuda_stream
    ts = []
    for i in range(25):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        rc = lib.fkb_launch_transform(dw.chains, dw.planes, dw.n_planes, stream)
        t1 = time.perf_counter()
        abi.check(rc)
        if i >= 5:
            ts.append((t1 - t0) * 1e6)
    torch.cuda.synchronize()
    ts.sort()
    out["fkb_launch_transform_us"] = {"median": ts[len(ts) // 2], "min": ts[0], "planes": dw.n_planes, "via": "ctypes"}
    exe = os.path.join(ROOT, "fusedkernellibrary_b200", "lib", "bench_frontend")
    if os.path.exists(exe):
        try:
            r = subprocess.run([exe, "30"], capture_output=True, text=True, timeout=120)
            out["fk_executeOperations_us"] = json.loads(r.stdout.strip().splitlines()[-1])
        except Exception as exc:
            out["fk_executeOperations_us"] = {"error": str(exc)}
    else:
        out["fk_executeOperations_us"] = {"error": "bench_frontend was not built"}
    out["reference_quotes_us_per_call"] = "19-70 (.github/skills/fkl-language-bindings/SKILL.md:90)"
    return out


def our_arm(args) -> None:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from fusedkernellibrary_b200 import abi, runtime
    wl, frames = shard_workload(rank, world, args.scaling)
    alg = wl.algorithmic_bytes()
    peak, peak_src = measured_peak()

    dw = runtime.DeviceWorkload(wl, poison=None)
    dw.plan()
    kernels_per_step = dw.kernel_launches()

    sampler = ClockSampler(torch.cuda.current_device(), period_s=0.004)
    for _ in range(max(3, args.warmup)):
        dw.launch_plan()
    torch.cuda.synchronize()
    # The K timed launches are captured once into a CUDA graph and replayed inside the CUDA-event bracket: the device
    # time of K back-to-back launches must not depend on how promptly the host thread gets to submit each one (with
    # one process per GPU and a clock sampler in each, eight ranks can outnumber the cores a box gives them).
    # --stream-launches submits them one by one instead.
    if args.stream_launches:
        timed = lambda: [dw.launch_plan() for _ in range(args.steps)]
    else:
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(args.steps):
                    dw.launch_plan()
        graph.replay()
        torch.cuda.synchronize()
        timed = graph.replay
    if world > 1:
        dist.barrier()
    # Ranks reach the barrier seconds apart (set-up times differ), and a GPU that idled there has dropped its clocks:
    # a few milliseconds of timed work right after the barrier would mostly measure the ramp back up.  So every rank
    # first runs a short stretch of the same launch (50 ms, during which the clock samples start), and the timed
    # launches follow it without a pause.  That is the headline: a kernel timed alone, as the copy that gave the
    # roofline's denominator was (best of ten 0.7 ms copies).  After about a tenth of a second of back-to-back launches
    # the GPU reaches its power limit and lowers the SM clock; the same replay timed in that state is reported beside
    # the headline as roofline.sustained.
    def stretch(seconds: float) -> None:
        t_end = time.perf_counter() + seconds
        while time.perf_counter() < t_end:
            for _ in range(20):
                dw.launch_plan()
            torch.cuda.synchronize()

    sampler.start()
    stretch(0.05)
    dt = time_launches(timed, 1, torch)
    stretch(0.03)
    clocks = sampler.stop()
    sustained_sampler = ClockSampler(torch.cuda.current_device(), period_s=0.02)
    sustained_sampler.start()
    stretch(0.6)
    dt_sustained = time_launches(timed, 1, torch)
    stretch(0.2)
    clocks_sustained = sustained_sampler.stop()
    if world > 1:
        dist.barrier()
    abi.check(abi.load().fkb_device_status())
    per_rank_ms = [dt / args.steps * 1e3]
    if world > 1:
        t = torch.tensor([dt], device="cuda", dtype=torch.float64)
        every = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        per_rank_ms = [float(e.item()) / args.steps * 1e3 for e in every]
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
        # every rank's clock record: the line reports the slowest GPU's clock and the union of the reasons, and keeps
        # the list, so that a GPU left with locked clocks shows next to its step time
        by_rank = [None] * world
        dist.all_gather_object(by_rank, clocks)
        known = [c["sm_mhz"] for c in by_rank if c.get("sm_mhz") is not None]
        clocks = {"sm_mhz": min(known) if known else None, "sm_max_mhz": clocks.get("sm_max_mhz"),
                  "reasons": sorted({r for c in by_rank for r in c.get("reasons", [])}),
                  "samples": sum(c.get("samples", 0) for c in by_rank),
                  "sm_mhz_by_rank": [c.get("sm_mhz") for c in by_rank]}
    if world > 1:
        t = torch.tensor([dt_sustained], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt_sustained = float(t.item())
        by_rank = [None] * world
        dist.all_gather_object(by_rank, clocks_sustained)
        known = [c["sm_mhz"] for c in by_rank if c.get("sm_mhz") is not None]
        clocks_sustained = {"sm_mhz": min(known) if known else None, "sm_max_mhz": clocks_sustained.get("sm_max_mhz"),
                            "reasons": sorted({r for c in by_rank for r in c.get("reasons", [])}),
                            "samples": sum(c.get("samples", 0) for c in by_rank)}
    ms_per_step = dt / args.steps * 1e3
    total_pixels = wl.out_pixels * world
    value = total_pixels / (dt / args.steps) / 1e9
    achieved = alg["total"] / (dt / args.steps) / 1e9

    # ---- end to end through the public entry point with host buffers: pinned sources up, launch, tensor down ----
    h_src = [torch.from_numpy(s).pin_memory() for s in wl.sources]
    lib = abi.load()

    # A step is pipelined by groups of frames on three streams, as a user feeding a camera batch would: upload the
    # frames of group g, launch the fused kernel over that group's planes (fkb_launch_transform with host descriptors),
    # download its planes of the tensor.  Consecutive steps alternate between two sets of device and pinned buffers, so
    # the uploads of step i + 1 run under the downloads of step i (a stream of batches, not one batch at a time): the host
    # link is busy in both directions all the time; every byte of every step still crosses it inside the timed region.
    group = 4  # frames per group
    n_groups = (len(h_src) + group - 1) // group
    planes_per_frame = dw.n_planes // len(h_src)
    plane_bytes = wl.out_sizes[0] // dw.n_planes
    s_up, s_run, s_down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    sets = [dw, runtime.DeviceWorkload(wl, poison=None)]
    # the same launches as a stream of independent batches: consecutive launches alternate between two CUDA streams
    two_sec = timed_plan_launches(sets, max(3, args.steps // 2), torch, barrier=dist.barrier if world > 1 else None, n_streams=2)
    two_ms, two_by_rank = gather_max(two_sec * 1e3, torch, dist, world)
    h_out = [torch.empty(wl.out_sizes[0], dtype=torch.uint8).pin_memory() for _ in sets]
    sub_planes = []
    for d in sets:
        per_set = []
        for g in range(n_groups):
            lo, hi = g * group * planes_per_frame, min((g + 1) * group, len(h_src)) * planes_per_frame
            arr = (abi.PlaneDesc * (hi - lo))()
            for i in range(hi - lo):
                arr[i] = d.planes[lo + i]
            per_set.append((lo, hi, arr))
        sub_planes.append(per_set)

    def run_steps(n_steps: int, with_kernels: bool):
        """n_steps steps back to back; with_kernels=False leaves the launches out (the copy bound)."""
        cur = torch.cuda.current_stream()
        for st in (s_up, s_run, s_down):
            st.wait_stream(cur)
        ran_all = [None, None]    # per buffer set: the last kernel that read its frames / the last download of its tensor
        down_all = [None, None]
        for step in range(n_steps):
            k = step % 2
            d = sets[k]
            if ran_all[k] is not None:
                s_up.wait_event(ran_all[k])     # the frames of this set are free again
                s_run.wait_event(down_all[k])   # and so is its output tensor
            for g, (lo, hi, arr) in enumerate(sub_planes[k]):
                with torch.cuda.stream(s_up):
                    for f in range(g * group, min((g + 1) * group, len(h_src))):
                        d.src[f].copy_(h_src[f], non_blocking=True)
                    up = s_up.record_event()
                with torch.cuda.stream(s_run):
                    s_run.wait_event(up)
                    if with_kernels:
                        abi.check(lib.fkb_launch_transform(d.chains, arr, hi - lo, s_run.cuda_stream))
                    ran = s_run.record_event()
                with torch.cuda.stream(s_down):
                    s_down.wait_event(ran)
                    h_out[k][lo * plane_bytes: hi * plane_bytes].copy_(d.out[0][lo * plane_bytes: hi * plane_bytes], non_blocking=True)
            ran_all[k] = ran
            down_all[k] = s_down.record_event()
        for st in (s_up, s_run, s_down):
            cur.wait_stream(st)

    e2e_steps = max(2, min(args.steps, 10))
    run_steps(2, True)
    if world > 1:
        dist.barrier()
    e2e_dt = time_launches(lambda: run_steps(e2e_steps, True), 1, torch)
    e2e_dt, _ = gather_max(e2e_dt, torch, dist, world)
    # the same copies without any kernel: what the host <-> device link of this box gives the steps at best
    run_steps(2, False)
    if world > 1:
        dist.barrier()
    copy_dt = time_launches(lambda: run_steps(e2e_steps, False), 1, torch)
    copy_dt, _ = gather_max(copy_dt, torch, dist, world)
    sets[1].close()
    e2e_value = total_pixels / (e2e_dt / e2e_steps) / 1e9
    h2d = sum(s.nbytes for s in wl.sources) + dw.n_planes * 224  # frames + one 224-byte plane record per plane
    d2h = wl.out_sizes[0]

    traffic, traffic_src = profiled_traffic(dw.n_planes)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "traffic_source": traffic_src, "peak_source": peak_src, "kernel": "fkb::staged_kernel",
                "algorithmic_bytes_per_launch": alg["total"], "frac_of_nominal_8TBs": achieved / 8000.0,
                "sustained": {"what": "the same K launches timed again after 0.6 s of back-to-back launches, when the GPU "
                                      "has reached its power limit (the headline is timed after 50 ms, like the copy that "
                                      "gave the peak)",
                              "ms_per_step": dt_sustained / args.steps * 1e3,
                              "frac": alg["total"] / (dt_sustained / args.steps) / 1e9 / peak, "clocks": clocks_sustained},
                "two_streams": {"what": "throughput of a stream of independent batches: consecutive launches (two buffer sets) "
                                        "alternate between two CUDA streams, so one launch's ramp-up runs under the tail of the "
                                        "launch before it; time per launch = time of the replay / launches, max over ranks",
                                "ms_per_step": two_ms, "gpix_s": total_pixels / (two_ms / 1e3) / 1e9,
                                "frac": alg["total"] / (two_ms / 1e3) / 1e9 / peak}}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(world, args.scaling, frames), "ms_per_step_by_rank": per_rank_ms,
        "roofline": roofline,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_dt / e2e_steps * 1e3, "steps": e2e_steps,
                "copy_bound_ms": copy_dt / e2e_steps * 1e3, "frac_of_copy_bound": copy_dt / e2e_dt,
                "copy_bound_gbs_per_gpu": (h2d + d2h) / (copy_dt / e2e_steps) / 1e9,
                "copy_bound": "the same pinned host <-> device copies on the same streams without any kernel, slowest rank: "
                              "the step cannot be faster than this on this box",
                "path": "per group of 4 frames on three streams: pinned host frames -> device, fkb_launch_transform (host "
                        "descriptors) over the group's planes, its planes of the float3 tensor -> pinned host; consecutive "
                        "steps alternate between two buffer sets, so one step's uploads run under the previous step's downloads"},
        "gpu_launches": args.steps * kernels_per_step,
        "clocks": clocks,
    }
    if world > 1 and args.scaling == "weak" and not args.no_other_configs:
        # the splits of ONE job the workload descriptions name, beside the weak-scaling headline
        dw.close()
        del dw, h_src, h_out, sets
        torch.cuda.empty_cache()
        t1_ms = sum(per_rank_ms) / len(per_rank_ms)
        roofline["strong_split"] = strong_split(rank, world, min(args.steps, 20), t1_ms, sum(two_by_rank) / len(two_by_rank), torch, dist)
        roofline["config5_sharded"] = config5_sharded(rank, world, min(args.steps, 20), peak, torch, dist)
    if rank == 0 and world == 1:
        roofline["host_cost"] = host_cost(dw, lib, abi, torch)
        if not args.no_cpu_baseline:
            threads = host_threads()
            sample_frames = 16
            best, px, kind = cpu_time_sample(sample_frames, threads, repeats=3)
            one, px1, _ = cpu_time_sample(2, 1, repeats=2)
            line["cpu_baseline"] = {"value": px / best / 1e9, "unit": UNIT, "cores": threads, "kind": kind,
                                    "sample": f"{sample_frames} of the 64 frames ({sample_frames * CROPS_PER_FRAME} planes), best of 3, "
                                              f"planes spread over {threads} host threads as independent single-threaded reference calls",
                                    "one_thread": {"value": px1 / one / 1e9, "unit": UNIT, "cores": 1,
                                                   "sample": "2 of the 64 frames (64 planes), best of 2: the backend as shipped (single-threaded)"}}
        ref_cuda = reference_cuda_main(torch, wl, dw, max(5, min(args.steps, 20)), ms_per_step)
        roofline["reference_cuda_backend"] = ref_cuda
        if not args.no_other_configs:
            dw.close()
            del dw, sets, h_src, h_out
            torch.cuda.empty_cache()
            steps_small = max(10, min(args.steps, 50))
            roofline["by_config"] = compact(other_configs(torch, steps_small, peak))
            roofline["by_config"]["batched_crop_resize"] = {"us": ms_per_step * 1e3, "ref_cuda_us": ref_cuda.get("ms_per_step", 0) * 1e3 or None,
                                                            "frac": achieved / peak, "gbs": achieved, "kernels": kernels_per_step}
            roofline["widened_rows"] = compact(other_configs(torch, steps_small, peak, widened=True))
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def compact(configs: dict) -> dict:
    """The per-configuration figures in the few keys that matter (they travel inside `roofline`)."""
    return {name: {"us": round(v["us_per_launch"], 3), "ref_cuda_us": (round(v["reference_cuda_us_per_launch"], 3)
                                                                         if isinstance(v["reference_cuda_us_per_launch"], float) else v["reference_cuda_us_per_launch"]),
                   "frac": round(v["frac_of_measured_peak"], 4), "gbs": round(v["hbm_gbs"], 1), "gpix_s": round(v["gpix_s"], 2),
                   "kernels": v["kernels_per_launch"]} for name, v in configs.items()}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak")
    ap.add_argument("--stream-launches", action="store_true", help="submit the timed launches one by one instead of replaying a CUDA graph of them")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        our_arm(args)


if __name__ == "__main__":
    main()
