"""Runs a few launches of one workload so that a profiler can capture them:

    python profile_case.py batched_crop_resize --frames 8 --launches 4
    python profile_case.py vertical_fusion --sets 4 --launches 8

The case is kept small (a few hundred MB on the device, but more than the 126 MB L2) so that a multi-pass capture
ends by itself quickly.  Prints the CUDA-event time per launch of the un-profiled run.
"""
from __future__ import annotations

import argparse

import torch

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from fusedkernellibrary_b200 import runtime, workloads as W  # noqa: E402


# workloads beside the five configurations that have a profile of their own
EXTRA = {
    # 32 crops of one 1920x1080 uchar4 frame -> 224x224 uchar4 (the four-channel chain of the benchmark's widened rows)
    "four_channel_crops": lambda: W.rgba_crops(dst=(224, 224), rects=tuple((30 * i, 15 * i, 200 + 8 * i, 160 + 4 * i) for i in range(32))),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("workload", choices=sorted(W.CONFIGS) + sorted(EXTRA))
    ap.add_argument("--frames", type=int, default=8, help="batched_crop_resize: frames (32 crops each)")
    ap.add_argument("--sets", type=int, default=1, help="rotate this many independent buffer sets (defeats the L2)")
    ap.add_argument("--launches", type=int, default=4)
    args = ap.parse_args()
    if args.workload == "batched_crop_resize":
        wl = W.batched_crop_resize(n_frames=args.frames)
    elif args.workload in EXTRA:
        wl = EXTRA[args.workload]()
    else:
        wl = W.CONFIGS[args.workload]()
    sets = [runtime.DeviceWorkload(wl, poison=None) for _ in range(args.sets)]
    for s in sets:
        s.plan()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.launches):
        sets[i % args.sets].launch_plan()
    stop.record()
    torch.cuda.synchronize()
    alg = wl.algorithmic_bytes()["total"]
    print(f"{wl.name}: {args.launches} launches, {start.elapsed_time(stop) / args.launches * 1e3:.1f} us per launch, "
          f"algorithmic bytes per launch {alg}")
    for s in sets:
        s.close()


if __name__ == "__main__":
    main()
