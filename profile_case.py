"""Runs a few launches of one workload so that a profiler can capture them:

    python profile_case.py batched_crop_resize --frames 8 --launches 4
    python profile_case.py vertical_fusion --sets 4 --launches 8

    python -c "from fusedkernellibrary_b200 import build; print(build.build_phase_clocks())"      # once, needs no GPU
    FKB_LIBRARY=fusedkernellibrary_b200/lib/libfkb_phase.so python profile_case.py batched_crop_resize --frames 64 --phase-clocks

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


PHASES = ["wait for the source rows", "compute + fence + warp sync", "issue the bulk store", "commit the bulk group",
          "arrive + issue the two bulk loads", "wait for the previous store's read"]


def phase_clocks(sets, launches: int) -> None:
    """Prints, per resize row of one warp, the cycles lane 0 spent in each phase of staged_kernel's row loop."""
    import ctypes as C
    from fusedkernellibrary_b200 import abi
    lib = abi.load()
    if not hasattr(lib, "fkb_debug_phase_clocks"):
        raise SystemExit("FKB_LIBRARY must name the phase-clock build (fusedkernellibrary_b200.build.build_phase_clocks())")
    lib.fkb_debug_phase_clocks.argtypes = [C.POINTER(C.c_ulonglong), C.c_int, C.c_int]
    sets[0].launch_plan()  # warm-up
    assert lib.fkb_debug_phase_clocks(None, 0, 1) == 0
    for i in range(launches):
        sets[i % len(sets)].launch_plan()
    out = (C.c_ulonglong * 12)()
    assert lib.fkb_debug_phase_clocks(out, len(out), 0) == 0
    rows, items = max(1, out[6]), max(1, out[10])
    print(f"{launches} launches, {rows} resize rows in {items} items; cycles per row of one warp (lane 0's clock):")
    for i, name in enumerate(PHASES):
        print(f"  {name:40s} {out[i] / rows:8.1f}")
    print(f"cycles per item: set-up {out[8] / items:.1f}, waiting for the first row's source rows {out[9] / items:.1f}, "
          f"whole item {out[7] / items:.1f} ({rows / items:.2f} rows per item)")
    for s in sets:
        s.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("workload", choices=sorted(W.CONFIGS) + sorted(EXTRA))
    ap.add_argument("--frames", type=int, default=8, help="batched_crop_resize: frames (32 crops each)")
    ap.add_argument("--sets", type=int, default=1, help="rotate this many independent buffer sets (defeats the L2)")
    ap.add_argument("--launches", type=int, default=4)
    ap.add_argument("--phase-clocks", action="store_true",
                    help="with FKB_LIBRARY naming the phase-clock build: cycles per resize row that a warp of staged_kernel spends in each phase")
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
    if args.phase_clocks:
        phase_clocks(sets, args.launches)
        return
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
