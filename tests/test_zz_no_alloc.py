"""GPU test of fkb_launch_transform_noalloc, the entry point for callers that are not allowed to create memory at the
time they launch: a process whose GPU memory has been handed out in full, a serving loop with a no-allocation rule, or
code running where the CUDA runtime refuses allocation calls.  It keeps its plane records in a fixed array inside the
library instead of buffers created on demand, so it must (1) produce exactly what fkb_launch_transform produces, (2) do
so again on a second call that finds the first call's records still in the array, and (3) refuse more planes than the
array holds.  The file name sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes as C
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from fusedkernellibrary_b200 import abi, workloads as W

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

FILL = 0xCD


def run(wl, entry_name):
    """Uploads the workload, launches it through the named C-ABI entry point, returns the output bytes."""
    from fusedkernellibrary_b200 import runtime
    lib = abi.load()
    dw = runtime.DeviceWorkload(wl, poison=FILL)
    try:
        entry = getattr(lib, entry_name)
        abi.check(entry(dw.chains, dw.planes, dw.n_planes, runtime.current_stream_ptr()))
        return dw.results()
    finally:
        dw.close()


def test_noalloc_entry_matches_regular_entry_on_two_calls_in_a_row():
    assert torch.cuda.is_available()
    # first call: 300 planes (more than travel in the kernel parameters), crops + resize + normalise to float3
    first = W.batched_crop_resize(n_frames=3, crops_per_frame=100, w=320, h=240, dst=(32, 24), crop_range=(4, 100))
    # second call: fewer, different planes and another chain (uchar3 output), so records of the first call stay
    # behind in the shared array beyond the ones this call rewrites
    second = W.readme_crops()
    for wl in (first, second):
        want = run(wl, "fkb_launch_transform")
        got = run(wl, "fkb_launch_transform_noalloc")
        for g, w in zip(got, want):
            assert np.array_equal(g, w)  # same tolerance as every other parity test here: bit-identical
    assert abi.load().fkb_device_status() == abi.OK


def test_noalloc_entry_rejects_more_planes_than_its_array_holds():
    lib = abi.load()
    wl = W.readme_crops()
    from fusedkernellibrary_b200 import runtime
    dw = runtime.DeviceWorkload(wl)
    try:
        # the size check comes before anything reads the plane array, so the short array is never indexed past its end
        rc = lib.fkb_launch_transform_noalloc(dw.chains, dw.planes, abi.NOALLOC_MAX_PLANES + 1, None)
        assert rc == abi.ERR_TOO_LARGE
        assert b"too large" in lib.fkb_status_string(rc)
        assert lib.fkb_launch_transform_noalloc(None, dw.planes, 1, None) == abi.ERR_NULL
    finally:
        dw.close()


def test_noalloc_entry_takes_exactly_its_maximum_and_conditional_planes():
    # 4096 planes, the most the fixed array holds: 32 frames x 128 tiny crops
    full = W.batched_crop_resize(n_frames=32, crops_per_frame=128, w=320, h=240, dst=(16, 16), crop_range=(4, 60))
    assert len(full.planes) == abi.NOALLOC_MAX_PLANES
    # a conditional batch read: planes beyond the used ones yield their default value (FKB_PLANE_DEFAULT)
    conditional = W.conditional_resize(used=5)
    for wl in (full, conditional):
        want = run(wl, "fkb_launch_transform")
        got = run(wl, "fkb_launch_transform_noalloc")
        for g, w in zip(got, want):
            assert np.array_equal(g, w)
    assert abi.load().fkb_device_status() == abi.OK


ONLY_NOALLOC = textwrap.dedent('''
    import sys
    sys.path.insert(0, sys.argv[1])
    import numpy as np, torch
    from fusedkernellibrary_b200 import abi, runtime, workloads as W
    wl = W.batched_crop_resize(n_frames=3, crops_per_frame=100, w=320, h=240, dst=(32, 24), crop_range=(4, 100))
    lib = abi.load()
    dw = runtime.DeviceWorkload(wl, poison=0xCD)          # the caller's buffers exist before the window opens
    stream = runtime.current_stream_ptr()
    abi.check(lib.fkb_launch_transform_noalloc(dw.chains, dw.planes, dw.n_planes, stream))   # warm-up call: kernels get loaded
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    abi.check(lib.fkb_launch_transform_noalloc(dw.chains, dw.planes, dw.n_planes, stream))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    out = dw.results()[0]
    print("FREE", free_before, free_after, int(out.astype(np.uint64).sum()))
''')


def test_noalloc_entry_alone_in_a_fresh_process_leaves_free_memory_unchanged(tmp_path):
    """In a process that never calls any other launch entry point (so no arena exists), the device's free memory is the
    same before and after a call of the no-allocation entry point, and the output is the regular entry point's."""
    from conftest import ROOT
    script = tmp_path / "only_noalloc.py"
    script.write_text(ONLY_NOALLOC)
    r = subprocess.run([sys.executable, str(script), ROOT], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    fields = [l for l in r.stdout.splitlines() if l.startswith("FREE ")][0].split()
    assert fields[1] == fields[2], f"free device memory changed across the call: {fields[1]} -> {fields[2]}"
    wl = W.batched_crop_resize(n_frames=3, crops_per_frame=100, w=320, h=240, dst=(32, 24), crop_range=(4, 100))
    want = run(wl, "fkb_launch_transform")[0]
    assert int(fields[3]) == int(want.astype(np.uint64).sum())
