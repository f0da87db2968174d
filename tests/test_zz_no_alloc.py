"""GPU test of fkb_launch_transform_noalloc, the entry point for callers that are not allowed to create memory at the
time they launch: a process whose GPU memory has been handed out in full, a serving loop with a no-allocation rule, or
code running where the CUDA runtime refuses allocation calls.  It keeps its plane records in a fixed array inside the
library instead of buffers created on demand, so it must (1) produce exactly what fkb_launch_transform produces, (2) do
so again on a second call that finds the first call's records still in the array, and (3) refuse more planes than the
array holds.  The file name sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes as C

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
