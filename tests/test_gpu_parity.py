"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a real GPU.

Tolerances of the contract: bit-exact for integer-only chains, <= 1 LSB per channel for uchar outputs after float
arithmetic, <= 1e-5 relative for float outputs.  The kernels follow the reference's operation order without FMA
contraction, so these tests assert the stronger property — bit-identical output buffers — and the stated tolerances
are checked as a consequence (``TOL_*`` below document them; a failure prints how far off the result is).
"""
import os

import numpy as np
import pytest

import oracle
from conftest import GOLDEN_CASES, conversion_kat_workload, ycbcr_round_trip, load_golden, read_uyvy_kat_workload, reference_kats
from fusedkernellibrary_b200 import abi, workloads as W

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL_U8_LSB = 1      # contract for uchar outputs after float math
TOL_F32_REL = 1e-5  # contract for float outputs
FILL = 0xCD         # bytes a launch must leave untouched (row padding, unused planes) keep this value


@pytest.fixture(scope="module", autouse=True)
def _needs_gpu():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    assert os.path.exists(abi.LIB_PATH), "libfkb.so missing: the CUDA path cannot run (no fallback exists)"


def gpu_run(wl, use_plan=False, force_gather=False, fill=FILL, tiny_route=False):
    """tiny_route=False switches off the routing of very small launches to the general kernel, so that small test
    cases still exercise the pipelined kernels; test_tiny_launch_routing covers the default behaviour."""
    from fusedkernellibrary_b200 import runtime
    os.environ["FKB_FORCE_GATHER"] = "1" if force_gather else "0"
    if tiny_route:
        os.environ.pop("FKB_TINY_PIXELS", None)
    else:
        os.environ["FKB_TINY_PIXELS"] = "0"
    try:
        dw = runtime.DeviceWorkload(wl, poison=fill)
        try:
            dw.launch_plan() if use_plan else dw.launch()
            return dw.results()
        finally:
            dw.close()
    finally:
        os.environ["FKB_FORCE_GATHER"] = "0"
        os.environ.pop("FKB_TINY_PIXELS", None)


def assert_same(wl, got, want):
    from fusedkernellibrary_b200 import runtime
    for i, (g, w) in enumerate(zip(got, want)):
        if np.array_equal(g, w):
            continue
        fmt = wl.chains[wl.planes[0].chain if len(wl.out_sizes) == 1 else i].dst_format
        loose = runtime.compare(g, w, fmt, TOL_U8_LSB, TOL_F32_REL)
        first = int(np.flatnonzero(g != w)[0])
        raise AssertionError(f"{wl.name} output {i}: {int((g != w).sum())} differing bytes (first at {first}); "
                             f"within contract tolerance: {loose}")


def check(wl, **kw):
    want = oracle.run_oracle(wl, threads=8, fill=FILL)
    assert_same(wl, gpu_run(wl, **kw), want)


SMALL = {
    "readme_crops": lambda: W.readme_crops(),
    "vertical_fusion": lambda: W.vertical_fusion(w=1280, h=96),
    "vertical_fusion_odd": lambda: W.vertical_fusion(w=333, h=41, pitch_align=64, dst_pitch_align=16),
    "nv12": lambda: W.nv12_preprocess(w=1280, h=720, dst=(320, 320)),
    "batched": lambda: W.batched_crop_resize(n_frames=4, crops_per_frame=8, w=960, h=540),
    "batched_tiny_crops": lambda: W.batched_crop_resize(n_frames=2, crops_per_frame=16, w=640, h=360, crop_range=(1, 40), dst=(96, 80)),
    "divergent": lambda: W.divergent_planes(n_per_seq=4, w=480, h=270),
    "divergent_odd": lambda: W.divergent_planes(n_per_seq=3, w=330, h=190),
    "crop_reorder": lambda: W.crop_reorder(n=5),
    # crops so thin that the letterboxed image has no column or no row (the whole plane is background), among usual ones
    "thin_crops": lambda: W.readme_crops(crops=((300, 125, 1, 500), (400, 125, 500, 1), (10, 10, 2, 700), (530, 270, 130, 140), (0, 0, 1, 1)), dst=(224, 224)),
    "rgba_crops": lambda: W.rgba_crops(),
    "rgba_crops_f32_reorder": lambda: W.rgba_crops(reorder=True, f32=True, w=333, h=211, dst=(77, 45), rects=((0, 0, 333, 211), (5, 7, 100, 90), (300, 180, 33, 31))),
    "rgba_crops_border": lambda: W.rgba_crops(w=200, h=120, dst=(64, 48), rects=((-20, -10, 90, 70), (150, 90, 120, 80), (10, 10, 50, 40)), border=abi.BORDER_CONSTANT),
    "rgba_crops_border_wrap": lambda: W.rgba_crops(f32=True, w=200, h=120, dst=(64, 48), rects=((-20, -10, 90, 70), (150, 90, 120, 80)), border=abi.BORDER_WRAP),
    "add_alpha_crops": lambda: W.add_alpha_crops(),
    "add_alpha_crops_f32_swap": lambda: W.add_alpha_crops(swap=True, f32=True, w=333, h=211, dst=(77, 45)),
    "add_alpha_image": lambda: W.add_alpha_image(),
    "add_alpha_image_swap": lambda: W.add_alpha_image(swap=True, w=1001, h=37),
    # gray conversions: one-channel outputs (uchar image; float / uchar tensors after a resize)
    "gray_image": lambda: W.gray_image(),
    "gray_image_bgra_odd": lambda: W.gray_image(bgr=True, src4=True, w=1001, h=37),
    "gray_image_4k": lambda: W.gray_image(bgr=True, w=3840, h=2160),
    "gray_crops_u8": lambda: W.gray_crops(),
    "gray_crops_f32_bgr": lambda: W.gray_crops(bgr=True, f32=True, w=333, h=211, dst=(77, 45), rects=((0, 0, 333, 211), (5, 7, 100, 60), (200, 100, 50, 111), (300, 200, 33, 11), (100, 50, 20, 20))),
    "bgra_crops": lambda: W.bgra_crops(),
    "batched_uchar4": lambda: W.batched_crop_resize(n_frames=4, crops_per_frame=8, w=960, h=540, src4=True),
    "bgra_crops_swap": lambda: W.bgra_crops(swap=True, w=333, h=97, dst=(111, 50)),
    "tsplit_resize": lambda: W.tsplit_resize(),
    "split_planes_f32": lambda: W.split_planes(),
    "split_planes_u8": lambda: W.split_planes(f32=False, dst=(333, 77)),
    "conditional_resize": lambda: W.conditional_resize(),
    "conditional_resize_large": lambda: W.conditional_resize(used=6, w=1920, h=1080, dst=(640, 360)),  # default planes as all-background planes
    "conditional_pointwise": lambda: W.conditional_pointwise(),
}


@pytest.mark.parametrize("case", reference_kats()["conversions"], ids=lambda c: c["code"])
def test_colour_conversion_known_answers_of_the_reference_tests(case):
    # utests/algorithm/image_processing/utest_color_conversion.h:76-101, 144-168, through the C ABI
    wl, want = conversion_kat_workload(case)
    for kw in [dict(), dict(tiny_route=True)]:
        assert np.array_equal(gpu_run(wl, **kw)[0][:want.size], want)


@pytest.mark.parametrize("case", reference_kats()["read_uyvy"], ids=lambda c: f"{c['w']}x{c['h']}")
def test_read_uyvy_known_answers_of_the_reference_tests(case):
    # utests/algorithm/image_processing/utest_color_conversion.h:299-348, through the C ABI
    wl, want = read_uyvy_kat_workload(case)
    assert np.array_equal(gpu_run(wl)[0][:want.size], want)


@pytest.mark.parametrize("rng", [abi.RANGE_LIMITED, abi.RANGE_FULL])
@pytest.mark.parametrize("prim", [abi.PRIMITIVES_BT601, abi.PRIMITIVES_BT709, abi.PRIMITIVES_BT2020])
def test_rgb_ycbcr_round_trip_property(rng, prim):
    # utests/algorithm/image_processing/utest_color_conversion.h:683-735, through the C ABI: back within 1 % of full scale,
    # and the same bytes as the oracle's round trip
    err = ycbcr_round_trip(gpu_run, rng, prim)
    assert err <= 255 * 0.01
    assert err == ycbcr_round_trip(oracle.run_oracle, rng, prim)


@pytest.mark.parametrize("name", sorted(SMALL))
@pytest.mark.parametrize("path", ["staged", "gather", "plan"])
def test_configurations_small(name, path):
    check(SMALL[name](), use_plan=(path == "plan"), force_gather=(path == "gather"))


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_fixtures(name):
    # fixtures were written by the reference CPU backend itself (tests/golden/make_golden.py)
    wl, want = load_golden(name)
    assert_same(wl, gpu_run(wl, fill=0), want)


@pytest.mark.parametrize("seed", range(120))
def test_random_launches(seed):
    wl = W.random_workload(seed)
    check(wl)
    if seed % 4 == 0:
        check(wl, force_gather=True)


@pytest.mark.parametrize("base", range(0, 60, 3))
def test_random_divergent_launches(base):
    # three random chains in one divergent launch, with uneven numbers of planes: the lowering deals the planes chain by
    # chain in turn, every plane must still land where its descriptor says
    wl = W.combine([W.random_workload(base + i) for i in range(3)])
    check(wl)
    check(wl, force_gather=True)
    check(wl, use_plan=True)


def test_tiny_launch_routing():
    # default behaviour: launches of fewer than 100 000 output pixels run through the general kernel
    for wl in [W.readme_crops(), W.vertical_fusion(w=200, h=100), W.divergent_planes(n_per_seq=1, w=128, h=72)]:
        check(wl, tiny_route=True)
        check(wl, tiny_route=True, use_plan=True)


def test_one_thin_crop_does_not_add_a_kernel_to_a_batch():
    # A crop whose letterboxed image has no column is all background.  It must stay in the batch's one fused launch: sent
    # to the general kernel, a single such plane once cost a 2048-plane launch more than its other 2047 planes together.
    from fusedkernellibrary_b200 import runtime
    rs = np.random.RandomState(5)
    rects = W.random_rects(63, 640, 480, 16, 300, rs) + [(100, 0, 1, 470)]  # round(224 / 470 * 1) = 0 columns
    wl = W.readme_crops(w=640, h=480, crops=tuple(rects), dst=(224, 224))
    os.environ["FKB_TINY_PIXELS"] = "0"
    try:
        dw = runtime.DeviceWorkload(wl)
        try:
            assert dw.kernel_launches() == 1
        finally:
            dw.close()
    finally:
        os.environ.pop("FKB_TINY_PIXELS", None)
    check(wl)
    check(wl, use_plan=True)


def test_edge_shapes():
    # 1x1 image, single-row / single-column images, crops touching every frame edge, extreme up- and down-scaling
    for wl in [
        W.vertical_fusion(w=1, h=1), W.vertical_fusion(w=1, h=40), W.vertical_fusion(w=47, h=1), W.vertical_fusion(w=16, h=16),
        W.readme_crops(w=64, h=48, crops=((0, 0, 1, 1), (63, 47, 1, 1), (0, 0, 64, 48), (0, 47, 64, 1), (63, 0, 1, 48)), dst=(32, 16)),
        W.readme_crops(w=640, h=480, crops=((0, 0, 640, 480), (3, 3, 634, 470)), dst=(16, 16)),     # 40x decimation
        W.readme_crops(w=64, h=48, crops=((5, 5, 2, 2), (1, 1, 3, 2)), dst=(640, 400)),             # 200x magnification
        W.readme_crops(w=640, h=480, crops=((100, 100, 58, 3),), dst=(1, 105)),                     # target rounds to zero height
        W.nv12_preprocess(w=2, h=2, dst=(5, 3)), W.nv12_preprocess(w=64, h=48, dst=(1, 1)),
        W.batched_crop_resize(n_frames=1, crops_per_frame=1, w=32, h=32, crop_range=(32, 32), dst=(224, 224)),
        # large source coordinates and scale factors in the thousands (tap positions are computed without conversions)
        W.readme_crops(w=16000, h=8, crops=((0, 0, 16000, 8), (1, 0, 15999, 7)), dst=(7, 3)),
        W.rgba_crops(w=4096, h=8, dst=(5, 3), rects=((0, 0, 4096, 8), (3, 1, 4001, 5))),
        W.nv12_preprocess(w=4096, h=16, dst=(3, 2)),
    ]:
        check(wl)
        check(wl, force_gather=True)


def test_nv12_colour_matrices():
    # limited-range bt601 (luma offset 16: the two-pixel kernel with a non-zero luma offset), then two matrices outside
    # that kernel's conditions (a Cb term in the red row; a fractional offset), which take the one-pixel NV12 kernel
    bt601_limited = (1.0, 0.0, 1.402, 1.0, -0.344136, -0.714136, 1.0, 1.772, 0.0)
    odd = (1.164, 0.25, 1.596, 1.164, -0.392, -0.813, 1.164, 2.017, 0.125)
    for kw in [dict(ccm=bt601_limited, yuv_sub=(16.0, 128.0, 128.0)), dict(ccm=odd, yuv_sub=(16.0, 128.0, 128.0)),
               dict(yuv_sub=(0.0, 127.5, 128.0))]:
        for shape in [dict(w=1280, h=720, dst=(321, 203)), dict(w=64, h=48, dst=(7, 5)), dict(w=66, h=50, dst=(300, 301))]:
            wl = W.nv12_preprocess(**shape, **kw)
            check(wl)
            check(wl, use_plan=True)


@pytest.mark.parametrize("fmt", [abi.PIX_NV12, abi.PIX_NV21, abi.PIX_UYVY])
@pytest.mark.parametrize("rng", [abi.RANGE_LIMITED, abi.RANGE_FULL])
@pytest.mark.parametrize("prim", [abi.PRIMITIVES_BT601, abi.PRIMITIVES_BT709, abi.PRIMITIVES_BT2020])
def test_yuv_formats_ranges_primitives(fmt, rng, prim):
    for shape in [dict(w=1280, h=720, dst=(321, 203)), dict(w=66, h=50, dst=(300, 301))]:
        wl = W.nv12_preprocess(**shape, src_format=fmt, colour=(rng, prim))
        check(wl)
        check(wl, force_gather=True)


@pytest.mark.parametrize("fmt", [abi.PIX_P010, abi.PIX_P210, abi.PIX_Y210])
@pytest.mark.parametrize("rng", [abi.RANGE_LIMITED, abi.RANGE_FULL])
@pytest.mark.parametrize("prim", [abi.PRIMITIVES_BT601, abi.PRIMITIVES_BT709, abi.PRIMITIVES_BT2020])
def test_ten_bit_yuv_formats(fmt, rng, prim):
    # ushort samples; odd sizes make the last chroma pair and the last chroma row serve one pixel only
    for shape in [dict(w=1280, h=720, dst=(321, 203)), dict(w=66, h=50, dst=(300, 301)), dict(w=130, h=46, dst=(33, 17), pitch_align=64)]:
        wl = W.nv12_preprocess(**shape, src_format=fmt, colour=(rng, prim))
        check(wl)
        check(wl, use_plan=True)
        check(wl, force_gather=True)


@pytest.mark.parametrize("mode", [abi.BORDER_CONSTANT, abi.BORDER_REPLICATE, abi.BORDER_REFLECT, abi.BORDER_WRAP, abi.BORDER_REFLECT_101])
def test_border_reader_modes(mode):
    for kw in [dict(), dict(w=37, h=23), dict(w=640, h=360, dst=(224, 224))]:
        wl = W.border_crops(mode, **kw)
        check(wl)
        check(wl, use_plan=True)


def test_border_constant_after_colour_conversion():
    check(W.nv12_border_constant())
    check(W.nv12_border_constant(w=640, h=360, rect=(500, 300, 400, 200), dst=(320, 320)))


@pytest.mark.parametrize("fmt", [abi.PIX_NV12, abi.PIX_NV21, abi.PIX_UYVY])
def test_write_yuv_images(fmt):
    for colour in [(abi.RANGE_FULL, abi.PRIMITIVES_BT709), (abi.RANGE_LIMITED, abi.PRIMITIVES_BT601)]:
        # (from 131 072 pixels on, a thread writes four pixels with word stores; odd widths and heights leave ragged ends)
        for size in [dict(w=322, h=180), dict(w=64, h=36), dict(w=1280, h=720), dict(w=33, h=21), dict(w=1002, h=563), dict(w=999, h=400)]:
            check(W.rgb_to_yuv_image(fmt, colour, **size))


def test_plan_relaunches_leave_the_item_counters_clean():
    # a launch with more items than resident warps claims its items from a counter pair that the kernel resets itself:
    # repeated launches of one plan (and of the same descriptors through the arena) must each produce the full output
    from fusedkernellibrary_b200 import runtime
    wl = W.batched_crop_resize(n_frames=4, crops_per_frame=32, w=640, h=360, dst=(224, 224), crop_range=(8, 300))
    want = oracle.run_oracle(wl, threads=8, fill=FILL)
    dw = runtime.DeviceWorkload(wl, poison=FILL)
    dw.plan()
    for _ in range(5):
        for t in dw.out:
            t.fill_(FILL)
        dw.launch_plan()
        assert_same(wl, dw.results(), want)
    for _ in range(6):
        for t in dw.out:
            t.fill_(FILL)
        dw.launch()
        assert_same(wl, dw.results(), want)
    dw.close()


@pytest.mark.parametrize("kind", [0, 1, 2])
@pytest.mark.parametrize("oldest_first", [0, 1])
def test_circular_tensor_updates(kind, oldest_first):
    # nine updates of a four-plane circular tensor, each one divergent launch (update sequence + copy sequence reading float
    # planes), device against the CPU checker after every update
    lib, orc = abi.load(), oracle.load_oracle()
    w, h, dw, dh, batch = 320, 180, 96, 64, 4
    pitch = w * 3
    frames = [np.random.RandomState(70 + k).randint(0, 256, pitch * h, dtype=np.uint8) for k in range(9)]
    mul = (0.5, 1.0, 2.0)
    size = batch * dw * dh * 12
    h_temp, h_out = np.zeros(size, np.uint8), np.zeros(size, np.uint8)
    d_temp, d_out = torch.zeros(size, dtype=torch.uint8, device="cuda"), torch.zeros(size, dtype=torch.uint8, device="cuda")
    d_frames = [torch.from_numpy(f).cuda() for f in frames]
    first_h = first_d = 0
    for k in range(9):
        ch, pl, first_h = W.circular_update_launch(kind, oldest_first, first_h, batch, frames[k].ctypes.data, w, h, pitch, dw, dh, mul,
                                                   h_temp.ctypes.data, h_out.ctypes.data)
        assert orc.fkb_oracle_run(ch, 2, pl, len(pl), 1) == 0
        ch, pl, first_d = W.circular_update_launch(kind, oldest_first, first_d, batch, d_frames[k].data_ptr(), w, h, pitch, dw, dh, mul,
                                                   d_temp.data_ptr(), d_out.data_ptr())
        assert lib.fkb_launch_divergent(ch, 2, pl, len(pl), torch.cuda.current_stream().cuda_stream) == abi.OK
        torch.cuda.synchronize()
        assert np.array_equal(d_out.cpu().numpy(), h_out) and np.array_equal(d_temp.cpu().numpy(), h_temp), (kind, oldest_first, k)
    assert lib.fkb_device_status() == abi.OK


def test_many_planes_use_the_descriptor_arena():
    # more planes than fit in the kernel parameters: descriptors travel through the pinned/device ring
    wl = W.batched_crop_resize(n_frames=3, crops_per_frame=100, w=320, h=240, dst=(32, 24), crop_range=(4, 100))
    check(wl)
    for _ in range(6):  # wrap the ring
        check(wl)


def test_more_planes_than_a_grid_dimension_holds():
    # 70 000 planes in one launch (gridDim.z ends at 65 535): the pipelined kernel finds a plane by searching the table,
    # the general kernel walks the planes in strides of its grid
    wl = W.batched_crop_resize(n_frames=7, crops_per_frame=10000, w=320, h=240, dst=(4, 3), crop_range=(2, 40))
    assert len(wl.planes) == 70000
    check(wl)
    check(wl, force_gather=True)


@pytest.mark.parametrize("dst", [(32, 1), (40, 2), (33, 3)])
def test_thousands_of_planes_of_one_to_three_rows(dst):
    # items of one, two and three rows, claimed from the counter; the last ones are dealt as two halves, and the second
    # half of a one-row item is empty
    wl = W.batched_crop_resize(n_frames=6, crops_per_frame=1000, w=320, h=240, dst=dst, crop_range=(2, 60))
    check(wl)
    check(wl, use_plan=True)


@pytest.mark.parametrize("frames,crops,dst", [(3, 70, (100, 37)), (5, 64, (224, 224)), (9, 50, (57, 113)), (2, 400, (33, 21)),
                                              (16, 32, (224, 224)), (7, 33, (300, 41))])
def test_mid_size_batches_of_odd_shapes(frames, crops, dst):
    # launches of a few items per warp: items claimed from the counter, the last ones in halves, rows per item by size
    wl = W.batched_crop_resize(n_frames=frames, crops_per_frame=crops, w=640, h=360, dst=dst, crop_range=(2, 300))
    check(wl)
    check(wl, use_plan=True)


def test_back_to_back_launches_on_side_streams():
    from fusedkernellibrary_b200 import runtime
    wls = [W.batched_crop_resize(n_frames=2, crops_per_frame=20, w=320, h=240, dst=(64, 64), seed=s) for s in range(3)]
    dws = [runtime.DeviceWorkload(w, poison=FILL) for w in wls]
    streams = [torch.cuda.Stream() for _ in dws]
    for _ in range(3):
        for dw, st in zip(dws, streams):
            with torch.cuda.stream(st):
                dw.launch()
    for wl, dw in zip(wls, dws):
        assert_same(wl, dw.results(), oracle.run_oracle(wl, fill=FILL))
        dw.close()


def test_device_status_is_clean_and_errors_are_codes():
    lib = abi.load()
    assert lib.fkb_device_status() == abi.OK
    wl = W.readme_crops()
    from fusedkernellibrary_b200 import runtime
    dw = runtime.DeviceWorkload(wl)
    dw.planes[0].crop_x = 5000  # rectangle outside the frame: refused on the host, nothing is launched
    assert lib.fkb_launch_transform(dw.chains, dw.planes, dw.n_planes, None) == abi.ERR_INVALID
    assert lib.fkb_device_status() == abi.OK


# ---------------------------------------------------------------------------------------------------------------
# full benchmark sizes: direct comparison where the oracle is fast, size-independent properties for the largest
# ---------------------------------------------------------------------------------------------------------------
def test_full_vertical_fusion():
    check(W.vertical_fusion())


def test_full_nv12():
    check(W.nv12_preprocess())


def test_full_divergent_properties():
    from fusedkernellibrary_b200 import runtime
    wl = W.divergent_planes()
    dw = runtime.DeviceWorkload(wl, poison=FILL)
    dw.launch()
    outA, outB = dw.results()
    dw.close()
    n, w, h = 4, 3840, 2160
    # planes 0..3: scale is exactly 2, so three bilinear weights are exactly 0 and the output is the even-pixel
    # subsample of the source (then an exact saturate cast)
    for i in range(n):
        src = wl.sources[i].reshape(h, w, 3)
        assert np.array_equal(outA[i * (w // 2) * (h // 2) * 3:(i + 1) * (w // 2) * (h // 2) * 3].reshape(h // 2, w // 2, 3), src[::2, ::2])
    # planes 4..7: x*scale - off in fp32, two roundings; planes 0..3 of the float tensor stay untouched
    f = outB.view(np.float32).reshape(2 * n, h, w, 3)
    assert np.all(outB[: n * w * h * 12] == FILL)
    for i in range(n):
        src = wl.sources[n + i].reshape(h, w, 3).astype(np.float32)
        want = src * np.float32(wl.extra["scales"][i]) - np.float32(wl.extra["offs"][i])
        assert np.array_equal(f[n + i], want)


def test_full_batched_crop_resize_properties():
    """64 frames x 32 crops -> 224x224x2048 float3 (1.2 GB): compared exactly against the oracle on a sample of planes,
    and over the whole tensor through properties that do not depend on the size."""
    from fusedkernellibrary_b200 import runtime
    wl = W.batched_crop_resize()
    dw = runtime.DeviceWorkload(wl, poison=None)
    dw.launch()
    torch.cuda.synchronize()
    assert abi.load().fkb_device_status() == abi.OK
    out = dw.out[0].view(torch.float32).view(2048, 224, 224, 3)
    # (1) range: inputs are 0..255, weights sum to 1 up to rounding, times 1/255
    assert float(out.min()) >= 0.0 and float(out.max()) <= 1.0 + 1e-6
    # (2) letterbox: everything outside each plane's target rectangle equals fp32(114 * fp32(1/255)) exactly
    bgv = np.float32(114.0) * np.float32(1.0 / 255.0)
    planes = dw.planes
    idx = list(range(0, 2048, 97)) + [2047]
    host = out[idx].cpu().numpy()
    for k, z in enumerate(idx):
        d = planes[z]
        m = np.ones((224, 224), bool)
        m[d.y1:d.y2 + 1, d.x1:d.x2 + 1] = False
        assert np.all(host[k][m] == bgv)
    # (3) exact parity on the sampled planes: rerun just those planes through the oracle
    sub = W.Workload(wl.name, wl.chains, wl.sources, [len(idx) * 224 * 224 * 12],
                     [W.PlaneSpec(**{**wl.planes[z].__dict__, "dst_offset": k * 224 * 224 * 12}) for k, z in enumerate(idx)])
    want = oracle.run_oracle(sub, threads=8)[0].view(np.float32).reshape(len(idx), 224, 224, 3)
    assert np.array_equal(host.view(np.uint32), want.view(np.uint32))
    # (4) idempotence / determinism: a second launch (through a plan) reproduces the first bit for bit
    first = out.clone()
    dw.launch_plan()
    torch.cuda.synchronize()
    assert torch.equal(first.view(torch.int32), out.view(torch.int32))
    # (5) the staged path and the general path agree on the whole tensor
    os.environ["FKB_FORCE_GATHER"] = "1"
    try:
        dw.launch()
        torch.cuda.synchronize()
    finally:
        os.environ["FKB_FORCE_GATHER"] = "0"
    assert torch.equal(first.view(torch.int32), out.view(torch.int32))
    dw.close()


def test_bounded_wait_runs_out_is_reported_and_leaves_the_context_usable():
    """Every device-side wait for a bulk copy has a time limit.  Here the staged kernel's loads are made to announce 16
    bytes that nothing delivers (a host-side test switch: no fault is involved, the copies themselves are complete), so
    the wait runs out: the kernel must end by itself, fkb_device_status() must report FKB_ERR_DEVICE_WAIT once and then
    be clear again, and the next launch on the same context must be correct."""
    from fusedkernellibrary_b200 import runtime
    wl = SMALL["batched"]()
    lib = abi.load()
    torch.cuda.synchronize()
    assert lib.fkb_device_status() == abi.OK
    os.environ.update(FKB_TEST_EXTRA_TX="16", FKB_WAIT_LIMIT_US="2000", FKB_TINY_PIXELS="0")
    try:
        dw = runtime.DeviceWorkload(wl, poison=FILL)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        dw.launch()
        stop.record()
        torch.cuda.synchronize()  # returns: the kernel gave up on its own
        assert start.elapsed_time(stop) < 2000.0  # a few waits of 2 ms each, not an endless one
    finally:
        for k in ("FKB_TEST_EXTRA_TX", "FKB_WAIT_LIMIT_US", "FKB_TINY_PIXELS"):
            os.environ.pop(k, None)
    assert lib.fkb_device_status() == abi.ERR_DEVICE_WAIT
    assert b"wait" in lib.fkb_status_string(abi.ERR_DEVICE_WAIT)
    assert lib.fkb_device_status() == abi.OK  # reading the status cleared it
    dw.close()
    check(wl)  # the same launch without the switch: correct, on the same context


def test_launches_of_one_plan_may_overlap_on_two_streams():
    """fkb_plan_launch gives every launch its own pair of work counters, so launches of one plan on different streams may
    run at the same time: the result is that of a single launch, and later launches of the plan still are."""
    from fusedkernellibrary_b200 import runtime
    wl = W.batched_crop_resize(n_frames=8)  # 256 planes: enough items for the kernel to claim them from a counter
    dw = runtime.DeviceWorkload(wl, poison=FILL)
    dw.launch()  # reference result through the one-shot entry point
    want = dw.results()[0].copy()
    dw.out[0].fill_(FILL)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    for _ in range(6):
        with torch.cuda.stream(s1):
            dw.launch_plan()
        with torch.cuda.stream(s2):
            dw.launch_plan()
    torch.cuda.synchronize()
    assert np.array_equal(dw.results()[0], want)
    dw.out[0].fill_(FILL)
    dw.launch_plan()
    assert np.array_equal(dw.results()[0], want)
    dw.close()


def test_a_launch_consumes_the_output_of_the_launch_before_it():
    """Launches of this size are submitted with programmatic stream serialisation allowed, so a kernel may be set up while
    the kernel before it in the stream still runs; it must not read anything before that kernel has completed.  A chain of
    three launches in one stream, each reading what the one before wrote (table-lookup kernel -> table-lookup kernel ->
    crop-resize kernel), run back to back and from a CUDA graph while the first launch's source alternates between two
    images, must give what the oracle gives for the image of the last round."""
    import dataclasses
    from fusedkernellibrary_b200 import runtime
    w, h = 1280, 720
    first = W.vertical_fusion(w=w, h=h, seed=31)
    other = W.vertical_fusion(w=w, h=h, seed=32)
    second = W.vertical_fusion(w=w, h=h, seed=33)   # its source buffer is replaced by the first launch's output
    third = W.readme_crops(w=w, h=h, crops=tuple((40 * i, 20 * i, 300 + 50 * i, 200 + 30 * i) for i in range(8)), dst=(224, 224))
    assert first.out_sizes[0] == second.sources[0].nbytes == third.sources[0].nbytes
    want = {}
    for name, wl in (("a", first), ("b", other)):
        out1 = oracle.run_oracle(wl, threads=8, fill=FILL)[0]
        out2 = oracle.run_oracle(dataclasses.replace(second, sources=[out1]), threads=8, fill=FILL)[0]
        want[name] = oracle.run_oracle(dataclasses.replace(third, sources=[out2]), threads=8, fill=FILL)[0]
    d1, d2, d3 = (runtime.DeviceWorkload(x, poison=FILL) for x in (first, second, third))
    d2.planes = second.bind([d1.out[0].data_ptr()], [t.data_ptr() for t in d2.out])
    d3.planes = third.bind([d2.out[0].data_ptr()], [t.data_ptr() for t in d3.out])
    images = {"a": d1.src[0].clone(), "b": torch.from_numpy(other.sources[0]).cuda()}

    def round_of(name):
        d1.src[0].copy_(images[name], non_blocking=True)
        for d in (d1, d2, d3):
            d.launch_plan()

    for name in "abababab":
        round_of(name)
    assert np.array_equal(d3.results()[0], want["b"])
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for name in "babababa":
                round_of(name)
    for _ in range(3):
        graph.replay()
    assert np.array_equal(d3.results()[0], want["a"])
    # and without a copy between the rounds: kernel follows kernel all the way (one-shot launches of at most 8 planes too)
    for _ in range(4):
        for d in (d1, d2, d3):
            d.launch()
    assert np.array_equal(d3.results()[0], want["a"])
    for d in (d1, d2, d3):
        d.close()


def test_stream_capture_small_launches_record_large_one_shot_launches_refuse():
    """A launch of at most eight planes carries its records in the kernel parameters and records into a CUDA graph; a
    larger one-shot launch (and the no-allocation entry point) stages records through host memory the library reuses, so
    on a capturing stream it returns FKB_ERR_UNSUPPORTED and records nothing — the capture itself stays valid."""
    from fusedkernellibrary_b200 import runtime
    lib = abi.load()
    big = runtime.DeviceWorkload(W.batched_crop_resize(n_frames=3, crops_per_frame=100, w=320, h=240, dst=(32, 24), crop_range=(4, 100)), poison=FILL)
    small = runtime.DeviceWorkload(W.readme_crops(), poison=FILL)
    big.launch()
    small.launch()  # warm: kernels are loaded and per-device look-ups are cached before the capture begins
    abi.check(lib.fkb_launch_transform_noalloc(big.chains, big.planes, big.n_planes, runtime.current_stream_ptr()))
    want = small.results()[0].copy()
    small.out[0].fill_(FILL)
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            rc_big = lib.fkb_launch_transform(big.chains, big.planes, big.n_planes, side.cuda_stream)
            rc_noalloc = lib.fkb_launch_transform_noalloc(big.chains, big.planes, big.n_planes, side.cuda_stream)
            rc_small = lib.fkb_launch_transform(small.chains, small.planes, small.n_planes, side.cuda_stream)
    assert rc_big == abi.ERR_UNSUPPORTED and rc_noalloc == abi.ERR_UNSUPPORTED and rc_small == abi.OK
    graph.replay()
    assert np.array_equal(small.results()[0], want)
    big.close()
    small.close()


def test_self_checking_build_finds_nothing_on_the_parity_cases():
    """libfkb_debug.so is the same library compiled with -DFKB_DEBUG: every bulk copy and every gathered tap is tested
    against the buffer its plane record describes before the access, a miss is recorded as FKB_ERR_DEVICE_CHECK and the
    access skipped (no trap).  It stands in for a memory checker.  The small configurations on all three paths, the golden
    fixtures and the random launches are run on it in a fresh process: results equal the oracle's and the status word
    stays clear (every one of those tests reads it)."""
    import subprocess
    import sys
    from fusedkernellibrary_b200 import build as fkb_build
    from conftest import ROOT
    lib = fkb_build.build_debug()
    env = dict(os.environ, FKB_LIBRARY=lib)
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_parity.py"), "-m", "gpu", "-x", "-q",
                        "-k", "configurations_small or golden_fixtures or random_launches or random_divergent or edge_shapes or border_reader_modes"],
                       capture_output=True, text=True, timeout=1200, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


def test_without_programmatic_stream_serialisation():
    """FKB_PDL=0 (read once per process) launches every kernel without the attribute: the small configurations, the
    chain of dependent launches and the launches on two streams give the same results in a fresh process."""
    import subprocess
    import sys
    from conftest import ROOT
    env = dict(os.environ, FKB_PDL="0")
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_parity.py"), "-m", "gpu", "-x", "-q",
                        "-k", "configurations_small or consumes_the_output or overlap_on_two_streams"],
                       capture_output=True, text=True, timeout=1200, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


SHRUNK_FRAME = '''
import os, sys
sys.path.insert(0, sys.argv[1])
import torch
from fusedkernellibrary_b200 import abi, runtime, workloads as W
wl = W.batched_crop_resize(n_frames=4, crops_per_frame=8, w=960, h=540)
lib = abi.load()
os.environ["FKB_TEST_SHRINK_FRAME"] = "1"
dw = runtime.DeviceWorkload(wl, poison=0xCD)
dw.launch()
torch.cuda.synchronize()
first = lib.fkb_device_status()
os.environ.pop("FKB_TEST_SHRINK_FRAME")
dw.launch()
torch.cuda.synchronize()
print("STATUS", first, lib.fkb_device_status())
'''


def test_self_checking_build_reports_a_copy_outside_its_frame(tmp_path):
    """The checker of the self-checking build has to fire when something is wrong: with plane records that claim source
    frames of a single row (a host-side test switch), its range tests fail for every source row below the first, the
    copies are skipped — nothing is read out of range, nothing traps — and fkb_device_status() reports
    FKB_ERR_DEVICE_CHECK once; the same launch without the switch is clean again."""
    import subprocess
    import sys
    from fusedkernellibrary_b200 import build as fkb_build
    from conftest import ROOT
    script = tmp_path / "shrunk_frame.py"
    script.write_text(SHRUNK_FRAME)
    env = dict(os.environ, FKB_LIBRARY=fkb_build.build_debug(), FKB_TINY_PIXELS="0")
    r = subprocess.run([sys.executable, str(script), ROOT], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    fields = [l for l in r.stdout.splitlines() if l.startswith("STATUS ")][0].split()
    assert int(fields[1]) == abi.ERR_DEVICE_CHECK and int(fields[2]) == abi.OK
