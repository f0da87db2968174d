"""CPU tests of the oracle: golden values from the reference's own unit tests, the committed fixtures produced by
the reference CPU backend, and (where the reference-backed checker was built) a direct comparison with it."""
import ctypes as C
import math

import numpy as np
import pytest

import oracle
from conftest import GOLDEN_CASES, conversion_kat_workload, ycbcr_round_trip, load_golden, read_uyvy_kat_workload, reference_kats
from fusedkernellibrary_b200 import abi, workloads as W


def test_saturate_cast_golden_values():
    # utests/algorithm/image_processing/utest_saturate/utest_saturate_common.h:60-75 (0.5->0, 1.5->2, 2.5->2, ties to
    # even), clamping at both ends, and NaN -> 0 (core/constexpr_libs/constexpr_saturate.h:97-100)
    sat = oracle.load_oracle().fkb_oracle_saturate_u8
    table = [(0.5, 0), (1.5, 2), (2.5, 2), (3.5, 4), (0.49999997, 0), (0.50000006, 1), (-1.5, 0), (-0.5, 0), (254.5, 254),
             (254.50002, 255), (255.0, 255), (255.5, 255), (1e9, 255), (-1e9, 0), (127.4, 127), (127.6, 128),
             (float("nan"), 0), (float("inf"), 255), (float("-inf"), 0)]
    for v, want in table:
        assert sat(v) == want, (v, want)
    if oracle.have_ref():
        ref = oracle.load_ref().fklref_saturate_u8
        rs = np.random.RandomState(0)
        vals = np.concatenate([rs.uniform(-20, 280, 20000), np.arange(-4, 260) + 0.5, np.arange(-4, 260)]).astype(np.float32)
        for v in vals:
            assert sat(float(v)) == ref(float(v)), v


def test_round_half_away_matches_std_round():
    f = oracle.load_oracle().fkb_oracle_round_half_away
    for v in [0.5, 1.5, 2.5, -0.5, -2.5, 0.49999997, 95.99999, 96.0, 58.5, 59.499996, 0.0]:
        want = math.copysign(math.floor(abs(np.float32(v)) + 0.5), v) if v != 0.49999997 else 0.0
        assert f(v) == want, v


def test_reorder_golden():
    # utests/algorithm/image_processing/utest_color_conversion.h:91-101: {100,150,200} -> {200,150,100}
    src = np.array([100, 150, 200] + [0] * 13, np.uint8)
    ch = W.chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C3, abi.WRITE_PACKED, [W.op(abi.OP_REORDER_ZYX)])
    wl = W.Workload("x", [ch], [src], [3], [W.PlaneSpec(0, 0, 0, 1, 1, 16, (0, 0, 1, 1), 1, 1, 3)])
    assert oracle.run_oracle(wl)[0].tolist() == [200, 150, 100]


def test_bt709_matrix_golden():
    # constants of utests/algorithm/image_processing/utest_color_conversion.h:441-447 (bt709, Full, 8 bit)
    want = np.array([1.0, 0.0, 1.57480001, 1.0, -0.187324256, -0.46812427, 1.0, 1.8556, 0.0], np.float32)
    assert np.array_equal(np.array(W.BT709_FULL_8BIT, np.float32), want)
    if oracle.have_ref():
        m = (C.c_float * 9)()
        oracle.load_ref().fklref_bt709_full_matrix(m)
        assert np.array_equal(np.array(list(m), np.float32), want)


RANGES = {"limited": abi.RANGE_LIMITED, "full": abi.RANGE_FULL}
PRIMS = {"bt601": abi.PRIMITIVES_BT601, "bt709": abi.PRIMITIVES_BT709, "bt2020": abi.PRIMITIVES_BT2020}


def test_colour_matrices_equal_the_reference_tests_constants():
    # the twelve 8-bit matrices the reference's unit test compares with == against ccMatrix
    # (utests/algorithm/image_processing/utest_color_conversion.h:407-509, 576-597): the oracle's and the library's
    # host functions must produce the same floats
    lib, prod = oracle.load_oracle(), abi.load()
    for key, vals in reference_kats()["matrices"].items():
        rng, prim, direction = key.split("/")
        want = np.array(vals, np.float32)
        got_o, got_p, off = (C.c_float * 9)(), (C.c_float * 9)(), (C.c_float * 3)()
        if direction == "ycbcr2rgb":
            assert lib.fkb_oracle_ycbcr_to_rgb(RANGES[rng], PRIMS[prim], got_o, off) == 0
            assert prod.fkb_ycbcr_to_rgb(RANGES[rng], PRIMS[prim], got_p, off) == 0
        else:
            assert lib.fkb_oracle_rgb_to_ycbcr(RANGES[rng], PRIMS[prim], got_o, off) == 0
            assert prod.fkb_rgb_to_ycbcr(RANGES[rng], PRIMS[prim], got_p, off) == 0
        assert np.array_equal(np.array(list(got_o), np.float32), want), key
        assert np.array_equal(np.array(list(got_p), np.float32), want), key


@pytest.mark.parametrize("case", reference_kats()["conversions"], ids=lambda c: c["code"])
def test_colour_conversion_known_answers(case):
    # utests/algorithm/image_processing/utest_color_conversion.h:76-101, 144-168
    wl, want = conversion_kat_workload(case)
    assert np.array_equal(oracle.run_oracle(wl)[0], want)


@pytest.mark.parametrize("case", reference_kats()["read_uyvy"], ids=lambda c: f"{c['w']}x{c['h']}")
def test_read_uyvy_known_answers(case):
    # utests/algorithm/image_processing/utest_color_conversion.h:299-348: every pixel of three small UYVY images
    wl, want = read_uyvy_kat_workload(case)
    assert np.array_equal(oracle.run_oracle(wl)[0], want)


@pytest.mark.parametrize("rng", sorted(RANGES))
@pytest.mark.parametrize("prim", sorted(PRIMS))
def test_rgb_ycbcr_round_trip_property(rng, prim):
    # utests/algorithm/image_processing/utest_color_conversion.h:683-735: back within 1 % of full scale
    assert ycbcr_round_trip(oracle.run_oracle, RANGES[rng], PRIMS[prim]) <= 255 * 0.01


# letterbox placement and scale factors the reference computes for the README crops (Resize<>::build run in the
# reference: resize.h:164-233): crop -> (target w, target h, x1, y1, fx, fy)
README_KNOWN = [
    ((60, 40), (96, 64, 16, 0, 0.625, 0.625)),
    ((130, 140), (59, 64, 34, 0, 2.20338988, 2.1875)),
    ((100, 35), (128, 45, 0, 9, 0.78125, 0.777777791)),
    ((40, 15), (128, 48, 0, 8, 0.3125, 0.3125)),
]


def test_resize_params_known_answers():
    lib = oracle.load_oracle()
    for (cw, chh), (tw, th, x1, y1, fx, fy) in README_KNOWN:
        d = abi.PlaneDesc()
        d.crop_w, d.crop_h, d.dst_w, d.dst_h = cw, chh, 128, 64
        assert lib.fkb_oracle_resize_params(abi.GEOM_RESIZE_PRESERVE_AR, C.byref(d)) == 0
        assert (d.x2 - d.x1 + 1, d.y2 - d.y1 + 1, d.x1, d.y1) == (tw, th, x1, y1)
        assert np.float32(d.fx) == np.float32(fx) and np.float32(d.fy) == np.float32(fy)
    d = abi.PlaneDesc()
    d.crop_w, d.crop_h, d.dst_w, d.dst_h = 3840, 2160, 640, 640
    assert lib.fkb_oracle_resize_params(abi.GEOM_RESIZE_IGNORE_AR, C.byref(d)) == 0
    assert (d.fx, d.fy) == (6.0, 3.375)


@pytest.mark.skipif(not oracle.have_ref(), reason="reference-backed checker not built")
def test_resize_params_against_reference():
    lib, ref = oracle.load_oracle(), oracle.load_ref()
    rs = np.random.RandomState(1)
    for _ in range(3000):
        sw, sh, dw, dh = (int(v) for v in rs.randint(1, 700, 4))
        # the reference's AspectRatio value -> this library's geometry code
        for ar, geom in ((0, abi.GEOM_RESIZE_PRESERVE_AR), (1, abi.GEOM_RESIZE_IGNORE_AR),
                         (2, abi.GEOM_RESIZE_PRESERVE_AR_RN_EVEN), (3, abi.GEOM_RESIZE_PRESERVE_AR_LEFT)):
            f2, r4 = (C.c_float * 2)(), (C.c_int32 * 4)()
            ref.fklref_resize_params(sw, sh, dw, dh, ar, f2, r4)
            d = abi.PlaneDesc()
            d.crop_w, d.crop_h, d.dst_w, d.dst_h = sw, sh, dw, dh
            lib.fkb_oracle_resize_params(geom, C.byref(d))
            got = (d.fx, d.fy, d.x1, d.y1, d.x2, d.y2)
            want = (f2[0], f2[1], r4[0], r4[1], r4[2], r4[3])
            # a target that rounds to zero divides by zero in both (inf, or nan for 0/0): compare those by class
            assert all(g == w or (np.isnan(g) and np.isnan(w)) for g, w in zip(got, want)), (sw, sh, dw, dh, ar, got, want)


@pytest.mark.skipif(not oracle.have_ref(), reason="reference-backed checker not built")
def test_ycbcr_matrices_against_reference():
    lib, ref = oracle.load_oracle(), oracle.load_ref()
    for rng in (abi.RANGE_LIMITED, abi.RANGE_FULL):
        for prim in (abi.PRIMITIVES_BT601, abi.PRIMITIVES_BT709, abi.PRIMITIVES_BT2020):
            want, got, sub = (C.c_float * 9)(), (C.c_float * 9)(), (C.c_float * 3)()
            assert ref.fklref_ycbcr_matrix(rng, prim, want) == 0
            assert lib.fkb_oracle_ycbcr_to_rgb(rng, prim, got, sub) == 0
            assert list(got) == list(want), (rng, prim)  # bit for bit
            assert list(sub) == [16.0 if rng == abi.RANGE_LIMITED else 0.0, 128.0, 128.0]
            want10, got10, sub10, refsub = (C.c_float * 9)(), (C.c_float * 9)(), (C.c_float * 3)(), (C.c_float * 2)()
            assert ref.fklref_ycbcr_matrix10(rng, prim, want10, refsub) == 0       # ten-bit samples
            assert lib.fkb_oracle_ycbcr_to_rgb_bits(10, rng, prim, got10, sub10) == 0
            assert list(got10) == list(want10), (rng, prim)
            assert list(sub10) == [refsub[0] if rng == abi.RANGE_LIMITED else 0.0, refsub[1], refsub[1]]
    assert lib.fkb_oracle_ycbcr_to_rgb_bits(9, 0, 0, got, sub) != 0


@pytest.mark.skipif(not oracle.have_ref(), reason="reference-backed checker not built")
def test_rgb_to_ycbcr_matrices_against_reference():
    lib, ref = oracle.load_oracle(), oracle.load_ref()
    for rng in (abi.RANGE_LIMITED, abi.RANGE_FULL):
        for prim in (abi.PRIMITIVES_BT601, abi.PRIMITIVES_BT709, abi.PRIMITIVES_BT2020):
            want, got, add = (C.c_float * 9)(), (C.c_float * 9)(), (C.c_float * 3)()
            assert ref.fklref_rgb_to_ycbcr_matrix(rng, prim, want) == 0
            assert lib.fkb_oracle_rgb_to_ycbcr(rng, prim, got, add) == 0
            assert list(got) == list(want), (rng, prim)
            assert list(add) == [16.0 if rng == abi.RANGE_LIMITED else 0.0, 128.0, 128.0]


WRITE_YUV_CASES = [(abi.PIX_NV12, abi.RANGE_FULL, abi.PRIMITIVES_BT709), (abi.PIX_NV12, abi.RANGE_LIMITED, abi.PRIMITIVES_BT601),
                   (abi.PIX_NV21, abi.RANGE_LIMITED, abi.PRIMITIVES_BT2020), (abi.PIX_NV21, abi.RANGE_FULL, abi.PRIMITIVES_BT601),
                   (abi.PIX_UYVY, abi.RANGE_LIMITED, abi.PRIMITIVES_BT709), (abi.PIX_UYVY, abi.RANGE_FULL, abi.PRIMITIVES_BT2020)]


@pytest.mark.skipif(not oracle.have_ref(), reason="reference-backed checker not built")
@pytest.mark.parametrize("fmt,rng,prim", WRITE_YUV_CASES)
def test_oracle_write_yuv_matches_reference_backend(fmt, rng, prim):
    for size in [dict(w=322, h=180), dict(w=64, h=36)]:
        wl = W.rgb_to_yuv_image(fmt, (rng, prim), **size)
        got, want = oracle.run_oracle(wl), oracle.run_ref(wl)
        assert np.array_equal(got[0], want[0])


YUV_CASES = [(abi.PIX_NV12, abi.RANGE_FULL, abi.PRIMITIVES_BT709), (abi.PIX_NV12, abi.RANGE_LIMITED, abi.PRIMITIVES_BT601),
             (abi.PIX_NV12, abi.RANGE_LIMITED, abi.PRIMITIVES_BT2020), (abi.PIX_NV21, abi.RANGE_FULL, abi.PRIMITIVES_BT601),
             (abi.PIX_NV21, abi.RANGE_LIMITED, abi.PRIMITIVES_BT709), (abi.PIX_UYVY, abi.RANGE_FULL, abi.PRIMITIVES_BT2020),
             (abi.PIX_UYVY, abi.RANGE_LIMITED, abi.PRIMITIVES_BT601),
             (abi.PIX_P010, abi.RANGE_LIMITED, abi.PRIMITIVES_BT2020), (abi.PIX_P010, abi.RANGE_FULL, abi.PRIMITIVES_BT709),
             (abi.PIX_P210, abi.RANGE_LIMITED, abi.PRIMITIVES_BT709), (abi.PIX_P210, abi.RANGE_FULL, abi.PRIMITIVES_BT2020),
             (abi.PIX_Y210, abi.RANGE_LIMITED, abi.PRIMITIVES_BT2020), (abi.PIX_Y210, abi.RANGE_FULL, abi.PRIMITIVES_BT601)]


@pytest.mark.skipif(not oracle.have_ref(), reason="reference-backed checker not built")
@pytest.mark.parametrize("fmt,rng,prim", YUV_CASES)
def test_oracle_yuv_formats_match_reference_backend(fmt, rng, prim):
    wl = W.nv12_preprocess(w=640, h=360, dst=(200, 150), src_format=fmt, colour=(rng, prim))
    got, want = oracle.run_oracle(wl, threads=4), oracle.run_ref(wl)
    assert np.array_equal(got[0], want[0])


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_oracle_matches_golden_fixture(name):
    wl, want = load_golden(name)
    got = oracle.run_oracle(wl)
    for g, w in zip(got, want):
        assert np.array_equal(g, w)  # bit-exact, integer and float outputs alike


# crops so thin that the letterboxed image has no column (or no row): the whole plane is background
THIN_CROPS = ((300, 125, 1, 500), (400, 125, 500, 1), (10, 10, 2, 700), (530, 270, 130, 140), (0, 0, 1, 1))


@pytest.mark.skipif(not oracle.have_ref(), reason="reference-backed checker not built")
@pytest.mark.parametrize("wl", [
    W.readme_crops(), W.vertical_fusion(w=1000, h=300), W.nv12_preprocess(w=1280, h=720, dst=(320, 320)),
    W.batched_crop_resize(n_frames=4, crops_per_frame=8, w=960, h=540), W.divergent_planes(n_per_seq=4, w=480, h=270),
    W.divergent_planes(n_per_seq=1, w=200, h=100), W.crop_reorder(n=5),
    W.border_crops(abi.BORDER_CONSTANT), W.border_crops(abi.BORDER_REPLICATE), W.border_crops(abi.BORDER_REFLECT),
    W.border_crops(abi.BORDER_WRAP), W.border_crops(abi.BORDER_REFLECT_101), W.border_crops(abi.BORDER_WRAP, w=37, h=23),
    W.border_crops(abi.BORDER_REFLECT, w=37, h=23), W.border_crops(abi.BORDER_REFLECT_101, w=37, h=23), W.nv12_border_constant(),
    W.rgba_crops(), W.rgba_crops(reorder=True), W.rgba_crops(f32=True), W.rgba_crops(reorder=True, f32=True),
    W.readme_crops(crops=THIN_CROPS, dst=(224, 224)),
    W.add_alpha_crops(), W.add_alpha_crops(swap=True), W.add_alpha_crops(f32=True), W.add_alpha_crops(swap=True, f32=True),
    W.add_alpha_image(), W.add_alpha_image(swap=True),
    W.gray_image(), W.gray_image(bgr=True), W.gray_image(src4=True), W.gray_image(bgr=True, src4=True, w=1001, h=37),
    W.gray_crops(), W.gray_crops(bgr=True), W.gray_crops(f32=True), W.gray_crops(bgr=True, f32=True, w=333, h=211, dst=(77, 45), rects=((0, 0, 333, 211), (5, 7, 100, 60), (200, 100, 50, 111), (300, 200, 33, 11), (100, 50, 20, 20))),
    W.bgra_crops(), W.bgra_crops(swap=True), W.split_planes(), W.split_planes(f32=False), W.tsplit_resize(), W.conditional_resize(), W.conditional_resize(used=0), W.conditional_resize(used=8), W.conditional_pointwise(),
], ids=lambda w: w.name + w.description[-7:].replace(" ", "_"))
def test_oracle_matches_reference_backend(wl):
    got, want = oracle.run_oracle(wl, threads=4), oracle.run_ref(wl, threads=4)
    for g, w in zip(got, want):
        assert np.array_equal(g, w)


@pytest.mark.skipif(not oracle.have_ref(), reason="reference-backed checker not built")
@pytest.mark.parametrize("kind", [0, 1, 2])          # TensorWrite<float3>, TensorSplit<float3>, TensorTSplit<float3>
@pytest.mark.parametrize("oldest_first", [0, 1])
def test_circular_tensor_updates_match_reference(kind, oldest_first):
    # CircularTensor<.., BATCH = 4>::update of the reference, n times, against the same updates written as divergent launches
    # (n >= BATCH: before that the reference copies planes of its uninitialised temporary tensor)
    lib, ref = oracle.load_oracle(), oracle.load_ref()
    w, h, dw, dh, batch = 160, 90, 48, 32, 4
    pitch = w * 3
    frames = [np.random.RandomState(50 + k).randint(0, 256, pitch * h, dtype=np.uint8) for k in range(9)]
    mul = (0.5, 1.0, 2.0)
    for n in (4, 6, 9):
        temp, out, first = np.zeros(batch * dw * dh * 12, np.uint8), np.zeros(batch * dw * dh * 12, np.uint8), 0
        for k in range(n):
            chains, planes, first = W.circular_update_launch(kind, oldest_first, first, batch, frames[k].ctypes.data, w, h, pitch, dw, dh, mul,
                                                             temp.ctypes.data, out.ctypes.data)
            assert lib.fkb_oracle_run(chains, 2, planes, len(planes), 1) == 0
        want = np.zeros_like(out)
        ptrs = (C.c_void_p * n)(*[f.ctypes.data for f in frames[:n]])
        assert ref.fklref_circular_updates(ptrs, n, w, h, pitch, dw, dh, (C.c_float * 3)(*mul), kind, oldest_first, want.ctypes.data) == 0
        assert np.array_equal(out, want), (kind, oldest_first, n)


def test_oracle_threads_do_not_change_results():
    wl = W.batched_crop_resize(n_frames=2, crops_per_frame=5, w=320, h=240, dst=(64, 64))
    a, b = oracle.run_oracle(wl, threads=1), oracle.run_oracle(wl, threads=4)
    assert np.array_equal(a[0], b[0])
