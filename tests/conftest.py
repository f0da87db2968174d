import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built_libraries():
    """The CUDA library and the CPU checkers are built in-tree; build whatever is missing (nvcc cross-compiles)."""
    from fusedkernellibrary_b200 import abi, build as fkb_build
    import oracle
    if not os.path.exists(abi.LIB_PATH):
        fkb_build.build()
    if not os.path.exists(oracle.ORACLE_SO):
        oracle.build()
    yield


def load_golden(name):
    import json
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    from make_golden import build_case, input_crc
    z = np.load(os.path.join(ROOT, "tests", "golden", name + ".npz"))
    wl = build_case(str(z["factory"]), json.loads(str(z["kwargs"])))
    assert int(z["input_crc"]) == input_crc(wl), "the seeded input generator drifted from the one that made the fixture"
    outs = [z[f"out{i}"] for i in range(len(wl.out_sizes))]
    return wl, outs


GOLDEN_CASES = ["readme_crops_full", "readme_crops_pitched", "vertical_fusion_small", "vertical_fusion_pitched",
                "nv12_small", "nv12_upscale", "batched_small", "divergent_small", "crop_reorder_small",
                "border_constant", "border_replicate", "border_reflect", "border_wrap", "border_reflect_101", "nv12_border_constant",
                "conditional_resize", "conditional_pointwise", "tsplit_resize", "split_planes_f32", "split_planes_u8",
                "nv21_limited_bt709", "uyvy_full_bt2020", "rgb_to_nv12", "rgb_to_nv21", "rgb_to_uyvy", "bgra_crops_swap",
                "rgba_crops_u8", "rgba_crops_f32_reorder", "p010_limited_bt2020", "p210_full_bt2020", "y210_full_bt601",
                "add_alpha_crops_u8_swap", "add_alpha_image", "gray_image_bgra", "gray_crops_u8", "gray_crops_f32_bgr"]


def reference_kats():
    """Golden values copied from the reference's own unit tests (tests/golden/reference_kats.json names the lines)."""
    import json
    with open(os.path.join(ROOT, "tests", "golden", "reference_kats.json")) as f:
        return json.load(f)


def conversion_kat_workload(case):
    """One of the reference's colour-conversion known answers as a one-row image: (workload, expected bytes)."""
    import numpy as np
    from fusedkernellibrary_b200 import abi, workloads as W
    cin, cout, n = len(case["in"][0]), len(case["out"][0]), len(case["in"])
    ops = {"COLOR_BGR2BGRA": [W.op(abi.OP_ADD_ALPHA, (255.0, 0.0, 0.0))], "COLOR_BGR2RGB": [W.op(abi.OP_REORDER_ZYX)],
           "COLOR_BGR2RGBA": [W.op(abi.OP_REORDER_ZYX), W.op(abi.OP_ADD_ALPHA, (255.0, 0.0, 0.0))],
           "COLOR_BGRA2RGB": [W.op(abi.OP_REORDER_ZYX)],
           "COLOR_RGB2GRAY": [W.op(abi.OP_RGB2GRAY, (1.0, 0.0, 0.0))],
           "COLOR_BGR2GRAY": [W.op(abi.OP_REORDER_ZYX), W.op(abi.OP_RGB2GRAY, (1.0, 0.0, 0.0))],
           "COLOR_BGRA2GRAY": [W.op(abi.OP_REORDER_ZYX), W.op(abi.OP_RGB2GRAY, (1.0, 0.0, 0.0))]}[case["code"]]
    src = np.zeros(16, np.uint8)
    src[:cin * n] = np.array(case["in"], np.uint8).ravel()
    ch = W.chain(abi.PIX_U8C4 if cin == 4 else abi.PIX_U8C3, abi.GEOM_NONE, {4: abi.PIX_U8C4, 3: abi.PIX_U8C3, 1: abi.PIX_U8C1}[cout], abi.WRITE_PACKED, ops)
    wl = W.Workload(case["code"], [ch], [src], [cout * n], [W.PlaneSpec(0, 0, 0, n, 1, 16, (0, 0, n, 1), n, 1, cout * n)])
    return wl, np.array(case["out"], np.uint8).ravel()


def read_uyvy_kat_workload(case):
    """One of the reference's ReadYUV<UYVY> images, written out as (Y,U,V) byte triples: (workload, expected bytes)."""
    import numpy as np
    from fusedkernellibrary_b200 import abi, workloads as W
    w, h = case["w"], case["h"]
    src = np.array(case["data"], np.uint8)
    ch = W.chain(abi.PIX_UYVY, abi.GEOM_NONE, abi.PIX_U8C3, abi.WRITE_PACKED, [])
    wl = W.Workload("read_uyvy", [ch], [src], [w * h * 3], [W.PlaneSpec(0, 0, 0, w, h, w * 2, (0, 0, w, h), w, h, w * 3)])
    return wl, np.array(case["out"], np.uint8).ravel()


def ycbcr_round_trip(run, rng, prim):
    """The property the reference's unit test checks for ConvertRGBToYUV (utest_color_conversion.h:683-735): seven colours
    -> RGB2YUV -> stored as bytes -> YUV2RGB come back within 1 % of full scale.  ``run(workload)`` returns the output
    buffers.  Returns the largest absolute error."""
    import ctypes as C
    import numpy as np
    from fusedkernellibrary_b200 import abi, workloads as W
    factors = [(0, 0, 0), (1, 1, 1), (1, 0, 0), (0, 1, 0), (0, 0, 1), (0.5, 0.5, 0.5), (0.2, 0.6, 0.9)]
    rgb = np.array([[int(np.float32(f) * np.float32(255.0)) for f in t] for t in factors], np.uint8)
    n = len(factors)
    lib = abi.load()
    m2, add, m, sub = (C.c_float * 9)(), (C.c_float * 3)(), (C.c_float * 9)(), (C.c_float * 3)()
    assert lib.fkb_rgb_to_ycbcr(rng, prim, m2, add) == 0 and lib.fkb_ycbcr_to_rgb(rng, prim, m, sub) == 0
    src = np.zeros(32, np.uint8)
    src[:3 * n] = rgb.ravel()
    fwd = W.chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C3, abi.WRITE_PACKED, [W.op(abi.OP_RGB2YUV), W.op(abi.OP_SATCAST_U8)],
                  ccm2=tuple(m2), yuv_add=tuple(add))
    plane = [W.PlaneSpec(0, 0, 0, n, 1, 32, (0, 0, n, 1), n, 1, 3 * n)]
    yuv = run(W.Workload("rgb_to_ycbcr", [fwd], [src], [3 * n], plane))[0]
    src2 = np.zeros(32, np.uint8)
    src2[:3 * n] = yuv[:3 * n]
    back = W.chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_F32C3, abi.WRITE_PACKED, [W.op(abi.OP_YUV2RGB)], ccm=tuple(m), yuv_sub=tuple(sub))
    plane2 = [W.PlaneSpec(0, 0, 0, n, 1, 32, (0, 0, n, 1), n, 1, 12 * n)]
    out = run(W.Workload("ycbcr_to_rgb", [back], [src2], [12 * n], plane2))[0]
    got = np.frombuffer(out.tobytes()[:12 * n], np.float32).reshape(n, 3)
    return float(np.abs(got - rgb.astype(np.float32)).max())
