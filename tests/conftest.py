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
                "add_alpha_crops_u8_swap", "add_alpha_image"]
