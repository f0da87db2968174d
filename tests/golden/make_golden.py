"""Generates the golden fixtures in this directory by running the REFERENCE CPU backend
(oracle/_ref/libfkl_ref.so, compiled from the reference headers by oracle/Makefile) on small seeded workloads.

Run where the reference is installed:  ``make -C oracle && python tests/golden/make_golden.py``.
Each ``<case>.npz`` stores the workload factory name, its keyword arguments (JSON), a CRC of the generated
inputs (so a drift of the input generator is caught) and the reference's output bytes.
"""
from __future__ import annotations

import json
import os
import sys
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from fusedkernellibrary_b200 import workloads as W  # noqa: E402

CASES = {
    "readme_crops_full": ("readme_crops", {}),
    "readme_crops_pitched": ("readme_crops", {"w": 500, "h": 300, "pitch_align": 512, "seed": 11,
                                              "crops": [[3, 5, 60, 40], [400, 125, 100, 175], [0, 0, 500, 300], [499, 299, 1, 1], [17, 250, 300, 20]]}),
    "vertical_fusion_small": ("vertical_fusion", {"w": 333, "h": 41, "seed": 12}),
    "vertical_fusion_pitched": ("vertical_fusion", {"w": 250, "h": 19, "seed": 13, "pitch_align": 256, "dst_pitch_align": 64}),
    "nv12_small": ("nv12_preprocess", {"w": 640, "h": 360, "dst": [96, 64], "seed": 14}),
    "nv12_upscale": ("nv12_preprocess", {"w": 64, "h": 36, "dst": [100, 70], "seed": 15}),
    "batched_small": ("batched_crop_resize", {"n_frames": 2, "crops_per_frame": 3, "w": 640, "h": 360, "dst": [64, 48],
                                              "crop_range": [8, 300], "seed": 16}),
    "divergent_small": ("divergent_planes", {"n_per_seq": 2, "w": 160, "h": 90, "seed": 17}),
    "crop_reorder_small": ("crop_reorder", {"n": 3, "w": 320, "h": 200, "crop_size": [50, 30], "seed": 18}),
    # chains beside the five configurations
    "border_constant": ("border_crops", {"mode": 1, "w": 120, "h": 72, "dst": [48, 40]}),
    "border_replicate": ("border_crops", {"mode": 2, "w": 120, "h": 72, "dst": [48, 40]}),
    "border_reflect": ("border_crops", {"mode": 3, "w": 37, "h": 23, "dst": [48, 40]}),
    "border_wrap": ("border_crops", {"mode": 4, "w": 37, "h": 23, "dst": [48, 40]}),
    "border_reflect_101": ("border_crops", {"mode": 5, "w": 37, "h": 23, "dst": [48, 40]}),
    "nv12_border_constant": ("nv12_border_constant", {}),
    "conditional_resize": ("conditional_resize", {"used": 5, "w": 160, "h": 90, "dst": [48, 32]}),
    "conditional_pointwise": ("conditional_pointwise", {"used": 3, "w": 100, "h": 20}),
    "tsplit_resize": ("tsplit_resize", {"w": 150, "h": 85, "dst": [48, 32]}),
    "split_planes_f32": ("split_planes", {"w": 150, "h": 85, "dst": [52, 32]}),
    "split_planes_u8": ("split_planes", {"w": 150, "h": 85, "dst": [52, 32], "f32": False}),
    "nv21_limited_bt709": ("nv12_preprocess", {"w": 320, "h": 180, "dst": [80, 60], "src_format": 4, "colour": [0, 1]}),
    "uyvy_full_bt2020": ("nv12_preprocess", {"w": 320, "h": 180, "dst": [80, 60], "src_format": 5, "colour": [1, 2]}),
    "p010_limited_bt2020": ("nv12_preprocess", {"w": 320, "h": 180, "dst": [80, 60], "src_format": 9, "colour": [0, 2]}),
    "p210_full_bt2020": ("nv12_preprocess", {"w": 322, "h": 90, "dst": [100, 70], "src_format": 10, "colour": [1, 2]}),
    "y210_full_bt601": ("nv12_preprocess", {"w": 320, "h": 180, "dst": [80, 60], "src_format": 11, "colour": [1, 0]}),
    "rgb_to_nv12": ("rgb_to_yuv_image", {"fmt": 3, "colour": [0, 0], "w": 162, "h": 90}),
    "rgb_to_nv21": ("rgb_to_yuv_image", {"fmt": 4, "colour": [0, 2], "w": 162, "h": 90}),
    "rgb_to_uyvy": ("rgb_to_yuv_image", {"fmt": 5, "colour": [1, 2], "w": 162, "h": 90}),
    "bgra_crops_swap": ("bgra_crops", {"swap": True, "w": 160, "h": 100, "dst": [48, 40]}),
    "add_alpha_crops_u8_swap": ("add_alpha_crops", {"swap": True, "w": 480, "h": 270, "dst": [32, 24]}),
    "add_alpha_image": ("add_alpha_image", {"w": 162, "h": 90}),
    "gray_image_bgra": ("gray_image", {"bgr": True, "src4": True, "w": 162, "h": 90}),
    "gray_crops_u8": ("gray_crops", {"w": 480, "h": 270, "dst": [32, 24], "rects": [[0, 0, 120, 40], [100, 200, 60, 40], [400, 20, 30, 50], [300, 100, 30, 30], [40, 40, 40, 40]]}),
    "gray_crops_f32_bgr": ("gray_crops", {"bgr": True, "f32": True, "w": 480, "h": 270, "dst": [32, 24],
                                          "rects": [[0, 0, 120, 40], [100, 200, 60, 40], [400, 20, 30, 50], [300, 100, 30, 30], [40, 40, 40, 40]]}),
    "rgba_crops_u8": ("rgba_crops", {"w": 480, "h": 270, "dst": [32, 32], "rects": [[0, 0, 120, 40], [100, 200, 60, 40], [400, 20, 30, 50], [300, 100, 30, 30], [40, 40, 40, 40]]}),
    "rgba_crops_f32_reorder": ("rgba_crops", {"reorder": True, "f32": True, "w": 480, "h": 270, "dst": [32, 32],
                                              "rects": [[0, 0, 120, 40], [100, 200, 60, 40], [400, 20, 30, 50], [300, 100, 30, 30], [40, 40, 40, 40]]}),
}


def build_case(factory: str, kwargs: dict):
    kw = {k: (tuple(tuple(x) if isinstance(x, list) else x for x in v) if isinstance(v, list) else v) for k, v in kwargs.items()}
    return getattr(W, factory)(**kw)


def input_crc(wl) -> int:
    c = 0
    for s in wl.sources:
        c = zlib.crc32(s.tobytes(), c)
    return c


def main() -> None:
    here = os.path.dirname(os.path.abspath(__file__))
    for name, (factory, kwargs) in CASES.items():
        if "--missing" in sys.argv and os.path.exists(os.path.join(here, name + ".npz")):
            continue  # keep the fixtures that exist
        wl = build_case(factory, kwargs)
        outs = oracle.run_ref(wl)
        np.savez_compressed(os.path.join(here, name + ".npz"), factory=factory, kwargs=json.dumps(kwargs),
                            input_crc=np.uint32(input_crc(wl)), **{f"out{i}": o for i, o in enumerate(outs)})
        print(name, [o.size for o in outs])


if __name__ == "__main__":
    main()
