"""TEST INFRASTRUCTURE — Python loaders for the two CPU checkers.  Only tests/, the smoke check and the benchmark's
CPU-baseline / reference arm may import this package; the product (fusedkernellibrary_b200) never does.

* ``liboracle.so``        — the restatement (oracle/fkb_oracle.cpp); always available (built by oracle/Makefile).
* ``_ref/libfkl_ref.so``  — the reference's own CPU backend compiled from its headers (oracle/ref_runner.cpp);
                            present when it was built where the reference is installed.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

from fusedkernellibrary_b200 import abi

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libfkl_ref.so")
REF_CUDA_SO = os.path.join(HERE, "_ref", "libfkl_ref_cuda.so")

_oracle = None
_ref = None


REF_DIR_DEFAULT = "/root/reference"


def build() -> None:
    """Compiles both checkers; the reference-backed ones only where the reference tree is installed (environment
    variable FKB_REF_DIR, else the default location above)."""
    ref_dir = os.environ.get("FKB_REF_DIR", REF_DIR_DEFAULT)
    subprocess.run(["make", "-s", "-C", HERE, f"FKB_REF_DIR={ref_dir}"], check=True)


def load_oracle() -> C.CDLL:
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_SO):
            build()
        lib = C.CDLL(ORACLE_SO)
        lib.fkb_oracle_resize_params.restype = C.c_int
        lib.fkb_oracle_resize_params.argtypes = [C.c_uint32, C.POINTER(abi.PlaneDesc)]
        lib.fkb_oracle_run.restype = C.c_int
        lib.fkb_oracle_run.argtypes = [C.POINTER(abi.ChainDesc), C.c_uint32, C.POINTER(abi.PlaneDesc), C.c_uint32, C.c_uint32]
        lib.fkb_oracle_ycbcr_to_rgb.restype = C.c_int
        lib.fkb_oracle_ycbcr_to_rgb.argtypes = [C.c_uint32, C.c_uint32, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        lib.fkb_oracle_ycbcr_to_rgb_bits.restype = C.c_int
        lib.fkb_oracle_ycbcr_to_rgb_bits.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        lib.fkb_oracle_rgb_to_ycbcr.restype = C.c_int
        lib.fkb_oracle_rgb_to_ycbcr.argtypes = [C.c_uint32, C.c_uint32, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        lib.fkb_oracle_saturate_u8.restype = C.c_uint8
        lib.fkb_oracle_saturate_u8.argtypes = [C.c_float]
        lib.fkb_oracle_round_half_away.restype = C.c_float
        lib.fkb_oracle_round_half_away.argtypes = [C.c_float]
        _oracle = lib
    return _oracle


def have_ref() -> bool:
    return os.path.exists(REF_SO)


def load_ref() -> C.CDLL:
    global _ref
    if _ref is None:
        lib = C.CDLL(REF_SO)
        u8p, f32p, i32p, pp = C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_void_p)
        lib.fklref_crop_resize_u8.argtypes = [pp, C.c_int, C.c_int, C.c_int, i32p, C.c_int, C.c_int, C.c_int, f32p, f32p, f32p, C.c_void_p, C.c_int]
        lib.fklref_crop_resize_f32.argtypes = [pp, C.c_int, C.c_int, C.c_int, i32p, C.c_int, C.c_int, C.c_int, f32p, f32p, C.c_void_p, C.c_int]
        lib.fklref_crop_reorder_u8.argtypes = [pp, C.c_int, C.c_int, C.c_int, i32p, C.c_int, C.c_void_p, C.c_int]
        lib.fklref_pointwise_u8.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, f32p, f32p, f32p, C.c_void_p, C.c_int]
        lib.fklref_nv12_resize_split.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, f32p, C.c_void_p]
        lib.fklref_divergent.argtypes = [pp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, f32p, C.c_void_p, C.c_void_p, C.c_int]
        lib.fklref_bt709_full_matrix.argtypes = [f32p]
        lib.fklref_saturate_u8.restype = C.c_uint8
        lib.fklref_saturate_u8.argtypes = [C.c_float]
        lib.fklref_resize_params.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, i32p]
        u8p = C.POINTER(C.c_uint8)
        lib.fklref_rgb_to_ycbcr_matrix.restype = C.c_int
        lib.fklref_rgb_to_ycbcr_matrix.argtypes = [C.c_int, C.c_int, f32p]
        lib.fklref_rgb_to_yuv_image.restype = C.c_int
        lib.fklref_rgb_to_yuv_image.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
        lib.fklref_circular_updates.restype = C.c_int
        lib.fklref_circular_updates.argtypes = [pp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, C.c_int, C.c_int, C.c_void_p]
        lib.fklref_add_alpha_crops.restype = C.c_int
        lib.fklref_add_alpha_crops.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, i32p, C.c_int, C.c_int, f32p, f32p, C.c_int, C.c_int, C.c_void_p]
        lib.fklref_gray_image.restype = C.c_int
        lib.fklref_gray_image.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
        lib.fklref_gray_crops.restype = C.c_int
        lib.fklref_gray_crops.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_void_p]
        lib.fklref_add_alpha_image.restype = C.c_int
        lib.fklref_add_alpha_image.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
        lib.fklref_rgba_crops.restype = C.c_int
        lib.fklref_rgba_crops.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, i32p, C.c_int, C.c_int, f32p, f32p, C.c_int, C.c_int, C.c_void_p]
        lib.fklref_bgra_crop_resize_f32.restype = C.c_int
        lib.fklref_bgra_crop_resize_f32.argtypes = [pp, C.c_int, C.c_int, C.c_int, i32p, C.c_int, C.c_int, f32p, C.c_int, C.c_void_p]
        lib.fklref_resize_split_planes.restype = C.c_int
        lib.fklref_resize_split_planes.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, C.c_int, C.c_void_p,
                                                   C.c_void_p, C.c_void_p, C.c_int]
        lib.fklref_resize_tsplit_f32.restype = C.c_int
        lib.fklref_resize_tsplit_f32.argtypes = [pp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, C.c_void_p]
        lib.fklref_border_crop_resize.restype = C.c_int
        lib.fklref_border_crop_resize.argtypes = [C.c_int, pp, C.c_int, C.c_int, C.c_int, i32p, f32p, C.c_int, C.c_int, f32p, f32p, C.c_void_p]
        lib.fklref_nv12_border_constant.restype = C.c_int
        lib.fklref_nv12_border_constant.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, i32p, f32p, C.c_int, C.c_int, C.c_void_p]
        lib.fklref_ycbcr_matrix.restype = C.c_int
        lib.fklref_ycbcr_matrix.argtypes = [C.c_int, C.c_int, f32p]
        lib.fklref_ycbcr_matrix10.restype = C.c_int
        lib.fklref_ycbcr_matrix10.argtypes = [C.c_int, C.c_int, f32p, f32p]
        lib.fklref_yuv10_resize_split.restype = C.c_int
        lib.fklref_yuv10_resize_split.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, f32p, C.c_void_p]
        lib.fklref_yuv_resize_split.restype = C.c_int
        lib.fklref_yuv_resize_split.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, f32p, C.c_void_p]
        lib.fklref_conditional_resize_f32.argtypes = [pp, C.c_int, C.c_int, C.c_int, C.c_int, u8p, C.c_int, C.c_int, f32p, C.c_void_p]
        lib.fklref_conditional_pointwise_u8.argtypes = [pp, C.c_int, C.c_int, C.c_int, C.c_int, u8p, f32p, C.c_void_p]
        for name in ("fklref_crop_resize_u8", "fklref_crop_resize_f32", "fklref_crop_reorder_u8", "fklref_pointwise_u8",
                     "fklref_nv12_resize_split", "fklref_divergent", "fklref_conditional_resize_f32",
                     "fklref_conditional_pointwise_u8"):
            getattr(lib, name).restype = C.c_int
        _ref = lib
    return _ref


_ref_cuda = None


def have_ref_cuda() -> bool:
    return os.path.exists(REF_CUDA_SO)


def load_ref_cuda() -> C.CDLL:
    """The reference's own CUDA backend compiled for sm_100a (oracle/ref_cuda_runner.cu); device pointers in, no timing inside."""
    global _ref_cuda
    if _ref_cuda is None:
        lib = C.CDLL(REF_CUDA_SO)
        f32p, i32p, pp = C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_void_p)
        lib.fklrefcuda_crop_resize_f32.restype = C.c_int
        lib.fklrefcuda_crop_resize_f32.argtypes = [pp, C.c_int, C.c_int, C.c_int, i32p, C.c_int, C.c_int, C.c_int, f32p, f32p, C.c_void_p, C.c_void_p]
        lib.fklrefcuda_pointwise_u8.restype = C.c_int
        lib.fklrefcuda_pointwise_u8.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, f32p, f32p, f32p, C.c_void_p, C.c_int, C.c_void_p]
        lib.fklrefcuda_nv12_resize_split.restype = C.c_int
        lib.fklrefcuda_nv12_resize_split.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, f32p, C.c_void_p, C.c_void_p]
        lib.fklrefcuda_readme_crops.restype = C.c_int
        lib.fklrefcuda_readme_crops.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, i32p, C.c_int, C.c_int, f32p, f32p, f32p, C.c_void_p, C.c_void_p]
        lib.fklrefcuda_divergent4.restype = C.c_int
        lib.fklrefcuda_divergent4.argtypes = [pp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, f32p, C.c_void_p, C.c_void_p, C.c_void_p]
        _ref_cuda = lib
    return _ref_cuda


def ref_cuda_launcher(wl, src_addrs, dst_addrs, stream_ptr):
    """Returns a zero-argument function that launches workload `wl` (device buffers at the given addresses) once through
    the reference CUDA backend on the given stream, or None when the workload has no reference CUDA runner."""
    lib = load_ref_cuda()
    p0, n, ch = wl.planes[0], len(wl.planes), wl.chains[0]
    if wl.name == "batched_crop_resize" and n % 32 == 0:
        frames = (C.c_void_p * n)(*[src_addrs[s.src] for s in wl.planes])
        flat = [v for s in wl.planes for v in s.crop]
        rects = (C.c_int32 * len(flat))(*flat)
        bg, mul = _f3(p0.bg), _f3(ch.ops[0].v)
        return lambda: lib.fklrefcuda_crop_resize_f32(frames, p0.src_w, p0.src_h, p0.src_pitch, rects, n, p0.dst_w, p0.dst_h, bg, mul,
                                                      dst_addrs[0], stream_ptr)
    if wl.name == "readme_crops" and n == 5:
        flat = [v for s in wl.planes for v in s.crop]
        rects = (C.c_int32 * len(flat))(*flat)
        bg, mul, sub = _f3(p0.bg), _f3(ch.ops[0].v), _f3(ch.ops[1].v)
        return lambda: lib.fklrefcuda_readme_crops(src_addrs[0], p0.src_w, p0.src_h, p0.src_pitch, rects, p0.dst_w, p0.dst_h, bg, mul, sub,
                                                   dst_addrs[0], stream_ptr)
    if wl.name == "divergent_planes" and n == 8:
        frames = (C.c_void_p * n)(*[src_addrs[s.src] for s in wl.planes])
        scales = (C.c_float * 4)(*[float(x) for x in wl.extra["scales"]])
        offs = (C.c_float * 4)(*[float(x) for x in wl.extra["offs"]])
        return lambda: lib.fklrefcuda_divergent4(frames, p0.src_w, p0.src_h, p0.src_pitch, p0.dst_w, p0.dst_h, scales, offs,
                                                 dst_addrs[0], dst_addrs[1], stream_ptr)
    if wl.name == "vertical_fusion":
        a, b, c = _f3(ch.ops[1].v), _f3(ch.ops[2].v), _f3(ch.ops[3].v)
        return lambda: lib.fklrefcuda_pointwise_u8(src_addrs[0], p0.src_w, p0.src_h, p0.src_pitch, a, b, c, dst_addrs[0], p0.dst_pitch, stream_ptr)
    if wl.name == "nv12_preprocess":
        a, b = _f3(ch.ops[1].v), _f3(ch.ops[2].v)
        return lambda: lib.fklrefcuda_nv12_resize_split(src_addrs[0], p0.src_w, p0.src_h, p0.src_pitch, p0.dst_w, p0.dst_h, a, b,
                                                        dst_addrs[0], stream_ptr)
    return None


def _f3(v):
    return (C.c_float * 3)(*[float(x) for x in v])


def run_oracle(wl, threads: int = 1, fill: int = 0):
    """Runs a Workload through the restatement on host memory.  Returns one uint8 array per output buffer;
    bytes the launch does not write keep the value ``fill``."""
    lib = load_oracle()
    outs = [np.full(n, fill, np.uint8) for n in wl.out_sizes]
    planes = wl.bind([s.ctypes.data for s in wl.sources], [o.ctypes.data for o in outs],
                     resize_params=lib.fkb_oracle_resize_params)
    rc = lib.fkb_oracle_run(wl.chain_array(), len(wl.chains), planes, len(wl.planes), threads)
    if rc != 0:
        raise RuntimeError(f"oracle returned {rc}")
    return outs


def run_ref(wl, threads: int = 1):
    """Runs a Workload of one of the known configuration shapes through the reference CPU backend."""
    lib = load_ref()
    outs = [np.zeros(n, np.uint8) for n in wl.out_sizes]
    p0 = wl.planes[0]
    n = len(wl.planes)

    def frame_ptrs(specs):
        return (C.c_void_p * len(specs))(*[wl.sources[s.src].ctypes.data for s in specs])

    def rects(specs):
        flat = [v for s in specs for v in s.crop]
        return (C.c_int32 * len(flat))(*flat)

    ch = wl.chains[0]
    if wl.name == "readme_crops":
        rc = lib.fklref_crop_resize_u8(frame_ptrs(wl.planes), p0.src_w, p0.src_h, p0.src_pitch, rects(wl.planes), n,
                                       p0.dst_w, p0.dst_h, _f3(p0.bg), _f3(ch.ops[0].v), _f3(ch.ops[1].v),
                                       outs[0].ctypes.data, threads)
    elif wl.name == "batched_crop_resize":
        rc = lib.fklref_crop_resize_f32(frame_ptrs(wl.planes), p0.src_w, p0.src_h, p0.src_pitch, rects(wl.planes), n,
                                        p0.dst_w, p0.dst_h, _f3(p0.bg), _f3(ch.ops[0].v), outs[0].ctypes.data, threads)
    elif wl.name == "crop_reorder":
        rc = lib.fklref_crop_reorder_u8(frame_ptrs(wl.planes), p0.src_w, p0.src_h, p0.src_pitch, rects(wl.planes), n,
                                        outs[0].ctypes.data, threads)
    elif wl.name == "vertical_fusion":
        rc = lib.fklref_pointwise_u8(wl.sources[0].ctypes.data, p0.src_w, p0.src_h, p0.src_pitch, _f3(ch.ops[1].v),
                                     _f3(ch.ops[2].v), _f3(ch.ops[3].v), outs[0].ctypes.data, p0.dst_pitch)
    elif wl.name.endswith("_preprocess") and wl.extra.get("colour") is not None:
        rng, prim = wl.extra["colour"]
        fn = lib.fklref_yuv10_resize_split if ch.src_format >= 9 else lib.fklref_yuv_resize_split  # ushort sample formats
        rc = fn(ch.src_format, rng, prim, wl.sources[0].ctypes.data, p0.src_w, p0.src_h, p0.src_pitch,
                                         p0.dst_w, p0.dst_h, _f3(ch.ops[1].v), _f3(ch.ops[2].v), outs[0].ctypes.data)
        if rc == -1:
            raise ValueError("the reference runner has no instantiation for this format / range / primitives")
    elif wl.name == "nv12_preprocess":
        rc = lib.fklref_nv12_resize_split(wl.sources[0].ctypes.data, p0.src_w, p0.src_h, p0.src_pitch, p0.dst_w, p0.dst_h,
                                          _f3(ch.ops[1].v), _f3(ch.ops[2].v), outs[0].ctypes.data)
    elif wl.name == "divergent_planes":
        k = n // 2
        scales = (C.c_float * k)(*[float(x) for x in wl.extra["scales"]])
        offs = (C.c_float * k)(*[float(x) for x in wl.extra["offs"]])
        rc = lib.fklref_divergent(frame_ptrs(wl.planes), p0.src_w, p0.src_h, p0.src_pitch, p0.dst_w, p0.dst_h, scales, offs,
                                  outs[0].ctypes.data, outs[1].ctypes.data, k)
    elif wl.name == "border_crops":
        flat = [v for r in wl.extra["rects"] for v in r]
        rc = lib.fklref_border_crop_resize(wl.extra["mode"] - 1, frame_ptrs(wl.planes), p0.src_w, p0.src_h, p0.src_pitch,
                                           (C.c_int32 * 16)(*flat), _f3(wl.extra["value"]), p0.dst_w, p0.dst_h, _f3(p0.bg),
                                           _f3(ch.ops[0].v), outs[0].ctypes.data)
    elif wl.name == "nv12_border_constant":
        rc = lib.fklref_nv12_border_constant(wl.sources[0].ctypes.data, p0.src_w, p0.src_h, p0.src_pitch,
                                             (C.c_int32 * 4)(*wl.extra["rect"]), _f3(wl.extra["value"]), p0.dst_w, p0.dst_h,
                                             outs[0].ctypes.data)
    elif wl.name == "rgb_to_yuv_image":
        rng, prim = wl.extra["colour"]
        rc = lib.fklref_rgb_to_yuv_image(wl.extra["fmt"], rng, prim, wl.sources[0].ctypes.data, p0.src_w, p0.src_h, p0.src_pitch,
                                         outs[0].ctypes.data, p0.dst_pitch)
        if rc == -1:
            raise ValueError("the reference runner has no instantiation for this format / range / primitives")
    elif wl.name == "add_alpha_crops":
        flat = [v for r in wl.extra["rects"] for v in r]
        rc = lib.fklref_add_alpha_crops(wl.sources[0].ctypes.data, p0.src_w, p0.src_h, p0.src_pitch, (C.c_int32 * 20)(*flat), p0.dst_w, p0.dst_h,
                                        _f3(wl.extra["m3"]), (C.c_float * 4)(*wl.extra["m4"]), int(wl.extra["swap"]), int(wl.extra["f32"]),
                                        outs[0].ctypes.data)
    elif wl.name == "gray_image":
        rc = lib.fklref_gray_image(wl.sources[0].ctypes.data, p0.src_w, p0.src_h, p0.src_pitch, int(wl.extra["bgr"]), int(wl.extra["src4"]),
                                   outs[0].ctypes.data, p0.dst_pitch)
    elif wl.name == "gray_crops":
        flat = [v for r in wl.extra["rects"] for v in r]
        rc = lib.fklref_gray_crops(wl.sources[0].ctypes.data, p0.src_w, p0.src_h, p0.src_pitch, (C.c_int32 * 20)(*flat), p0.dst_w, p0.dst_h,
                                   C.c_float(wl.extra["mul"]), int(wl.extra["bgr"]), int(wl.extra["f32"]), outs[0].ctypes.data)
    elif wl.name == "add_alpha_image":
        rc = lib.fklref_add_alpha_image(wl.sources[0].ctypes.data, p0.src_w, p0.src_h, p0.src_pitch, int(wl.extra["swap"]),
                                        outs[0].ctypes.data, p0.dst_pitch)
    elif wl.name == "rgba_crops":
        flat = [v for r in wl.extra["rects"] for v in r]
        m1, a1 = (C.c_float * 4)(*wl.extra["m1"]), (C.c_float * 4)(*wl.extra["a1"])
        rc = lib.fklref_rgba_crops(wl.sources[0].ctypes.data, p0.src_w, p0.src_h, p0.src_pitch, (C.c_int32 * 20)(*flat), p0.dst_w, p0.dst_h,
                                   m1, a1, 1 if wl.extra["reorder"] else 0, 1 if wl.extra["f32"] else 0, outs[0].ctypes.data)
    elif wl.name == "bgra_crops":
        flat = [v for r in wl.extra["rects"] for v in r]
        rc = lib.fklref_bgra_crop_resize_f32(frame_ptrs(wl.planes), p0.src_w, p0.src_h, p0.src_pitch, (C.c_int32 * 16)(*flat),
                                             p0.dst_w, p0.dst_h, _f3(ch.ops[ch.n_ops - 1].v), 1 if wl.extra["swap"] else 0, outs[0].ctypes.data)
    elif wl.name == "split_planes":
        base = outs[0].ctypes.data
        rc = lib.fklref_resize_split_planes(wl.sources[0].ctypes.data, p0.src_w, p0.src_h, p0.src_pitch, p0.dst_w, p0.dst_h,
                                            _f3(ch.ops[0].v), 1 if wl.extra["f32"] else 0, base, base + p0.dst_planes[0],
                                            base + p0.dst_planes[1], p0.dst_pitch)
    elif wl.name == "tsplit_resize":
        rc = lib.fklref_resize_tsplit_f32(frame_ptrs(wl.planes), p0.src_w, p0.src_h, p0.src_pitch, p0.dst_w, p0.dst_h,
                                          _f3(ch.ops[0].v), outs[0].ctypes.data)
    elif wl.name in ("conditional_resize", "conditional_pointwise"):
        dflt = (C.c_uint8 * 3)(*[int(v) for v in wl.extra["default"]])
        every = list(wl.planes)
        if wl.name == "conditional_resize":
            rc = lib.fklref_conditional_resize_f32(frame_ptrs(every), p0.src_w, p0.src_h, p0.src_pitch, wl.extra["used"], dflt,
                                                   p0.dst_w, p0.dst_h, _f3(ch.ops[0].v), outs[0].ctypes.data)
        else:
            rc = lib.fklref_conditional_pointwise_u8(frame_ptrs(every), p0.src_w, p0.src_h, p0.src_pitch, wl.extra["used"], dflt,
                                                     _f3(ch.ops[1].v), outs[0].ctypes.data)
    else:
        raise ValueError(f"no reference runner for workload {wl.name}")
    if rc != 0:
        raise RuntimeError(f"reference runner returned {rc}")
    return outs
