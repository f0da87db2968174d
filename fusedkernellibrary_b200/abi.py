"""ctypes mirror of include/fkb/fkb.h and the loader of the CUDA library.

This module is plumbing for the Python test and benchmark harness: it declares the C structs, loads
``lib/libfkb.so`` (built by :mod:`fusedkernellibrary_b200.build`) and declares every entry point's
signature.  There is no CPU fallback: if the library is missing, :func:`load` raises.
"""
from __future__ import annotations

import ctypes as C
import os

MAX_OPS = 12
MAX_PLANE_PARAMS = 4
MAX_CHAINS = 8
NOALLOC_MAX_PLANES = 4096

OK, ERR_NULL, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_TOO_LARGE, ERR_DEVICE_WAIT, ERR_DEVICE_CHECK = 0, -1, -2, -3, -4, -5, -6, -7

PIX_U8C3, PIX_F32C3, PIX_NV12, PIX_NV21, PIX_UYVY, PIX_U8C4, PIX_F32C4, PIX_F32P3 = 1, 2, 3, 4, 5, 6, 7, 8
PIX_P010, PIX_P210, PIX_Y210 = 9, 10, 11
PIX_U8C1, PIX_F32C1 = 12, 13  # one-channel destinations (after OP_RGB2GRAY)
RANGE_LIMITED, RANGE_FULL = 0, 1
PRIMITIVES_BT601, PRIMITIVES_BT709, PRIMITIVES_BT2020 = 0, 1, 2
GEOM_NONE, GEOM_RESIZE_IGNORE_AR, GEOM_RESIZE_PRESERVE_AR = 0, 1, 2
GEOM_RESIZE_PRESERVE_AR_RN_EVEN, GEOM_RESIZE_PRESERVE_AR_LEFT = 3, 4
PLANE_DEFAULT = 0x80000000  # fkb_plane_desc.chain bit: the plane's read yields bg (conditional batch read)
WRITE_PACKED, WRITE_SPLIT, WRITE_SPLIT_PLANES, WRITE_NV12, WRITE_NV21, WRITE_UYVY = 1, 2, 3, 4, 5, 6
BORDER_NONE, BORDER_CONSTANT, BORDER_REPLICATE, BORDER_REFLECT, BORDER_WRAP, BORDER_REFLECT_101 = 0, 1, 2, 3, 4, 5
OP_CAST_F32, OP_MUL, OP_ADD, OP_SUB, OP_DIV, OP_REORDER_ZYX, OP_YUV2RGB, OP_SATCAST_U8, OP_RGB2YUV, OP_ADD_ALPHA = 1, 2, 3, 4, 5, 6, 7, 8, 9, 10
OP_RGB2GRAY = 11


class Op(C.Structure):
    _fields_ = [("code", C.c_uint16), ("plane_slot", C.c_int16), ("v", C.c_float * 3)]


class ChainDesc(C.Structure):
    _fields_ = [
        ("src_format", C.c_uint32), ("geometry", C.c_uint32), ("dst_format", C.c_uint32),
        ("write_kind", C.c_uint32), ("n_ops", C.c_uint32), ("n_pre_ops", C.c_uint32),
        ("ops", Op * MAX_OPS), ("ccm", C.c_float * 9), ("yuv_sub", C.c_float * 3),
        ("ccm2", C.c_float * 9), ("yuv_add", C.c_float * 3),
        ("border", C.c_uint32), ("border_at", C.c_uint32), ("border_value", C.c_float * 3),
        ("op_w", C.c_float * MAX_OPS), ("border_value_w", C.c_float),
    ]


class PlaneDesc(C.Structure):
    _fields_ = [
        ("src", C.c_void_p), ("src_chroma", C.c_void_p), ("dst", C.c_void_p),
        ("src_pitch", C.c_uint32), ("src_w", C.c_uint32), ("src_h", C.c_uint32),
        ("crop_x", C.c_uint32), ("crop_y", C.c_uint32), ("crop_w", C.c_int32), ("crop_h", C.c_int32),
        ("dst_w", C.c_uint32), ("dst_h", C.c_uint32), ("dst_pitch", C.c_uint32),
        ("dst_channel_stride", C.c_uint64),
        ("fx", C.c_float), ("fy", C.c_float),
        ("x1", C.c_int32), ("y1", C.c_int32), ("x2", C.c_int32), ("y2", C.c_int32),
        ("bg", C.c_float * 3), ("chain", C.c_uint32),
        ("params", (C.c_float * 3) * MAX_PLANE_PARAMS),
        ("dst_y", C.c_void_p), ("dst_z", C.c_void_p),
        ("bg_w", C.c_float), ("params_w", C.c_float * MAX_PLANE_PARAMS),
    ]


assert C.sizeof(Op) == 16 and C.sizeof(ChainDesc) == 384 and C.sizeof(PlaneDesc) == 200

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libfkb.so")
# the self-checking build (every bulk copy and gathered tap tested against its buffer first; see FKB_ERR_DEVICE_CHECK)
DEBUG_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libfkb_debug.so")

# name -> (restype, argtypes); every symbol include/fkb/fkb.h declares
SIGNATURES = {
    "fkb_resize_params": (C.c_int, [C.c_uint32, C.POINTER(PlaneDesc)]),
    "fkb_ycbcr_to_rgb": (C.c_int, [C.c_uint32, C.c_uint32, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "fkb_ycbcr_to_rgb_bits": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "fkb_rgb_to_ycbcr": (C.c_int, [C.c_uint32, C.c_uint32, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "fkb_validate": (C.c_int, [C.POINTER(ChainDesc), C.c_uint32, C.POINTER(PlaneDesc), C.c_uint32]),
    "fkb_launch_transform": (C.c_int, [C.POINTER(ChainDesc), C.POINTER(PlaneDesc), C.c_uint32, C.c_void_p]),
    "fkb_launch_transform_noalloc": (C.c_int, [C.POINTER(ChainDesc), C.POINTER(PlaneDesc), C.c_uint32, C.c_void_p]),
    "fkb_launch_divergent": (C.c_int, [C.POINTER(ChainDesc), C.c_uint32, C.POINTER(PlaneDesc), C.c_uint32, C.c_void_p]),
    "fkb_plan_create": (C.c_int, [C.POINTER(ChainDesc), C.c_uint32, C.POINTER(PlaneDesc), C.c_uint32, C.POINTER(C.c_void_p)]),
    "fkb_plan_launch": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fkb_plan_destroy": (None, [C.c_void_p]),
    "fkb_plan_kernel_launches": (C.c_uint32, [C.c_void_p]),
    "fkb_device_status": (C.c_int, []),
    "fkb_last_cuda_error": (C.c_int, []),
    "fkb_status_string": (C.c_char_p, [C.c_int]),
    "fkb_abi_version": (C.c_uint32, []),
}

_lib = None


def load() -> C.CDLL:
    """Loads lib/libfkb.so (or the build FKB_LIBRARY names) and declares the signatures.  Raises if it was not built."""
    global _lib
    if _lib is None:
        # FKB_LIBRARY names another build of the same library, e.g. the self-checking one
        path = os.environ.get("FKB_LIBRARY") or LIB_PATH
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run `python -m fusedkernellibrary_b200.build` "
                               "(there is no CPU fallback)")
        lib = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class FkbError(RuntimeError):
    def __init__(self, status: int):
        self.status = status
        msg = load().fkb_status_string(status).decode()
        if status == ERR_CUDA:
            msg += f" (cudaError {load().fkb_last_cuda_error()})"
        super().__init__(f"fkb status {status}: {msg}")


def check(status: int) -> None:
    if status != OK:
        raise FkbError(status)
