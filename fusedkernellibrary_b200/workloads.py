"""Seeded synthetic workloads in the shapes of the five benchmark configurations, lowered to fkb descriptors.

A :class:`Workload` holds host source buffers (numpy), the chain descriptors and one :class:`PlaneSpec` per
output plane (which source buffer, which output buffer, byte offsets, geometry).  ``bind`` turns the specs
into an ``fkb_plane_desc`` array for a given set of buffer base addresses — host addresses for the CPU
checker, device addresses for the CUDA library — so both run on exactly the same description.

The inputs stand in for the frames the reference's examples read from disk or cameras: no public dataset is
involved, every byte comes from ``numpy.random.RandomState(seed)``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import abi

BT709_FULL_8BIT = (1.0, 0.0, 1.57480001, 1.0, -0.187324256, -0.46812427, 1.0, 1.8556, 0.0)
"""YCbCr->RGB matrix of ConvertYUVToRGB<p8bit, Full, bt709> as the reference evaluates it in fp32
(algorithms/image_processing/itu_color.h:185-258; golden copy in
utests/algorithm/image_processing/utest_color_conversion.h:441-447)."""


def op(code: int, v=(0.0, 0.0, 0.0), slot: int = -1) -> abi.Op:
    o = abi.Op()
    o.code, o.plane_slot = code, slot
    o.v[:] = [float(np.float32(x)) for x in v]
    return o


def chain(src_format, geometry, dst_format, write_kind, ops, n_pre_ops=0, ccm=None, yuv_sub=None, border=0, border_at=0,
          border_value=(0.0, 0.0, 0.0), ccm2=None, yuv_add=None, op_w=None) -> abi.ChainDesc:
    ch = abi.ChainDesc()
    ch.src_format, ch.geometry, ch.dst_format, ch.write_kind = src_format, geometry, dst_format, write_kind
    ch.n_ops, ch.n_pre_ops = len(ops), n_pre_ops
    for i, o in enumerate(ops):
        ch.ops[i] = o
    if ccm is not None:
        ch.ccm[:] = ccm
    if yuv_sub is not None:
        ch.yuv_sub[:] = yuv_sub
    if ccm2 is not None:
        ch.ccm2[:] = ccm2
    if yuv_add is not None:
        ch.yuv_add[:] = yuv_add
    ch.border, ch.border_at = border, border_at
    ch.border_value[:] = border_value[:3]
    if len(border_value) > 3:
        ch.border_value_w = border_value[3]
    if op_w is not None:  # four-channel chains: the fourth operand of each op
        for i, wv in enumerate(op_w):
            ch.op_w[i] = float(np.float32(wv))
    return ch


@dataclass
class PlaneSpec:
    src: int                     # index into Workload.sources
    dst: int                     # index into Workload.out_sizes
    dst_offset: int              # byte offset of this plane inside the output buffer
    src_w: int
    src_h: int
    src_pitch: int
    crop: tuple                  # (x, y, w, h)
    dst_w: int
    dst_h: int
    dst_pitch: int
    chain: int = 0
    dst_channel_stride: int = 0
    bg: tuple = (0.0, 0.0, 0.0)
    params: tuple = ()           # up to four float3 operands
    chroma_offset: int = 0       # NV12: byte offset of the UV rows inside the source buffer
    dst_planes: tuple = ()       # WRITE_SPLIT_PLANES: byte offsets of the second and third channel plane in the output buffer
    default: bool = False        # a plane beyond usedPlanes of a conditional batch read: its read yields `bg`


@dataclass
class Workload:
    name: str
    chains: list
    sources: list                # list of np.uint8 arrays (flat)
    out_sizes: list              # bytes of each output buffer
    planes: list                 # list of PlaneSpec
    description: str = ""
    extra: dict = field(default_factory=dict)

    @property
    def out_pixels(self) -> int:
        return sum(p.dst_w * p.dst_h for p in self.planes)

    def chain_array(self):
        arr = (abi.ChainDesc * len(self.chains))()
        for i, c in enumerate(self.chains):
            arr[i] = c
        return arr

    def bind(self, src_addrs, dst_addrs, resize_params=None):
        """Returns (fkb_plane_desc * n) with pointers set.  ``resize_params(geometry, plane_ptr)`` fills the
        resize factors (the library's fkb_resize_params by default)."""
        if resize_params is None:
            resize_params = abi.load().fkb_resize_params
        arr = (abi.PlaneDesc * len(self.planes))()
        for i, s in enumerate(self.planes):
            d = arr[i]
            ch = self.chains[s.chain]
            d.src = src_addrs[s.src]
            d.src_chroma = src_addrs[s.src] + s.chroma_offset if ch.src_format in (abi.PIX_NV12, abi.PIX_NV21, abi.PIX_P010, abi.PIX_P210) else None
            d.dst = dst_addrs[s.dst] + s.dst_offset
            d.src_pitch, d.src_w, d.src_h = s.src_pitch, s.src_w, s.src_h
            d.crop_x, d.crop_y, d.crop_w, d.crop_h = s.crop
            d.dst_w, d.dst_h, d.dst_pitch = s.dst_w, s.dst_h, s.dst_pitch
            d.dst_channel_stride = s.dst_channel_stride
            if s.dst_planes:
                d.dst_y, d.dst_z = dst_addrs[s.dst] + s.dst_planes[0], dst_addrs[s.dst] + s.dst_planes[1]
            d.bg[:] = s.bg[:3]
            if len(s.bg) > 3:
                d.bg_w = s.bg[3]
            d.chain = s.chain | (abi.PLANE_DEFAULT if s.default else 0)
            for k, pv in enumerate(s.params):
                d.params[k][:] = pv
            if s.default:
                d.src, d.src_chroma = None, None
            elif ch.geometry != abi.GEOM_NONE:
                rc = resize_params(ch.geometry, C.byref(d))
                if rc != 0:
                    raise ValueError(f"resize params failed for plane {i}: {rc}")
        return arr

    # -- algorithmic bytes ---------------------------------------------------------------------------------
    def algorithmic_bytes(self) -> dict:
        """Distinct source bytes addressed by at least one tap of the launch (deduplicated per source buffer)
        plus output bytes written.  Background pixels address nothing."""
        lib = abi.load()
        masks = {}
        out_bytes = 0
        for s in self.planes:
            ch = self.chains[s.chain]
            uyvy = ch.src_format == abi.PIX_UYVY
            nv12 = ch.src_format in (abi.PIX_NV12, abi.PIX_NV21) or uyvy  # one luma byte per pixel, one chroma pair per 2 (x2) pixels
            elt = {abi.PIX_F32C3: 12, abi.PIX_U8C3: 3, abi.PIX_F32C4: 16, abi.PIX_U8C4: 4, abi.PIX_U8C1: 1, abi.PIX_F32C1: 4}[ch.dst_format]
            out_bytes += s.dst_w * s.dst_h * elt
            if s.default or ch.border:
                continue
            if s.src not in masks:
                masks[s.src] = (np.zeros((s.src_h, s.src_w), bool),
                                np.zeros((s.src_h if uyvy else (s.src_h + 1) // 2, (s.src_w + 1) // 2), bool) if nv12 else None)
            cx, cy, cw, chh = s.crop
            if ch.geometry == abi.GEOM_NONE:
                cols = np.arange(s.dst_w) + cx
                rows = np.arange(s.dst_h) + cy
            else:
                d = abi.PlaneDesc()
                d.crop_w, d.crop_h, d.dst_w, d.dst_h = cw, chh, s.dst_w, s.dst_h
                lib.fkb_resize_params(ch.geometry, C.byref(d))
                tw, th = d.x2 - d.x1 + 1, d.y2 - d.y1 + 1

                def taps(n, f, extent):
                    s_ = np.arange(n, dtype=np.float32) * np.float32(f)
                    a = np.floor(s_).astype(np.int64)
                    return np.unique(np.concatenate([np.minimum(a, extent - 1), np.minimum(a + 1, extent - 1)]))
                cols = taps(tw, d.fx, cw) + cx
                rows = taps(th, d.fy, chh) + cy
            m, muv = masks[s.src]
            m[np.ix_(rows, cols)] = True
            if nv12:
                muv[np.ix_(rows if uyvy else np.unique(rows >> 1), np.unique(cols >> 1))] = True
        src_bytes = 0
        for m, muv in masks.values():
            src_bytes += int(m.sum()) * (1 if muv is not None else 3)
            if muv is not None:
                src_bytes += int(muv.sum()) * 2
        return {"src": src_bytes, "dst": out_bytes, "total": src_bytes + out_bytes}


def _frame(seed: int, nbytes: int, lo: int = 0, hi: int = 256) -> np.ndarray:
    return np.random.RandomState(seed).randint(lo, hi, size=nbytes, dtype=np.uint8)


def _pitch(row_bytes: int, align: int) -> int:
    return (row_bytes + align - 1) // align * align


# ------------------------------------------------------------------------------------------------------------
# the five configurations (every size is a parameter so tests can run reduced versions)
# ------------------------------------------------------------------------------------------------------------
README_CROPS = ((300, 125, 60, 40), (400, 125, 60, 40), (530, 270, 130, 140), (560, 115, 100, 35), (572, 196, 40, 15))


def readme_crops(w=1920, h=1080, crops=README_CROPS, dst=(128, 64), seed=1, pitch_align=16) -> Workload:
    """Config 1: one uchar3 frame, crops -> Resize PRESERVE_AR (bg 0) -> Mul 2 -> Sub 128 -> SaturateCast ->
    TensorWrite<uchar3>.  The reference program is tests/examples/readme_test_code.h:26-106."""
    pitch = _pitch(w * 3, pitch_align)
    ch = chain(abi.PIX_U8C3, abi.GEOM_RESIZE_PRESERVE_AR, abi.PIX_U8C3, abi.WRITE_PACKED,
               [op(abi.OP_MUL, (2, 2, 2)), op(abi.OP_SUB, (128, 128, 128)), op(abi.OP_SATCAST_U8)])
    dw, dh = dst
    planes = [PlaneSpec(0, 0, i * dw * dh * 3, w, h, pitch, c, dw, dh, dw * 3, bg=(0.0, 0.0, 0.0)) for i, c in enumerate(crops)]
    return Workload("readme_crops", [ch], [_frame(seed, pitch * h)], [dw * dh * 3 * len(crops)], planes,
                    f"{len(crops)} crops of one {w}x{h} uchar3 frame -> {dw}x{dh} uchar3 tensor")


def vertical_fusion(w=3840, h=2160, seed=2, pitch_align=16, dst_pitch_align=16) -> Workload:
    """Config 2: Cast -> Mul -> Add -> Div -> BGR2RGB -> SaturateCast on every pixel, uchar3 -> uchar3."""
    pitch, dpitch = _pitch(w * 3, pitch_align), _pitch(w * 3, dst_pitch_align)
    ch = chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C3, abi.WRITE_PACKED,
               [op(abi.OP_CAST_F32), op(abi.OP_MUL, (0.5, 1.5, 2.0)), op(abi.OP_ADD, (10, -20, 5)),
                op(abi.OP_DIV, (1.7, 1.7, 1.7)), op(abi.OP_REORDER_ZYX), op(abi.OP_SATCAST_U8)])
    planes = [PlaneSpec(0, 0, 0, w, h, pitch, (0, 0, w, h), w, h, dpitch)]
    return Workload("vertical_fusion", [ch], [_frame(seed, pitch * h)], [dpitch * h], planes,
                    f"{w}x{h} uchar3 -> uchar3, six fused element-wise ops")


def nv12_preprocess(w=3840, h=2160, dst=(640, 640), seed=3, pitch_align=16, ccm=None, yuv_sub=(0.0, 128.0, 128.0),
                    src_format=abi.PIX_NV12, colour=None) -> Workload:
    """Config 3: ReadYUV<NV12> -> ConvertYUVToRGB<p8bit,Full,bt709> -> Resize IGNORE_AR -> Sub mean -> Div std ->
    TensorSplit<float3> (planar CHW fp32).  ``src_format`` selects NV21, UYVY or one of the 10-bit formats (P010, P210,
    Y210: ushort samples in 0..1023) instead; ``colour=(range, primitives)`` takes the matrix and offsets from
    fkb_ycbcr_to_rgb_bits for the format's depth (required for the 10-bit formats)."""
    wide = src_format in (abi.PIX_P010, abi.PIX_P210, abi.PIX_Y210)
    packed = src_format in (abi.PIX_UYVY, abi.PIX_Y210)
    pitch = _pitch(w * (2 if packed else 1) * (2 if wide else 1), pitch_align)
    dw, dh = dst
    if colour is not None:
        m, sub = (C.c_float * 9)(), (C.c_float * 3)()
        if abi.load().fkb_ycbcr_to_rgb_bits(10 if wide else 8, colour[0], colour[1], m, sub) != 0:
            raise ValueError("fkb_ycbcr_to_rgb_bits refused the colour description")
        ccm, yuv_sub = tuple(m), tuple(sub)
    elif wide:
        raise ValueError("a 10-bit source needs colour=(range, primitives)")
    mean, std = ((496.7, 466.9, 415.6), (234.2, 229.1, 230.2)) if wide else ((123.675, 116.28, 103.53), (58.395, 57.12, 57.375))
    ch = chain(src_format, abi.GEOM_RESIZE_IGNORE_AR, abi.PIX_F32C3, abi.WRITE_SPLIT,
               [op(abi.OP_YUV2RGB), op(abi.OP_SUB, mean), op(abi.OP_DIV, std)],
               n_pre_ops=1, ccm=BT709_FULL_8BIT if ccm is None else ccm, yuv_sub=yuv_sub)
    planes = [PlaneSpec(0, 0, 0, w, h, pitch, (0, 0, w, h), dw, dh, dw * 4, dst_channel_stride=dw * dh * 4,
                        chroma_offset=pitch * h)]
    name = {abi.PIX_NV12: "nv12_preprocess", abi.PIX_NV21: "nv21_preprocess", abi.PIX_UYVY: "uyvy_preprocess",
            abi.PIX_P010: "p010_preprocess", abi.PIX_P210: "p210_preprocess", abi.PIX_Y210: "y210_preprocess"}[src_format]
    rows = h if packed else 2 * h if src_format == abi.PIX_P210 else h + h // 2
    if wide:  # samples over the whole 10-bit scale, stored as they are in 16-bit words
        frame = np.random.RandomState(seed).randint(40, 1000, size=pitch * rows // 2).astype(np.uint16).view(np.uint8)
    else:
        frame = _frame(seed, pitch * rows, 16, 236)
    return Workload(name, [ch], [frame], [dw * dh * 12], planes,
                    f"{name[:4].upper()} {w}x{h} -> planar fp32 3x{dh}x{dw}", extra={"colour": colour})


def tsplit_resize(w=300, h=170, dst=(96, 64), seed=13) -> Workload:
    """Four frames -> Resize IGNORE_AR -> Mul -> TensorTSplit<float3>: a colour-plane-transposed tensor (all first
    channels of the four images, then all second ones, then all third ones)."""
    pitch = _pitch(w * 3, 16)
    dw, dh = dst
    plane = dw * dh * 4
    ch = chain(abi.PIX_U8C3, abi.GEOM_RESIZE_IGNORE_AR, abi.PIX_F32C3, abi.WRITE_SPLIT, [op(abi.OP_MUL, (0.25, 1.0, 2.5))])
    planes = [PlaneSpec(i, 0, i * plane, w, h, pitch, (0, 0, w, h), dw, dh, dw * 4, dst_channel_stride=4 * plane) for i in range(4)]
    return Workload("tsplit_resize", [ch], [_frame(seed + i, pitch * h) for i in range(4)], [12 * plane], planes,
                    "4 frames -> transposed planar fp32 tensor")


def border_crops(mode=abi.BORDER_REPLICATE, w=200, h=120, dst=(96, 80), value=(9, 77, 250), seed=14) -> Workload:
    """Four frames -> BorderReader<mode> -> Crop (rectangles that leave the frame on every side; one stays inside) ->
    Resize PRESERVE_AR -> Mul -> TensorWrite<float3>."""
    pitch = _pitch(w * 3, 16)
    dw, dh = dst
    ch = chain(abi.PIX_U8C3, abi.GEOM_RESIZE_PRESERVE_AR, abi.PIX_F32C3, abi.WRITE_PACKED, [op(abi.OP_MUL, (0.5, 1.0, 2.0))],
               border=mode, border_at=0, border_value=tuple(float(v) for v in value))
    rects = [(-30, -20, 100, 90), (w - 40, h - 25, 90, 70), (20, 10, 64, 48), (-w // 2, h - 10, 2 * w, 60)]
    planes = [PlaneSpec(i, 0, i * dw * dh * 12, w, h, pitch, (x & 0xffffffff, y & 0xffffffff, cw, chh), dw, dh, dw * 12,
                        bg=(114.0, 114.0, 114.0)) for i, (x, y, cw, chh) in enumerate(rects)]
    return Workload("border_crops", [ch], [_frame(seed + i, pitch * h) for i in range(4)], [4 * dw * dh * 12], planes,
                    f"BorderReader mode {mode}", extra={"mode": mode, "value": value, "rects": rects})


def nv12_border_constant(w=128, h=72, dst=(80, 60), rect=(-16, -8, 160, 90), value=(12.5, 200.25, 99.0), seed=15) -> Workload:
    """ReadYUV<NV12> -> ConvertYUVToRGB -> BorderReader<CONSTANT>(float3) -> Crop -> Resize IGNORE_AR -> TensorSplit<float3>:
    the constant stands for the converted colour."""
    pitch = _pitch(w, 16)
    dw, dh = dst
    ch = chain(abi.PIX_NV12, abi.GEOM_RESIZE_IGNORE_AR, abi.PIX_F32C3, abi.WRITE_SPLIT, [op(abi.OP_YUV2RGB)], n_pre_ops=1,
               ccm=BT709_FULL_8BIT, yuv_sub=(0.0, 128.0, 128.0), border=abi.BORDER_CONSTANT, border_at=1, border_value=value)
    x, y, cw, chh = rect
    planes = [PlaneSpec(0, 0, 0, w, h, pitch, (x & 0xffffffff, y & 0xffffffff, cw, chh), dw, dh, dw * 4, dst_channel_stride=dw * dh * 4,
                        chroma_offset=pitch * h)]
    return Workload("nv12_border_constant", [ch], [_frame(seed, pitch * (h + h // 2), 16, 236)], [dw * dh * 12], planes,
                    "NV12 with a constant border in RGB", extra={"value": value, "rect": rect})


def split_planes(w=300, h=170, dst=(100, 64), seed=16, f32=True) -> Workload:
    """One frame -> Resize IGNORE_AR -> Mul [-> SaturateCast] -> SplitWrite: three separate planes, here at unequal
    distances inside one buffer (second plane last, a gap before the third)."""
    pitch = _pitch(w * 3, 16)
    dw, dh = dst
    elt = 4 if f32 else 1
    dpitch = _pitch(dw * elt, 16)
    plane = dpitch * dh
    ops = [op(abi.OP_MUL, (0.5, 1.0, 1.5))] + ([] if f32 else [op(abi.OP_SATCAST_U8)])
    ch = chain(abi.PIX_U8C3, abi.GEOM_RESIZE_IGNORE_AR, abi.PIX_F32C3 if f32 else abi.PIX_U8C3, abi.WRITE_SPLIT_PLANES, ops)
    planes = [PlaneSpec(0, 0, 0, w, h, pitch, (0, 0, w, h), dw, dh, dpitch, dst_planes=(3 * plane + 64, plane + 32))]
    return Workload("split_planes", [ch], [_frame(seed, pitch * h)], [4 * plane + 64], planes,
                    "SplitWrite into three separate planes " + ("f32" if f32 else "u8"), extra={"f32": f32, "plane": plane})


def rgb_to_yuv_image(fmt=abi.PIX_NV12, colour=(abi.RANGE_FULL, abi.PRIMITIVES_BT709), w=322, h=180, seed=17) -> Workload:
    """PerThreadRead<uchar3> (R,G,B) -> ConvertRGBToYUV -> SaturateCast -> WriteYUV<NV12|NV21|UYVY>."""
    pitch = _pitch(w * 3, 16)
    m, add = (C.c_float * 9)(), (C.c_float * 3)()
    if abi.load().fkb_rgb_to_ycbcr(colour[0], colour[1], m, add) != 0:
        raise ValueError("fkb_rgb_to_ycbcr refused the colour description")
    kind = {abi.PIX_NV12: abi.WRITE_NV12, abi.PIX_NV21: abi.WRITE_NV21, abi.PIX_UYVY: abi.WRITE_UYVY}[fmt]
    ch = chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C3, kind, [op(abi.OP_RGB2YUV), op(abi.OP_SATCAST_U8)], ccm2=tuple(m), yuv_add=tuple(add))
    uyvy = fmt == abi.PIX_UYVY
    opitch = _pitch(w * 2 if uyvy else w, 16)
    size = opitch * h if uyvy else opitch * (h + (h + 1) // 2)  # an odd height still has a chroma row for its last line
    planes = [PlaneSpec(0, 0, 0, w, h, pitch, (0, 0, w, h), w, h, opitch, dst_planes=() if uyvy else (opitch * h, 0))]
    return Workload("rgb_to_yuv_image", [ch], [_frame(seed, pitch * h)], [size], planes, f"RGB -> format {fmt} colour {colour}",
                    extra={"fmt": fmt, "colour": colour})


def bgra_crops(swap=False, w=320, h=200, dst=(96, 80), seed=18) -> Workload:
    """Four uchar4 frames -> Crop -> Resize IGNORE_AR -> alpha discarded (BGRA2BGR, or BGRA2RGB with ``swap``) -> Mul ->
    TensorWrite<float3>."""
    pitch = _pitch(w * 4, 16)
    dw, dh = dst
    ops = ([op(abi.OP_REORDER_ZYX)] if swap else []) + [op(abi.OP_MUL, (0.5, 1.0, 2.0))]
    ch = chain(abi.PIX_U8C4, abi.GEOM_RESIZE_IGNORE_AR, abi.PIX_F32C3, abi.WRITE_PACKED, ops)
    rects = [(0, 0, w, h), (10, 20, 100, 60), (w - 37, h - 21, 37, 21), (5, 5, 8, 9)]
    planes = [PlaneSpec(i, 0, i * dw * dh * 12, w, h, pitch, r, dw, dh, dw * 12) for i, r in enumerate(rects)]
    return Workload("bgra_crops", [ch], [_frame(seed + i, pitch * h) for i in range(4)], [4 * dw * dh * 12], planes,
                    "uchar4 frames, alpha discarded" + (" swap" if swap else ""), extra={"swap": swap, "rects": rects})


RGBA_RECTS = ((0, 0, 120, 40), (100, 200, 60, 40), (400, 20, 30, 50), (1000, 800, 30, 30), (40, 40, 40, 40))


def rgba_crops(reorder=False, f32=False, w=1920, h=1080, dst=(64, 64), rects=RGBA_RECTS, seed=19, border=0) -> Workload:
    """The four-channel pipeline of the reference's compiler-explorer example: one uchar4 frame, five crops -> Resize ->
    Mul -> Add -> [Mul 255 -> [BGRA2RGBA] -> SaturateCast -> TensorWrite<uchar4> | [BGRA2RGBA] -> TensorWrite<float4>]."""
    pitch = _pitch(w * 4, 16)
    dw, dh = dst
    m1, a1 = (0.33 / 255.0, 0.5 / 255.0, 1.0 / 255.0, 0.25 / 255.0), (0.5, 0.25, 0.0, 0.125)
    ops, op_w = [op(abi.OP_MUL, m1[:3]), op(abi.OP_ADD, a1[:3])], [m1[3], a1[3]]
    if not f32:
        ops.append(op(abi.OP_MUL, (255.0,) * 3)); op_w.append(255.0)
    if reorder:
        ops.append(op(abi.OP_REORDER_ZYX)); op_w.append(0.0)
    if not f32:
        ops.append(op(abi.OP_SATCAST_U8)); op_w.append(0.0)
    elt = 16 if f32 else 4
    ch = chain(abi.PIX_U8C4, abi.GEOM_RESIZE_IGNORE_AR, abi.PIX_F32C4 if f32 else abi.PIX_U8C4, abi.WRITE_PACKED, ops, op_w=op_w,
               border=border, border_value=(9.0, 99.0, 199.0, 250.0))
    planes = [PlaneSpec(0, 0, i * dw * dh * elt, w, h, pitch, (x & 0xffffffff, y & 0xffffffff, cw, chh), dw, dh, dw * elt)
              for i, (x, y, cw, chh) in enumerate(rects)]
    return Workload("rgba_crops", [ch], [_frame(seed, pitch * h)], [len(rects) * dw * dh * elt], planes,
                    f"four channels reorder={reorder} f32={f32}", extra={"reorder": reorder, "f32": f32, "m1": m1, "a1": a1, "rects": rects})


def add_alpha_crops(swap=False, f32=False, w=640, h=360, dst=(64, 48), seed=21) -> Workload:
    """One uchar3 frame, five crops -> Resize -> Mul<float3> -> ColorConversion<COLOR_BGR2BGRA | COLOR_BGR2RGBA, float3, float4>
    (an opaque alpha channel of 255 is appended, after a channel swap with ``swap``) -> Mul<float4> ->
    [SaturateCast -> TensorWrite<uchar4> | TensorWrite<float4>]."""
    pitch = _pitch(w * 3, 16)
    dw, dh = dst
    m3, m4 = (0.5, 1.25, 2.0), (1.0, 0.5, 0.75, 0.5)
    rects = [(10, 20, 100, 60), (w // 2, h // 3, 64, 48), (0, 0, w, h), (w - 33, h - 21, 33, 21), (w // 3, h // 3, w // 5, h // 2)]
    ops, op_w = [op(abi.OP_MUL, m3)], [0.0]
    if swap:
        ops.append(op(abi.OP_REORDER_ZYX)); op_w.append(0.0)
    ops += [op(abi.OP_ADD_ALPHA, (255.0, 0.0, 0.0)), op(abi.OP_MUL, m4[:3])]
    op_w += [0.0, m4[3]]
    if not f32:
        ops.append(op(abi.OP_SATCAST_U8)); op_w.append(0.0)
    elt = 16 if f32 else 4
    ch = chain(abi.PIX_U8C3, abi.GEOM_RESIZE_IGNORE_AR, abi.PIX_F32C4 if f32 else abi.PIX_U8C4, abi.WRITE_PACKED, ops, op_w=op_w)
    planes = [PlaneSpec(0, 0, i * dw * dh * elt, w, h, pitch, r, dw, dh, dw * elt) for i, r in enumerate(rects)]
    return Workload("add_alpha_crops", [ch], [_frame(seed, pitch * h)], [5 * dw * dh * elt], planes,
                    f"opaque alpha appended swap={swap} f32={f32}", extra={"swap": swap, "f32": f32, "m3": m3, "m4": m4, "rects": rects})


def add_alpha_image(swap=False, w=322, h=180, seed=22) -> Workload:
    """PerThreadRead<uchar3> -> ColorConversion<COLOR_BGR2BGRA | COLOR_BGR2RGBA, uchar3, uchar4> -> PerThreadWrite<uchar4>."""
    pitch, opitch = _pitch(w * 3, 16), _pitch(w * 4, 64)
    ops = ([op(abi.OP_REORDER_ZYX)] if swap else []) + [op(abi.OP_ADD_ALPHA, (255.0, 0.0, 0.0))]
    ch = chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C4, abi.WRITE_PACKED, ops)
    planes = [PlaneSpec(0, 0, 0, w, h, pitch, (0, 0, w, h), w, h, opitch)]
    return Workload("add_alpha_image", [ch], [_frame(seed, pitch * h)], [opitch * h], planes, f"uchar3 -> uchar4 swap={swap}",
                    extra={"swap": swap})


GRAY_RECTS = ((30, 20, 200, 120), (300, 60, 64, 200), (0, 0, 640, 360), (500, 300, 140, 60), (123, 45, 33, 77))


def gray_image(bgr=False, src4=False, w=322, h=180, seed=23) -> Workload:
    """ColorConversion<COLOR_RGB2GRAY | COLOR_BGR2GRAY | COLOR_RGBA2GRAY | COLOR_BGRA2GRAY, uchar3 | uchar4, uchar> on a whole
    image: PerThreadRead -> conversion -> PerThreadWrite<_2D, uchar>."""
    sp = 4 if src4 else 3
    pitch = _pitch(w * sp, 16)
    ops = ([op(abi.OP_REORDER_ZYX)] if bgr else []) + [op(abi.OP_RGB2GRAY, (1.0, 0.0, 0.0))]
    ch = chain(abi.PIX_U8C4 if src4 else abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C1, abi.WRITE_PACKED, ops)
    opitch = _pitch(w, 16)
    plane = PlaneSpec(0, 0, 0, w, h, pitch, (0, 0, w, h), w, h, opitch)
    return Workload("gray_image", [ch], [_frame(seed, pitch * h)], [opitch * h], [plane], f"gray image bgr={bgr} src4={src4}",
                    extra={"bgr": bgr, "src4": src4})


def gray_crops(bgr=False, f32=False, w=640, h=360, dst=(96, 64), rects=GRAY_RECTS, mul=1.25, seed=24) -> Workload:
    """One uchar3 frame, five crops -> Resize -> ColorConversion<COLOR_RGB2GRAY | COLOR_BGR2GRAY, float3, float> -> Mul<float> ->
    [SaturateCast<float, uchar> -> TensorWrite<uchar> | TensorWrite<float>]."""
    pitch = _pitch(w * 3, 16)
    dw, dh = dst
    ops = ([op(abi.OP_REORDER_ZYX)] if bgr else []) + [op(abi.OP_RGB2GRAY), op(abi.OP_MUL, (mul, 0.0, 0.0))]
    if not f32:
        ops.append(op(abi.OP_SATCAST_U8))
    elt = 4 if f32 else 1
    ch = chain(abi.PIX_U8C3, abi.GEOM_RESIZE_IGNORE_AR, abi.PIX_F32C1 if f32 else abi.PIX_U8C1, abi.WRITE_PACKED, ops)
    planes = [PlaneSpec(0, 0, i * dw * dh * elt, w, h, pitch, r, dw, dh, dw * elt) for i, r in enumerate(rects)]
    return Workload("gray_crops", [ch], [_frame(seed, pitch * h)], [len(rects) * dw * dh * elt], planes, f"gray crops bgr={bgr} f32={f32}",
                    extra={"bgr": bgr, "f32": f32, "rects": rects, "mul": mul})


def conditional_resize(used=5, w=320, h=180, dst=(96, 64), default=(7, 200, 33), seed=11) -> Workload:
    """BatchRead<CONDITIONAL_WITH_DEFAULT> over eight frames of which `used` are read -> Resize IGNORE_AR -> Mul ->
    TensorWrite<float3>; the other planes come out as Mul(float3(default))."""
    pitch = _pitch(w * 3, 16)
    dw, dh = dst
    ch = chain(abi.PIX_U8C3, abi.GEOM_RESIZE_IGNORE_AR, abi.PIX_F32C3, abi.WRITE_PACKED, [op(abi.OP_MUL, (0.5, 1.25, 3.0))])
    planes = [PlaneSpec(i, 0, i * dw * dh * 12, w, h, pitch, (0, 0, w, h), dw, dh, dw * 12, bg=tuple(float(v) for v in default),
                        default=i >= used) for i in range(8)]
    return Workload("conditional_resize", [ch], [_frame(seed + i, pitch * h) for i in range(8)], [8 * dw * dh * 12], planes,
                    f"8 planes, {used} used, default {default}", extra={"used": used, "default": default})


def conditional_pointwise(used=3, w=200, h=40, default=(250, 0, 129), seed=12) -> Workload:
    """The same conditional batch read without a Resize: Cast -> Mul -> SaturateCast -> TensorWrite<uchar3>."""
    pitch = _pitch(w * 3, 16)
    ch = chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C3, abi.WRITE_PACKED,
               [op(abi.OP_CAST_F32), op(abi.OP_MUL, (1.5, 0.25, 2.0)), op(abi.OP_SATCAST_U8)])
    planes = [PlaneSpec(i, 0, i * w * h * 3, w, h, pitch, (0, 0, w, h), w, h, w * 3, bg=tuple(float(v) for v in default),
                        default=i >= used) for i in range(8)]
    return Workload("conditional_pointwise", [ch], [_frame(seed + i, pitch * h) for i in range(8)], [8 * w * h * 3], planes,
                    f"8 planes, {used} used, default {default}", extra={"used": used, "default": default})


def random_rects(n, w, h, lo, hi, rs: np.random.RandomState):
    """x,y uniform in the frame, w,h uniform in [lo,hi], clipped to the frame."""
    out = []
    for _ in range(n):
        x, y = int(rs.randint(0, w)), int(rs.randint(0, h))
        cw, ch = int(rs.randint(lo, hi + 1)), int(rs.randint(lo, hi + 1))
        out.append((x, y, min(cw, w - x), min(ch, h - y)))
    return out


def batched_crop_resize(n_frames=64, crops_per_frame=32, w=1920, h=1080, dst=(224, 224), crop_range=(16, 512),
                        seed=4, pitch_align=16, frame_seed_base=1000, src4=False) -> Workload:
    """Config 4: per frame, random crops -> Resize PRESERVE_AR (bg 114) -> Mul 1/255 -> TensorWrite<float3>.  With
    ``src4`` the frames are uchar4 and the chain discards their alpha channel."""
    pitch = _pitch(w * (4 if src4 else 3), pitch_align)
    dw, dh = dst
    ch = chain(abi.PIX_U8C4 if src4 else abi.PIX_U8C3, abi.GEOM_RESIZE_PRESERVE_AR, abi.PIX_F32C3, abi.WRITE_PACKED,
               [op(abi.OP_MUL, (1.0 / 255.0,) * 3)])
    rs = np.random.RandomState(seed)
    rects = random_rects(n_frames * crops_per_frame, w, h, crop_range[0], crop_range[1], rs)
    planes = [PlaneSpec(i // crops_per_frame, 0, i * dw * dh * 12, w, h, pitch, r, dw, dh, dw * 12, bg=(114.0, 114.0, 114.0))
              for i, r in enumerate(rects)]
    sources = [_frame(frame_seed_base + f, pitch * h) for f in range(n_frames)]
    return Workload("batched_crop_resize_uchar4" if src4 else "batched_crop_resize", [ch], sources, [dw * dh * 12 * len(planes)], planes,
                    f"{n_frames} frames {w}x{h} uchar3 x {crops_per_frame} crops -> {dw}x{dh} float3 tensor",
                    extra={"n_frames": n_frames, "crops_per_frame": crops_per_frame})


def divergent_planes(n_per_seq=4, w=3840, h=2160, seed=5, pitch_align=16) -> Workload:
    """Config 5: one launch over 2n planes.  Planes [0,n): Resize IGNORE_AR to w/2 x h/2 -> SaturateCast -> uchar3
    tensor.  Planes [n,2n): Cast -> Mul scale_i -> Sub offset_i -> float3 written at the global plane index of a
    2n-plane tensor (as DivergentBatchTransformDPP passes the global z through)."""
    pitch = _pitch(w * 3, pitch_align)
    dw, dh = w // 2, h // 2
    c0 = chain(abi.PIX_U8C3, abi.GEOM_RESIZE_IGNORE_AR, abi.PIX_U8C3, abi.WRITE_PACKED, [op(abi.OP_SATCAST_U8)])
    c1 = chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_F32C3, abi.WRITE_PACKED,
               [op(abi.OP_CAST_F32), op(abi.OP_MUL, slot=0), op(abi.OP_SUB, slot=1)])
    rs = np.random.RandomState(seed)
    scales = rs.uniform(0.5, 2.0, n_per_seq).astype(np.float32)
    offs = rs.uniform(0.0, 64.0, n_per_seq).astype(np.float32)
    planes = []
    for i in range(n_per_seq):
        planes.append(PlaneSpec(i, 0, i * dw * dh * 3, w, h, pitch, (0, 0, w, h), dw, dh, dw * 3, chain=0))
    for i in range(n_per_seq):
        z = n_per_seq + i
        planes.append(PlaneSpec(z, 1, z * w * h * 12, w, h, pitch, (0, 0, w, h), w, h, w * 12, chain=1,
                                params=((float(scales[i]),) * 3, (float(offs[i]),) * 3)))
    sources = [_frame(seed * 100 + f, pitch * h) for f in range(2 * n_per_seq)]
    return Workload("divergent_planes", [c0, c1], sources, [dw * dh * 3 * n_per_seq, w * h * 12 * 2 * n_per_seq], planes,
                    f"{2 * n_per_seq} uchar3 {w}x{h} planes, two chains in one launch",
                    extra={"scales": scales, "offs": offs})


def crop_reorder(n=3, w=640, h=360, crop_size=(100, 60), seed=6, pitch_align=16) -> Workload:
    """Integer-only chain: crops -> BGR2RGB on uchar3 -> TensorWrite<uchar3> (must be bit-exact)."""
    pitch = _pitch(w * 3, pitch_align)
    cw, chh = crop_size
    ch = chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C3, abi.WRITE_PACKED, [op(abi.OP_REORDER_ZYX)])
    rs = np.random.RandomState(seed)
    rects = [(int(rs.randint(0, w - cw + 1)), int(rs.randint(0, h - chh + 1)), cw, chh) for _ in range(n)]
    planes = [PlaneSpec(0, 0, i * cw * chh * 3, w, h, pitch, r, cw, chh, cw * 3) for i, r in enumerate(rects)]
    return Workload("crop_reorder", [ch], [_frame(seed, pitch * h)], [cw * chh * 3 * n], planes,
                    f"{n} crops {cw}x{chh} of a {w}x{h} uchar3 frame, channel reorder only")


# ---------------------------------------------------------------------------------------------------------------
# sharding over GPUs: the path has no exchange step, a shard is a subset of the planes with the frames they read
# ---------------------------------------------------------------------------------------------------------------
def shard_by_frame(wl: Workload, rank: int, world: int) -> Workload:
    """The batched workload split by frame, as one 64-frame batch is divided over the GPUs of a box: rank r keeps frames
    [r * n / world, (r + 1) * n / world), the planes cropped from them, and a dense output tensor of just those planes
    (in the whole job they are a contiguous range of the result tensor's planes)."""
    n = len(wl.sources)
    lo, hi = rank * n // world, (rank + 1) * n // world
    keep = [p for p in wl.planes if lo <= p.src < hi]
    plane_bytes = keep[0].dst_pitch * keep[0].dst_h
    planes = [PlaneSpec(**{**p.__dict__, "src": p.src - lo, "dst_offset": i * plane_bytes}) for i, p in enumerate(keep)]
    return Workload(wl.name, wl.chains, wl.sources[lo:hi], [len(planes) * plane_bytes], planes, wl.description,
                    extra={**wl.extra, "n_frames": hi - lo, "first_frame": lo})


def plane_partition(n_planes: int, world: int) -> list:
    """Which planes of the divergent launch each rank runs: plane z goes to rank z % world.  The launch lists the planes
    of its first chain first and those of its second chain after them, in equal numbers, so for world sizes up to that
    number every rank gets as many planes of one kind as of the other; beyond it a rank holds a single plane and the
    slowest kind of plane bounds the speed-up."""
    return [[z for z in range(n_planes) if z % world == r] for r in range(world)]


def shard_by_plane(wl: Workload, rank: int, world: int) -> Workload:
    """The divergent launch split by plane.  A plane keeps its chain and its place in the output tensors (every sequence
    of the reference's DivergentBatchTransformDPP sees the global plane index, core/execution_model/
    data_parallel_patterns.h:322-331), so each rank holds output tensors of the global shape and writes its planes of
    them; it holds only the frames its planes read."""
    mine = plane_partition(len(wl.planes), world)[rank]
    frames = sorted({wl.planes[z].src for z in mine})
    planes = [PlaneSpec(**{**wl.planes[z].__dict__, "src": frames.index(wl.planes[z].src)}) for z in mine]
    return Workload(wl.name, wl.chains, [wl.sources[f] for f in frames], list(wl.out_sizes), planes, wl.description,
                    extra={**wl.extra, "global_planes": mine})


def combine(parts) -> Workload:
    """One divergent launch out of several single-chain workloads: chain c is the chain of parts[c], its planes follow
    those of the chains before it (the order in which a divergent launch of the reference lists its sequences); sources
    and output buffers are kept apart."""
    chains, sources, out_sizes, planes = [], [], [], []
    for c, wl in enumerate(parts):
        assert len(wl.chains) == 1
        s0, o0 = len(sources), len(out_sizes)
        chains.append(wl.chains[0])
        sources += list(wl.sources)
        out_sizes += list(wl.out_sizes)
        planes += [PlaneSpec(**{**p.__dict__, "src": p.src + s0, "dst": p.dst + o0, "chain": c}) for p in wl.planes]
    return Workload("combined_" + "_".join(wl.name for wl in parts), chains, sources, out_sizes, planes,
                    f"divergent launch of {len(parts)} chains")


CONFIGS = {
    "readme_crops": readme_crops,
    "vertical_fusion": vertical_fusion,
    "nv12_preprocess": nv12_preprocess,
    "batched_crop_resize": batched_crop_resize,
    "divergent_planes": divergent_planes,
}


def random_workload(seed: int, max_dim: int = 260) -> Workload:
    """A random but valid launch: random source format, geometry, op chain (type-correct), write kind, plane count,
    crops, sizes and pitches (aligned and unaligned).  Used to fuzz the kernels against the CPU checker."""
    rs = np.random.RandomState(seed)
    nv12 = rs.rand() < 0.3
    geometry = int(rs.choice([abi.GEOM_NONE, abi.GEOM_RESIZE_IGNORE_AR, abi.GEOM_RESIZE_PRESERVE_AR]))
    if geometry == abi.GEOM_RESIZE_PRESERVE_AR and seed % 3:  # separate generator: earlier seeds keep their launches otherwise
        geometry = (abi.GEOM_RESIZE_PRESERVE_AR, abi.GEOM_RESIZE_PRESERVE_AR_RN_EVEN, abi.GEOM_RESIZE_PRESERVE_AR_LEFT)[seed % 3]
    n_planes = int(rs.randint(1, 6))
    slots_used = 0

    def arith():
        nonlocal slots_used
        code = int(rs.choice([abi.OP_MUL, abi.OP_ADD, abi.OP_SUB, abi.OP_DIV]))
        vals = tuple(float(v) for v in (rs.uniform(0.3, 3.0, 3) if code in (abi.OP_MUL, abi.OP_DIV) else rs.uniform(-40, 40, 3)))
        if slots_used < abi.MAX_PLANE_PARAMS and rs.rand() < 0.3:
            slots_used += 1
            return op(code, slot=slots_used - 1)
        return op(code, vals)

    ops, is_f32 = [], False
    if nv12 and rs.rand() < 0.8:
        ops.append(op(abi.OP_YUV2RGB)); is_f32 = True
    elif rs.rand() < 0.4:
        ops.append(op(abi.OP_CAST_F32)); is_f32 = True
        if rs.rand() < 0.5:
            ops.append(arith())
    if rs.rand() < 0.2:
        ops.append(op(abi.OP_REORDER_ZYX))
    n_pre = len(ops) if geometry != abi.GEOM_NONE else 0
    if geometry != abi.GEOM_NONE:
        is_f32 = True
    elif not is_f32 and rs.rand() < 0.7:
        ops.append(op(abi.OP_CAST_F32)); is_f32 = True
    if is_f32:
        for _ in range(int(rs.randint(0, 4))):
            ops.append(arith() if rs.rand() < 0.8 else op(abi.OP_REORDER_ZYX))
        if rs.rand() < 0.5:
            ops.append(op(abi.OP_SATCAST_U8)); is_f32 = False
    dst_format = abi.PIX_F32C3 if is_f32 else abi.PIX_U8C3
    split = rs.rand() < 0.25
    gray = seed % 7 == 5  # a grey conversion ends the chain (decided by the seed alone: other seeds keep their launches)
    if gray:
        g = np.random.RandomState(1000 + seed)
        split = False
        if is_f32:
            ops.append(op(abi.OP_RGB2GRAY))
            if g.rand() < 0.6:
                ops.append(op(abi.OP_MUL, (float(g.uniform(0.3, 1.5)),) * 3))
            if g.rand() < 0.5:
                ops.append(op(abi.OP_SATCAST_U8)); is_f32 = False
        else:
            ops.append(op(abi.OP_RGB2GRAY, (1.0, 0.0, 0.0)))
        dst_format = abi.PIX_F32C1 if is_f32 else abi.PIX_U8C1
    ch = chain(abi.PIX_NV12 if nv12 else abi.PIX_U8C3, geometry, dst_format, abi.WRITE_SPLIT if split else abi.WRITE_PACKED,
               ops, n_pre_ops=n_pre, ccm=BT709_FULL_8BIT, yuv_sub=(0.0, 128.0, 128.0))

    w, h = int(rs.randint(2, max_dim)), int(rs.randint(2, max_dim))
    if nv12:
        w, h = w + (w & 1), h + (h & 1)
    align = int(rs.choice([1, 4, 16, 64, 512]))
    src4 = not nv12 and seed % 5 == 3  # a uchar4 source whose alpha is discarded (decided by the seed alone: other seeds keep their launches)
    if src4:
        ch.src_format = abi.PIX_U8C4
    pitch = _pitch(w if nv12 else w * (4 if src4 else 3), max(align, 2 if nv12 else 1))
    src = _frame(seed + 7, pitch * (h + h // 2 if nv12 else h), 16 if nv12 else 0, 236 if nv12 else 256)
    elt = {abi.PIX_F32C3: 4 if split else 12, abi.PIX_U8C3: 1 if split else 3, abi.PIX_F32C1: 4, abi.PIX_U8C1: 1}[dst_format]
    dalign = int(rs.choice([1, 16, 64])) if dst_format in (abi.PIX_U8C3, abi.PIX_U8C1) else int(rs.choice([4, 16, 64]))
    planes, off = [], 0
    for _ in range(n_planes):
        cw, chh = int(rs.randint(1, w + 1)), int(rs.randint(1, h + 1))
        cx, cy = int(rs.randint(0, w - cw + 1)), int(rs.randint(0, h - chh + 1))
        if rs.rand() < 0.3:
            cx -= cx % 16
        if geometry == abi.GEOM_NONE:
            dw, dh = cw, chh
        else:
            dw, dh = int(rs.randint(1, max_dim)), int(rs.randint(1, max_dim))
        dpitch = _pitch(dw * elt, dalign)
        plane_bytes = dpitch * dh
        cstride = _pitch(plane_bytes, 16) if split else 0
        total = cstride * 3 if split else plane_bytes
        params = tuple(tuple(float(v) for v in rs.uniform(0.5, 2.5, 3)) for _ in range(slots_used))
        planes.append(PlaneSpec(0, 0, off, w, h, pitch, (cx, cy, cw, chh), dw, dh, dpitch, dst_channel_stride=cstride,
                                bg=tuple(float(v) for v in rs.uniform(0, 255, 3)), params=params,
                                chroma_offset=pitch * h))
        off += _pitch(total, int(rs.choice([4, 16, 256])))
    return Workload(f"random_{seed}", [ch], [src], [off], planes, "random launch")


# ---------------------------------------------------------------------------------------------------------------
# CircularTensor::update (core/data/circular_tensor.h:111-161) as one divergent launch
# ---------------------------------------------------------------------------------------------------------------
def circular_update_launch(kind, oldest_first, first, batch, frame_addr, frame_w, frame_h, frame_pitch, dw, dh, mul, temp_addr, out_addr):
    """Descriptors of one update of a circular tensor of ``batch`` planes of dw x dh float pixels.

    kind 0: packed float3 planes (TensorWrite<float3>); 1: planar channels per plane (TensorSplit<float3>); 2: the
    colour-plane-transposed tensor (TensorTSplit<float3>).  The update sequence (frame -> Resize IGNORE_AR -> Mul -> write)
    runs twice: into plane ``first``-derived of the temporary tensor (the reference's mid-chain CircularTensorWrite) and into
    its plane of the output; the copy sequence moves the other batch - 1 planes from the temporary tensor to the output in
    circular order.  Returns (chain array, plane array, next ``first``)."""
    packed = kind == 0
    px = dw * dh
    if packed:
        plane_step, chan_step, pitch, wk, copy_src = px * 12, 0, dw * 12, abi.WRITE_PACKED, abi.PIX_F32C3
    elif kind == 1:
        plane_step, chan_step, pitch, wk, copy_src = px * 12, px * 4, dw * 4, abi.WRITE_SPLIT, abi.PIX_F32P3
    else:
        plane_step, chan_step, pitch, wk, copy_src = px * 4, px * 4 * batch, dw * 4, abi.WRITE_SPLIT, abi.PIX_F32P3
    update = chain(abi.PIX_U8C3, abi.GEOM_RESIZE_IGNORE_AR, abi.PIX_F32C3, wk, [op(abi.OP_MUL, mul)])
    copy = chain(copy_src, abi.GEOM_NONE, abi.PIX_F32C3, wk, [])
    chains = (abi.ChainDesc * 2)(update, copy)
    lib = abi.load()
    planes = []

    def dst(d, base, z):
        d.dst = base + z * plane_step
        d.dst_w, d.dst_h, d.dst_pitch, d.dst_channel_stride = dw, dh, pitch, chan_step

    # where the new image goes: (z + first) mod batch in the temporary tensor, z in the output (z = the update sequence's plane)
    zu = batch - 1 if oldest_first else 0
    for base, z in ((temp_addr, (zu + first) % batch), (out_addr, zu)):
        d = abi.PlaneDesc()
        d.src, d.src_pitch, d.src_w, d.src_h = frame_addr, frame_pitch, frame_w, frame_h
        d.crop_x, d.crop_y, d.crop_w, d.crop_h = 0, 0, frame_w, frame_h
        dst(d, base, z)
        d.chain = 0
        lib.fkb_resize_params(abi.GEOM_RESIZE_IGNORE_AR, C.byref(d))
        planes.append(d)
    for z in range(batch):
        if z == zu:
            continue
        zs = (z + first) % batch if oldest_first else (first - z) % batch  # Ascendent / Descendent read (memory_operations.h:423-431)
        d = abi.PlaneDesc()
        d.src = temp_addr + zs * plane_step
        d.src_chroma = d.src + chan_step if not packed else None
        d.src_pitch, d.src_w, d.src_h = pitch, dw, dh
        d.crop_x, d.crop_y, d.crop_w, d.crop_h = 0, 0, dw, dh
        dst(d, out_addr, z)
        d.chain = 1
        planes.append(d)
    arr = (abi.PlaneDesc * len(planes))(*planes)
    return chains, arr, (first + 1) % batch
