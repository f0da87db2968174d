// TEST INFRASTRUCTURE — not part of the product.  Only tests/, the smoke check and the benchmark's CPU
// baseline may load this file's library; the CUDA path never does.
//
// A plain, scalar CPU restatement of the arithmetic the FusedKernelLibrary CPU backend performs for a
// fused TransformDPP chain, driven by the same descriptors the CUDA kernels take (include/fkb/fkb.h).
// Parity status: PINNED.  It is checked bit-for-bit against (1) the reference's own golden values
// (saturate rounding, BGR<->RGB reorder, bt709 matrix constants) and (2) the outputs of the reference
// CPU backend itself, compiled from the reference headers by oracle/ref_runner.cpp, on every benchmark
// configuration and on the fixtures under tests/golden/.
//
// Must be compiled with -O2 -ffp-contract=off and without -march=native: an FMA contraction changes the
// results (also the reference's own).
//
// Reference lines restated (paths relative to the reference's include/fused_kernel/):
//   loop nest z,y,x ............... core/execution_model/data_parallel_patterns.h:271-283
//   divergent chain selection ...... core/execution_model/data_parallel_patterns.h:322-331
//   batch plane selection .......... core/execution_model/operation_model/batch_operations.h:205-212
//   uchar3 read, pitched ........... algorithms/basic_ops/memory_operations.h:34-38, core/data/rawptr.h:203-213
//   NV12 read ...................... algorithms/image_processing/color_conversion.h:219-238
//   crop ........................... algorithms/image_processing/crop.h:36-39
//   resize (host parameters) ....... algorithms/image_processing/resize.h:164-233, 266-278
//   resize (per pixel) ............. algorithms/image_processing/resize.h:86-98, 117-123
//   bilinear interpolation ......... algorithms/image_processing/interpolation.h:70-104
//   YCbCr -> RGB ................... algorithms/image_processing/color_conversion.h:150-174,
//                                    algorithms/basic_ops/algebraic.h:42-56,
//                                    core/constexpr_libs/constexpr_vector_exec.h:66-78 (sum order)
//   Mul/Add/Sub/Div ................ algorithms/basic_ops/arithmetic.h:23-137
//   Cast ........................... algorithms/basic_ops/cast.h:22-33
//   channel reorder ................ algorithms/basic_ops/vector_ops.h:43-56
//   saturate cast .................. core/constexpr_libs/constexpr_saturate.h:28-150
//   writes ......................... algorithms/basic_ops/memory_operations.h:92-97, 167-170, 189-205
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "fkb/fkb.h"

namespace {

struct V3 {
    float c[4] = {0.f, 0.f, 0.f, 0.f};  // three channels, or four for the chains that keep the alpha channel (the fourth is ignored otherwise)
};
// channels a chain carries: four when its destination is uchar4 / float4
inline int channels(const fkb_chain_desc& ch) { return (ch.dst_format == FKB_PIX_U8C4 || ch.dst_format == FKB_PIX_F32C4) ? 4 : 3; }

// round-half-away-from-zero, as cxp::round (core/constexpr_libs/constexpr_cmath.h:354-385)
inline float round_half_away(float v) {
    if (v != v || v == 0.f) return v;
    const float a = v < 0.f ? -v : v;
    if (a >= 8388608.0f) return v;  // already integral
    const float t = static_cast<float>(static_cast<int>(a));
    const float r = (a - t) >= 0.5f ? t + 1.f : t;
    return v < 0.f ? -r : r;
}

// SaturateCast<float,uchar>: NaN -> 0, ties to even, clamp to [0,255]
// (constexpr_saturate.h:28-66 banker_round, 97-117 clamp)
inline uint8_t sat_u8(float s) {
    if (s != s) return 0;
    const bool neg = s < 0.f;
    const float a = neg ? -s : s;
    float rounded;
    if (a >= 9007199254740992.0f) {
        rounded = s;
    } else {
        long long i = static_cast<long long>(a);
        const float diff = a - static_cast<float>(i);
        if (diff > 0.5f) {
            i += 1;
        } else if (diff >= 0.5f) {
            if (i % 2 != 0) i += 1;
        }
        const float r = static_cast<float>(i);
        rounded = neg ? -r : r;
    }
    if (rounded >= 255.f) return 255;
    if (rounded <= 0.f) return 0;
    return static_cast<uint8_t>(rounded);
}

inline void operand(const fkb_chain_desc& ch, uint32_t i, const fkb_plane_desc& pl, float o[4]) {
    const fkb_op& op = ch.ops[i];
    const float* s = op.plane_slot >= 0 ? pl.params[op.plane_slot] : op.v;
    o[0] = s[0]; o[1] = s[1]; o[2] = s[2];
    o[3] = op.plane_slot >= 0 ? pl.params_w[op.plane_slot] : ch.op_w[i];
}

inline V3 apply_ops(V3 v, const fkb_chain_desc& ch, const fkb_plane_desc& pl, uint32_t first, uint32_t last) {
    for (uint32_t i = first; i < last; ++i) {
        const fkb_op& op = ch.ops[i];
        const int nc = channels(ch);
        float p[4];
        switch (op.code) {
        case FKB_OP_CAST_F32:  // static_cast<float>(uchar): exact
            break;
        case FKB_OP_MUL: operand(ch, i, pl, p); for (int c = 0; c < nc; ++c) v.c[c] = v.c[c] * p[c]; break;
        case FKB_OP_ADD: operand(ch, i, pl, p); for (int c = 0; c < nc; ++c) v.c[c] = v.c[c] + p[c]; break;
        case FKB_OP_SUB: operand(ch, i, pl, p); for (int c = 0; c < nc; ++c) v.c[c] = v.c[c] - p[c]; break;
        case FKB_OP_DIV: operand(ch, i, pl, p); for (int c = 0; c < nc; ++c) v.c[c] = v.c[c] / p[c]; break;
        case FKB_OP_REORDER_ZYX: { const float t = v.c[0]; v.c[0] = v.c[2]; v.c[2] = t; break; }
        case FKB_OP_YUV2RGB: {
            const float a = v.c[0] - ch.yuv_sub[0], b = v.c[1] - ch.yuv_sub[1], d = v.c[2] - ch.yuv_sub[2];
            V3 r;
            for (int c = 0; c < 3; ++c)
                r.c[c] = ((a * ch.ccm[3 * c + 0]) + (b * ch.ccm[3 * c + 1])) + (d * ch.ccm[3 * c + 2]);
            v = r;
            break;
        }
        case FKB_OP_RGB2YUV: {  // ConvertRGBToYUV::exec (color_conversion.h:188-198): matrix, then the offsets
            V3 r;
            for (int c = 0; c < 3; ++c) {
                const float y = ((v.c[0] * ch.ccm2[3 * c + 0]) + (v.c[1] * ch.ccm2[3 * c + 1])) + (v.c[2] * ch.ccm2[3 * c + 2]);
                r.c[c] = ch.yuv_add[c] != 0.f ? y + ch.yuv_add[c] : y;  // Full range: the luma is returned as computed
            }
            v = r;
            break;
        }
        case FKB_OP_SATCAST_U8:
            for (int c = 0; c < nc; ++c) v.c[c] = static_cast<float>(sat_u8(v.c[c]));
            break;
        case FKB_OP_RGB2GRAY: {  // RGB2Gray<I,O,CCIR_601>::exec (color_conversion.h:57-78): luminance, then std::nearbyint — also
                                 // for O = float, because std::is_signed_v<float> is true and that branch comes first (:65-70)
            const float l = (v.c[0] * 0.299f) + (v.c[1] * 0.587f) + (v.c[2] * 0.114f);
            v.c[0] = std::nearbyint(l);
            break;
        }
        case FKB_OP_ADD_ALPHA:  // AddOpaqueAlpha::exec (color_conversion.h:89-92): the input's channels, then maxDepthValue<CD>
            v.c[3] = op.v[0];
            break;
        default: break;
        }
    }
    return v;
}

// Read of frame pixel (X,Y).
inline V3 read_frame(const fkb_chain_desc& ch, const fkb_plane_desc& pl, size_t X, size_t Y) {
    const uint8_t* base = static_cast<const uint8_t*>(pl.src);
    V3 v;
    if (ch.src_format == FKB_PIX_NV12) {
        const uint8_t* uv = static_cast<const uint8_t*>(pl.src_chroma) + (Y >> 1) * pl.src_pitch + (X >> 1) * 2;
        v.c[0] = base[Y * pl.src_pitch + X];
        v.c[1] = uv[0];
        v.c[2] = uv[1];
    } else if (ch.src_format == FKB_PIX_NV21) {  // color_conversion.h:240-254: the pair is (V,U)
        const uint8_t* vu = static_cast<const uint8_t*>(pl.src_chroma) + (Y >> 1) * pl.src_pitch + (X >> 1) * 2;
        v.c[0] = base[Y * pl.src_pitch + X];
        v.c[1] = vu[1];
        v.c[2] = vu[0];
    } else if (ch.src_format == FKB_PIX_UYVY) {  // color_conversion.h:255-265: one uchar4 (U, Y0, V, Y1) per two pixels
        const uint8_t* g = base + Y * pl.src_pitch + (X >> 1) * 4;
        v.c[0] = (X & 1) ? g[3] : g[1];
        v.c[1] = g[0];
        v.c[2] = g[2];
    } else if (ch.src_format == FKB_PIX_P010 || ch.src_format == FKB_PIX_P210) {  // color_conversion.h:219-238, ushort samples
        const size_t cy = ch.src_format == FKB_PIX_P010 ? (Y >> 1) : Y;             // 4:2:0 halves the chroma rows, 4:2:2 does not
        const uint16_t* uv = reinterpret_cast<const uint16_t*>(static_cast<const uint8_t*>(pl.src_chroma) + cy * pl.src_pitch) + (X >> 1) * 2;
        v.c[0] = reinterpret_cast<const uint16_t*>(base + Y * pl.src_pitch)[X];
        v.c[1] = uv[0];
        v.c[2] = uv[1];
    } else if (ch.src_format == FKB_PIX_Y210) {  // color_conversion.h:255-265: ushort4 (Y0, U, Y1, V) per two pixels
        const uint16_t* g = reinterpret_cast<const uint16_t*>(base + Y * pl.src_pitch) + (X >> 1) * 4;
        v.c[0] = (X & 1) ? g[2] : g[0];
        v.c[1] = g[1];
        v.c[2] = g[3];
    } else if (ch.src_format == FKB_PIX_F32C3) {  // TensorRead<float3> / PerThreadRead<float3>
        const float* p = reinterpret_cast<const float*>(base + Y * pl.src_pitch) + X * 3;
        v.c[0] = p[0]; v.c[1] = p[1]; v.c[2] = p[2];
    } else if (ch.src_format == FKB_PIX_F32P3) {  // TensorPack / TensorTPack: one float plane per channel
        const size_t step = static_cast<size_t>(static_cast<const uint8_t*>(pl.src_chroma) - base);
        const uint8_t* p = base + Y * pl.src_pitch + X * 4;
        v.c[0] = *reinterpret_cast<const float*>(p); v.c[1] = *reinterpret_cast<const float*>(p + step);
        v.c[2] = *reinterpret_cast<const float*>(p + 2 * step);
    } else if (ch.src_format == FKB_PIX_U8C4) {  // uchar4 whose alpha is discarded (Discard<uchar4,uchar3>, color_conversion.h:448-452)
        const uint8_t* p = base + Y * pl.src_pitch + X * 4;
        v.c[0] = p[0]; v.c[1] = p[1]; v.c[2] = p[2]; v.c[3] = p[3];
    } else {
        const uint8_t* p = base + Y * pl.src_pitch + X * 3;
        v.c[0] = p[0]; v.c[1] = p[1]; v.c[2] = p[2];
    }
    return v;
}

// BorderReader index maps (border_reader.h:211-330): idx = low(high(i)), written out per mode.  `n` is the extent of
// the back operation along the axis (last = n - 1).
inline int border_index(uint32_t mode, int i, int n) {
    const int last = n - 1;
    switch (mode) {
    case FKB_BORDER_REPLICATE: {                     // :211-232
        const int hi = i < last ? i : last;
        return hi > 0 ? hi : 0;
    }
    case FKB_BORDER_REFLECT: {                       // :234-256
        const int hi = last - std::abs(last - i) + (i > last ? 1 : 0);
        return (std::abs(hi) - (hi < 0 ? 1 : 0)) % (last + 1);
    }
    case FKB_BORDER_WRAP: {                          // :258-287
        const int hi = i < n ? i : i % n;
        return hi >= 0 ? hi : hi - ((hi - n + 1) / n) * n;
    }
    case FKB_BORDER_REFLECT_101: {                   // :289-311
        const int hi = std::abs(last - std::abs(last - i)) % (last + 1);
        return std::abs(hi) % (last + 1);
    }
    default: return i;
    }
}

// Value of crop-relative pixel (cx,cy) after ops[0..n_tap_ops): Crop adds the rectangle origin as signed integers
// (crop.h:36-39); a BorderReader, if the chain has one, sits between the first border_at ops and the Crop
// (border_reader.h:177-209 for CONSTANT, :166-172 for the index-mapping modes).
inline V3 tap(const fkb_chain_desc& ch, const fkb_plane_desc& pl, int cx, int cy, uint32_t n_tap_ops) {
    const int X = cx + static_cast<int>(pl.crop_x), Y = cy + static_cast<int>(pl.crop_y);
    if (ch.border == FKB_BORDER_NONE)
        return apply_ops(read_frame(ch, pl, static_cast<size_t>(X), static_cast<size_t>(Y)), ch, pl, 0, n_tap_ops);
    const int w = static_cast<int>(pl.src_w), h = static_cast<int>(pl.src_h);
    if (ch.border == FKB_BORDER_CONSTANT) {
        V3 v;
        if (X >= 0 && X < w && Y >= 0 && Y < h) {
            v = apply_ops(read_frame(ch, pl, static_cast<size_t>(X), static_cast<size_t>(Y)), ch, pl, 0, ch.border_at);
        } else {
            v.c[0] = ch.border_value[0]; v.c[1] = ch.border_value[1]; v.c[2] = ch.border_value[2]; v.c[3] = ch.border_value_w;
        }
        return apply_ops(v, ch, pl, ch.border_at, n_tap_ops);
    }
    const int bx = border_index(ch.border, X, w), by = border_index(ch.border, Y, h);
    return apply_ops(read_frame(ch, pl, static_cast<size_t>(bx), static_cast<size_t>(by)), ch, pl, 0, n_tap_ops);
}

inline V3 pixel(const fkb_chain_desc& ch, const fkb_plane_desc& pl, int x, int y) {
    if (pl.chain & FKB_PLANE_DEFAULT) {
        // a plane beyond usedPlanes of BatchRead<CONDITIONAL_WITH_DEFAULT> (batch_operations.h:262-266): the read —
        // including a Resize fused into it (iop_fuser.h:71-88) — yields the default value; the later ops still run
        V3 d;
        d.c[0] = pl.bg[0]; d.c[1] = pl.bg[1]; d.c[2] = pl.bg[2]; d.c[3] = pl.bg_w;
        return apply_ops(d, ch, pl, ch.geometry == FKB_GEOM_NONE ? 0 : ch.n_pre_ops, ch.n_ops);
    }
    if (ch.geometry == FKB_GEOM_NONE) {
        return tap(ch, pl, x, y, ch.n_ops);
    }
    V3 v;
    int tx = x, ty = y;
    bool inside = true;
    if (ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR) {
        inside = x >= pl.x1 && x <= pl.x2 && y >= pl.y1 && y <= pl.y2;
        tx = x - pl.x1; ty = y - pl.y1;
    }
    if (!inside) {
        v.c[0] = pl.bg[0]; v.c[1] = pl.bg[1]; v.c[2] = pl.bg[2]; v.c[3] = pl.bg_w;
    } else {
        const float sx = tx * pl.fx, sy = ty * pl.fy;
        int x1 = static_cast<int>(std::floor(sx)), y1 = static_cast<int>(std::floor(sy));
        const int x2 = x1 + 1, y2 = y1 + 1;
        const int x2r = x2 < pl.crop_w - 1 ? x2 : pl.crop_w - 1, y2r = y2 < pl.crop_h - 1 ? y2 : pl.crop_h - 1;
        // The reference reads x1,y1 unclamped; they stay inside the crop for every sane scale.  Clamp the
        // address only (weights still use the unclamped values) so a degenerate scale cannot read outside.
        const int x1r = x1 < pl.crop_w - 1 ? x1 : pl.crop_w - 1, y1r = y1 < pl.crop_h - 1 ? y1 : pl.crop_h - 1;
        const V3 p00 = tap(ch, pl, x1r, y1r, ch.n_pre_ops);
        const V3 p10 = tap(ch, pl, x2r, y1r, ch.n_pre_ops);
        const V3 p01 = tap(ch, pl, x1r, y2r, ch.n_pre_ops);
        const V3 p11 = tap(ch, pl, x2r, y2r, ch.n_pre_ops);
        const float w00 = (x2 - sx) * (y2 - sy), w10 = (sx - x1) * (y2 - sy);
        const float w01 = (x2 - sx) * (sy - y1), w11 = (sx - x1) * (sy - y1);
        for (int c = 0; c < channels(ch); ++c)
            v.c[c] = (p00.c[c] * w00) + (p10.c[c] * w10) + (p01.c[c] * w01) + (p11.c[c] * w11);
    }
    return apply_ops(v, ch, pl, ch.n_pre_ops, ch.n_ops);
}

void run_plane(const fkb_chain_desc& ch, const fkb_plane_desc& pl) {
    uint8_t* dst = static_cast<uint8_t*>(pl.dst);
    for (uint32_t y = 0; y < pl.dst_h; ++y) {
        for (uint32_t x = 0; x < pl.dst_w; ++x) {
            const V3 v = pixel(ch, pl, static_cast<int>(x), static_cast<int>(y));
            uint8_t* row = dst + static_cast<size_t>(y) * pl.dst_pitch;
            if (ch.dst_format == FKB_PIX_U8C1) {  // PerThreadWrite / TensorWrite of uchar: the one channel a gray conversion leaves
                row[x] = static_cast<uint8_t>(v.c[0]);
            } else if (ch.dst_format == FKB_PIX_F32C1) {
                reinterpret_cast<float*>(row)[x] = v.c[0];
            } else if (channels(ch) == 4) {  // PerThreadWrite / TensorWrite of uchar4 or float4
                if (ch.dst_format == FKB_PIX_F32C4) {
                    float* q = reinterpret_cast<float*>(row) + static_cast<size_t>(x) * 4;
                    for (int c = 0; c < 4; ++c) q[c] = v.c[c];
                } else {
                    uint8_t* q = row + static_cast<size_t>(x) * 4;
                    for (int c = 0; c < 4; ++c) q[c] = static_cast<uint8_t>(v.c[c]);
                }
            } else if (ch.write_kind >= FKB_WRITE_NV12) {  // WriteYUV::exec (color_conversion.h:309-383)
                const uint8_t yy = static_cast<uint8_t>(v.c[0]), cb = static_cast<uint8_t>(v.c[1]), cr = static_cast<uint8_t>(v.c[2]);
                if (ch.write_kind == FKB_WRITE_UYVY) {
                    uint8_t* g = row + static_cast<size_t>(x >> 1) * 4;
                    if (x & 1u) g[3] = yy; else { g[0] = cb; g[1] = yy; g[2] = cr; }
                } else {
                    row[x] = yy;
                    uint8_t* uv = static_cast<uint8_t*>(pl.dst_y) + static_cast<size_t>(y >> 1) * pl.dst_pitch + static_cast<size_t>(x >> 1) * 2;
                    if (ch.write_kind == FKB_WRITE_NV12) {
                        if (!(x & 1u) && !(y & 1u)) { uv[0] = cb; uv[1] = cr; }
                    } else {
                        // NV21: every pixel stores its (Cr,Cb) pair; this loop visits pixels in raster order, as the
                        // reference's CPU backend does, so the last pixel of each 2x2 block is what stays
                        uv[0] = cr; uv[1] = cb;
                    }
                }
            } else if (ch.write_kind == FKB_WRITE_SPLIT_PLANES) {  // SplitWrite (memory_operations.h:360-393): one RawPtr per channel
                uint8_t* const base[3] = {dst, static_cast<uint8_t*>(pl.dst_y), static_cast<uint8_t*>(pl.dst_z)};
                for (int c = 0; c < 3; ++c) {
                    uint8_t* q = base[c] + static_cast<size_t>(y) * pl.dst_pitch;
                    if (ch.dst_format == FKB_PIX_F32C3) reinterpret_cast<float*>(q)[x] = v.c[c];
                    else q[x] = static_cast<uint8_t>(v.c[c]);
                }
            } else if (ch.write_kind == FKB_WRITE_SPLIT) {
                for (int c = 0; c < 3; ++c) {
                    uint8_t* q = row + static_cast<size_t>(c) * pl.dst_channel_stride;
                    if (ch.dst_format == FKB_PIX_F32C3) reinterpret_cast<float*>(q)[x] = v.c[c];
                    else q[x] = static_cast<uint8_t>(v.c[c]);
                }
            } else if (ch.dst_format == FKB_PIX_F32C3) {
                float* q = reinterpret_cast<float*>(row) + static_cast<size_t>(x) * 3;
                q[0] = v.c[0]; q[1] = v.c[1]; q[2] = v.c[2];
            } else {
                uint8_t* q = row + static_cast<size_t>(x) * 3;
                q[0] = static_cast<uint8_t>(v.c[0]); q[1] = static_cast<uint8_t>(v.c[1]); q[2] = static_cast<uint8_t>(v.c[2]);
            }
        }
    }
}

}  // namespace

extern "C" {

// Resize<INTER_LINEAR,AR>::build host arithmetic (resize.h:164-205, 208-233, 266-278).
int fkb_oracle_resize_params(uint32_t geometry, fkb_plane_desc* pl) {
    const int sw = pl->crop_w, sh = pl->crop_h, dw = static_cast<int>(pl->dst_w), dh = static_cast<int>(pl->dst_h);
    if (sw <= 0 || sh <= 0 || dw <= 0 || dh <= 0) return FKB_ERR_INVALID;
    if (geometry == FKB_GEOM_RESIZE_IGNORE_AR) {
        const double cfx = static_cast<double>(dw) / static_cast<double>(sw);
        const double cfy = static_cast<double>(dh) / static_cast<double>(sh);
        pl->fx = static_cast<float>(1.0 / cfx);
        pl->fy = static_cast<float>(1.0 / cfy);
        pl->x1 = 0; pl->y1 = 0; pl->x2 = dw - 1; pl->y2 = dh - 1;
        return FKB_OK;
    }
    if (geometry < FKB_GEOM_RESIZE_PRESERVE_AR || geometry > FKB_GEOM_RESIZE_PRESERVE_AR_LEFT) return FKB_ERR_INVALID;
    // compute_target_size (resize.h:206-233); RN_EVEN (resize.h:212-222) evens the fitted dimension
    const bool even = geometry == FKB_GEOM_RESIZE_PRESERVE_AR_RN_EVEN;
    const float scale = dh / static_cast<float>(sh);
    int tw = static_cast<int>(round_half_away(scale * sw)), th = dh;
    if (even) tw = tw - (tw % 2);
    if (tw > dw) {
        const float scale2 = dw / static_cast<float>(sw);
        tw = dw;
        th = static_cast<int>(round_half_away(scale2 * sh));
        if (even) th = th - (th % 2);
    }
    const double cfx = static_cast<double>(tw) / sw, cfy = static_cast<double>(th) / sh;
    pl->fx = static_cast<float>(1.0 / cfx);
    pl->fy = static_cast<float>(1.0 / cfy);
    pl->x1 = geometry == FKB_GEOM_RESIZE_PRESERVE_AR_LEFT ? 0 : (dw - tw) / 2;  // resize.h:176-178
    pl->y1 = (dh - th) / 2;
    pl->x2 = pl->x1 + tw - 1;
    pl->y2 = pl->y1 + th - 1;
    return FKB_OK;
}

// ccMatrix<CR, CP, YCbCr2RGB, p8bit> and subCoefficients<p8bit> (itu_color.h:112-124, 142-153, 185-258), with the
// luma offset dropped for Full range as ConvertYUVToRGB::exec does (color_conversion.h:163-171).
int fkb_oracle_ycbcr_to_rgb_bits(uint32_t bits, uint32_t range, uint32_t primitives, float* ccm, float* yuv_sub);
int fkb_oracle_ycbcr_to_rgb(uint32_t range, uint32_t primitives, float* ccm, float* yuv_sub) {
    return fkb_oracle_ycbcr_to_rgb_bits(8, range, primitives, ccm, yuv_sub);
}
int fkb_oracle_ycbcr_to_rgb_bits(uint32_t bits, uint32_t range, uint32_t primitives, float* ccm, float* yuv_sub) {
    // maxDepthValue (itu_color.h:104-110), subCoefficients (:119-124), rangeLimits (:160-165) of the integer depths
    float max_v, sub_y, sub_c, lim_y, lim_c;
    switch (bits) {
    case 8: max_v = 255.f; sub_y = 16.f; sub_c = 128.f; lim_y = 219.f; lim_c = 224.f; break;
    case 10: max_v = 1023.f; sub_y = 64.f; sub_c = 512.f; lim_y = 876.f; lim_c = 896.f; break;
    case 12: max_v = 4095.f; sub_y = 256.f; sub_c = 2048.f; lim_y = 3504.f; lim_c = 3584.f; break;
    default: return FKB_ERR_INVALID;
    }
    float kr, kb;
    switch (primitives) {
    case FKB_PRIMITIVES_BT601: kr = 0.299f; kb = 0.114f; break;
    case FKB_PRIMITIVES_BT709: kr = 0.2126f; kb = 0.0722f; break;
    case FKB_PRIMITIVES_BT2020: kr = 0.2627f; kb = 0.0593f; break;
    default: return FKB_ERR_INVALID;
    }
    const float kg = 1.0f - kr - kb;
    ccm[0] = 1.0f; ccm[1] = 0.0f; ccm[2] = 2.0f * (1.0f - kr);
    ccm[3] = 1.0f; ccm[4] = -2.0f * kb * (1.0f - kb) / kg; ccm[5] = -2.0f * kr * (1.0f - kr) / kg;
    ccm[6] = 1.0f; ccm[7] = 2.0f * (1.0f - kb); ccm[8] = 0.0f;
    if (range == FKB_RANGE_LIMITED) {
        const float sy = max_v / lim_y, sc = max_v / lim_c;
        for (int r = 0; r < 3; ++r) { ccm[3 * r] *= sy; ccm[3 * r + 1] *= sc; ccm[3 * r + 2] *= sc; }
    } else if (range != FKB_RANGE_FULL) {
        return FKB_ERR_INVALID;
    }
    yuv_sub[0] = range == FKB_RANGE_LIMITED ? sub_y : 0.f;
    yuv_sub[1] = sub_c; yuv_sub[2] = sub_c;
    return FKB_OK;
}

// ccMatrix<CR, CP, RGB2YCbCr, p8bit> (itu_color.h:193-218) and the offsets ConvertRGBToYUV adds (color_conversion.h:191-197).
int fkb_oracle_rgb_to_ycbcr(uint32_t range, uint32_t primitives, float* ccm2, float* yuv_add) {
    float kr, kb;
    switch (primitives) {
    case FKB_PRIMITIVES_BT601: kr = 0.299f; kb = 0.114f; break;
    case FKB_PRIMITIVES_BT709: kr = 0.2126f; kb = 0.0722f; break;
    case FKB_PRIMITIVES_BT2020: kr = 0.2627f; kb = 0.0593f; break;
    default: return FKB_ERR_INVALID;
    }
    const float kg = 1.0f - kr - kb;
    ccm2[0] = kr; ccm2[1] = kg; ccm2[2] = kb;
    ccm2[3] = -kr / (2.0f * (1.0f - kb)); ccm2[4] = -kg / (2.0f * (1.0f - kb)); ccm2[5] = 0.5f;
    ccm2[6] = 0.5f; ccm2[7] = -kg / (2.0f * (1.0f - kr)); ccm2[8] = -kb / (2.0f * (1.0f - kr));
    if (range == FKB_RANGE_LIMITED) {
        const float sy = 219.f / 255.f, sc = 224.f / 255.f;
        for (int i = 0; i < 3; ++i) { ccm2[i] *= sy; ccm2[3 + i] *= sc; ccm2[6 + i] *= sc; }
    } else if (range != FKB_RANGE_FULL) {
        return FKB_ERR_INVALID;
    }
    yuv_add[0] = range == FKB_RANGE_LIMITED ? 16.f : 0.f;
    yuv_add[1] = 128.f; yuv_add[2] = 128.f;
    return FKB_OK;
}

// Runs the launch on host memory: every src/dst pointer in `planes` is a host address.
// n_threads > 1 splits the planes over std::threads (planes are independent); results do not depend on it.
int fkb_oracle_run(const fkb_chain_desc* chains, uint32_t n_chains, const fkb_plane_desc* planes,
                   uint32_t n_planes, uint32_t n_threads) {
    if (!chains || !planes) return FKB_ERR_NULL;
    for (uint32_t z = 0; z < n_planes; ++z)
        if ((planes[z].chain & ~FKB_PLANE_DEFAULT) >= n_chains) return FKB_ERR_INVALID;
    if (n_threads <= 1 || n_planes <= 1) {
        for (uint32_t z = 0; z < n_planes; ++z) run_plane(chains[planes[z].chain & ~FKB_PLANE_DEFAULT], planes[z]);
        return FKB_OK;
    }
    if (n_threads > n_planes) n_threads = n_planes;
    std::vector<std::thread> pool;
    for (uint32_t t = 0; t < n_threads; ++t)
        pool.emplace_back([=] {
            for (uint32_t z = t; z < n_planes; z += n_threads) run_plane(chains[planes[z].chain & ~FKB_PLANE_DEFAULT], planes[z]);
        });
    for (auto& th : pool) th.join();
    return FKB_OK;
}

// Single scalar helpers exported for the golden-value tests.
uint8_t fkb_oracle_saturate_u8(float v) { return sat_u8(v); }
float fkb_oracle_round_half_away(float v) { return round_half_away(v); }

}  // extern "C"
