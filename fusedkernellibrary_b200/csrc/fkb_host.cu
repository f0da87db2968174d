// Host side of the C ABI (include/fkb/fkb.h): descriptor validation, lowering of a launch to plane records
// and a tile schedule, the descriptor arena, plans, and the entry points themselves.
//
// Reference behaviour mirrored here (paths relative to the reference's include/fused_kernel/):
//   * executeOperations is asynchronous on the caller's stream, never synchronises, and reports launch
//     errors right after the launch (core/execution_model/executors.h:316-351).  The reference throws
//     std::runtime_error (core/utils/utils.h:100-114); a C ABI cannot, so every entry point returns a status.
//   * Output geometry is the ActiveThreads of the first IOp (executors.h:316-329); here it is dst_w x dst_h of
//     each plane.
//   * Resize<>::build computes its parameters on the host in double and stores floats
//     (algorithms/image_processing/resize.h:164-233, 266-278): fkb_resize_params.
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "fkb_device.cuh"
#include "fkb_launch.h"

namespace fkb {
namespace {

thread_local int t_last_cuda_error = 0;

// An NVTX range around the host side of an entry point (the reference wraps its tests in NVTX ranges behind ENABLE_NVTX,
// tests/nvtx.h:18-104): visible in a timeline profiler, a few nanoseconds when no tool is attached.
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};

#define FKB_CUDA(expr)                                              \
    do {                                                            \
        const cudaError_t e_ = (expr);                              \
        if (e_ != cudaSuccess) {                                    \
            t_last_cuda_error = static_cast<int>(e_);               \
            (void)cudaGetLastError();                               \
            return FKB_ERR_CUDA;                                    \
        }                                                           \
    } while (0)

enum ValueType { VT_U8 = 0, VT_F32 = 1 };

// -------------------------------------------------------------------------------------------------------
// validation
// -------------------------------------------------------------------------------------------------------
int check_ops(const fkb_chain_desc& ch, uint32_t first, uint32_t last, ValueType& t) {
    for (uint32_t i = first; i < last; ++i) {
        const fkb_op& op = ch.ops[i];
        if (op.plane_slot >= static_cast<int>(FKB_MAX_PLANE_PARAMS) || op.plane_slot < -1) return FKB_ERR_INVALID;
        switch (op.code) {
        case FKB_OP_CAST_F32: if (t != VT_U8) return FKB_ERR_INVALID; t = VT_F32; break;
        case FKB_OP_MUL: case FKB_OP_ADD: case FKB_OP_SUB: case FKB_OP_DIV: if (t != VT_F32) return FKB_ERR_INVALID; break;
        case FKB_OP_REORDER_ZYX: break;
        case FKB_OP_YUV2RGB: case FKB_OP_RGB2YUV: if (t != VT_U8) return FKB_ERR_INVALID; t = VT_F32; break;
        case FKB_OP_SATCAST_U8: if (t != VT_F32) return FKB_ERR_INVALID; t = VT_U8; break;
        case FKB_OP_ADD_ALPHA: break;  // uchar3 -> uchar4 or float3 -> float4; check_chain counts it
        case FKB_OP_RGB2GRAY:          // uchar3 -> uchar (rounded) or float3 -> float; check_chain counts it and checks what follows
            if (op.v[0] != 0.f) { if (t != VT_U8) return FKB_ERR_INVALID; }
            else t = VT_F32;
            break;
        default: return FKB_ERR_UNSUPPORTED;
        }
    }
    return FKB_OK;
}

int check_chain(const fkb_chain_desc& ch) {
    const bool float_src = ch.src_format == FKB_PIX_F32C3 || ch.src_format == FKB_PIX_F32P3;
    const bool wide_yuv = ch.src_format == FKB_PIX_P010 || ch.src_format == FKB_PIX_P210 || ch.src_format == FKB_PIX_Y210;
    if (ch.src_format != FKB_PIX_U8C3 && ch.src_format != FKB_PIX_NV12 && ch.src_format != FKB_PIX_NV21 &&
        ch.src_format != FKB_PIX_UYVY && ch.src_format != FKB_PIX_U8C4 && !float_src && !wide_yuv) return FKB_ERR_UNSUPPORTED;
    const bool four = ch.dst_format == FKB_PIX_U8C4 || ch.dst_format == FKB_PIX_F32C4;  // the chain keeps four channels
    if (ch.dst_format != FKB_PIX_U8C3 && ch.dst_format != FKB_PIX_F32C3 && ch.dst_format != FKB_PIX_U8C1 && ch.dst_format != FKB_PIX_F32C1 && !four)
        return FKB_ERR_UNSUPPORTED;
    uint32_t n_alpha = 0;  // AddOpaqueAlpha: the step from three channels to four
    for (uint32_t i = 0; i < ch.n_ops && i < FKB_MAX_OPS; ++i) n_alpha += ch.ops[i].code == FKB_OP_ADD_ALPHA;
    // RGB2Gray: at most once, after the interpolation, nothing behind it that needs three channels, and a one-channel write
    const bool one = ch.dst_format == FKB_PIX_U8C1 || ch.dst_format == FKB_PIX_F32C1;
    uint32_t n_gray = 0, gray_at = 0;
    for (uint32_t i = 0; i < ch.n_ops && i < FKB_MAX_OPS; ++i)
        if (ch.ops[i].code == FKB_OP_RGB2GRAY) { ++n_gray; gray_at = i; }
    if (one != (n_gray == 1) || n_gray > 1) return FKB_ERR_INVALID;
    if (one) {
        if (ch.write_kind != FKB_WRITE_PACKED || float_src || ch.n_ops > FKB_MAX_OPS) return FKB_ERR_UNSUPPORTED;
        if (ch.geometry != FKB_GEOM_NONE && gray_at < ch.n_pre_ops) return FKB_ERR_UNSUPPORTED;
        for (uint32_t i = gray_at + 1; i < ch.n_ops; ++i) {
            const uint32_t c = ch.ops[i].code;
            if (c != FKB_OP_CAST_F32 && c != FKB_OP_MUL && c != FKB_OP_ADD && c != FKB_OP_SUB && c != FKB_OP_DIV && c != FKB_OP_SATCAST_U8) return FKB_ERR_INVALID;
        }
    }
    if (four) {
        if ((ch.src_format != FKB_PIX_U8C4 && ch.src_format != FKB_PIX_U8C3) || ch.write_kind != FKB_WRITE_PACKED) return FKB_ERR_UNSUPPORTED;
        if (n_alpha != (ch.src_format == FKB_PIX_U8C3 ? 1u : 0u)) return FKB_ERR_INVALID;
        for (uint32_t i = 0; i < ch.n_ops && i < FKB_MAX_OPS; ++i)
            if (ch.ops[i].code == FKB_OP_YUV2RGB || ch.ops[i].code == FKB_OP_RGB2YUV) return FKB_ERR_UNSUPPORTED;
    } else if (n_alpha) {
        return FKB_ERR_INVALID;
    }
    if (ch.geometry > FKB_GEOM_RESIZE_PRESERVE_AR_LEFT) return FKB_ERR_UNSUPPORTED;
    if (ch.write_kind < FKB_WRITE_PACKED || ch.write_kind > FKB_WRITE_UYVY) return FKB_ERR_UNSUPPORTED;
    if (ch.write_kind >= FKB_WRITE_NV12 && ch.dst_format != FKB_PIX_U8C3) return FKB_ERR_INVALID;  // WriteYUV takes byte triples
    if (ch.n_ops > FKB_MAX_OPS || ch.n_pre_ops > ch.n_ops) return FKB_ERR_INVALID;
    if (ch.border > FKB_BORDER_REFLECT_101) return FKB_ERR_UNSUPPORTED;
    if (ch.border && ch.border_at > (ch.geometry == FKB_GEOM_NONE ? ch.n_ops : ch.n_pre_ops)) return FKB_ERR_INVALID;
    ValueType t = float_src ? VT_F32 : VT_U8;  // the byte reads produce uchar3, the tensor reads float3
    int rc;
    if (ch.geometry == FKB_GEOM_NONE) {
        if ((rc = check_ops(ch, 0, ch.n_ops, t)) != FKB_OK) return rc;
    } else {
        if ((rc = check_ops(ch, 0, ch.n_pre_ops, t)) != FKB_OK) return rc;
        t = VT_F32;  // the interpolation returns float_<cn> whatever it reads
        if ((rc = check_ops(ch, ch.n_pre_ops, ch.n_ops, t)) != FKB_OK) return rc;
    }
    const ValueType want = (ch.dst_format == FKB_PIX_F32C3 || ch.dst_format == FKB_PIX_F32C4 || ch.dst_format == FKB_PIX_F32C1) ? VT_F32 : VT_U8;
    return t == want ? FKB_OK : FKB_ERR_INVALID;  // the Write's input type must be the chain's output type
}

int check_plane(const fkb_chain_desc& ch, const fkb_plane_desc& pl) {
    const bool dflt = (pl.chain & FKB_PLANE_DEFAULT) != 0;  // the read yields bg: no source is touched
    if ((!dflt && !pl.src) || !pl.dst) return FKB_ERR_NULL;
    const bool nv12 = ch.src_format == FKB_PIX_NV12 || ch.src_format == FKB_PIX_NV21;  // luma plane + interleaved chroma rows
    const bool float_src = ch.src_format == FKB_PIX_F32C3 || ch.src_format == FKB_PIX_F32P3;
    const bool semi16 = ch.src_format == FKB_PIX_P010 || ch.src_format == FKB_PIX_P210;
    const bool uyvy = ch.src_format == FKB_PIX_UYVY;
    if (!dflt) {
        if ((nv12 || semi16 || ch.src_format == FKB_PIX_F32P3) && !pl.src_chroma) return FKB_ERR_NULL;
        if ((semi16 || ch.src_format == FKB_PIX_Y210) &&
            ((reinterpret_cast<uintptr_t>(pl.src) & 1) || (reinterpret_cast<uintptr_t>(pl.src_chroma) & 1) || (pl.src_pitch & 1))) return FKB_ERR_INVALID;
        if (float_src && ((reinterpret_cast<uintptr_t>(pl.src) & 3) || (reinterpret_cast<uintptr_t>(pl.src_chroma) & 3) || (pl.src_pitch & 3))) return FKB_ERR_INVALID;
        if (pl.src_w == 0 || pl.src_h == 0) return FKB_ERR_INVALID;
        const uint64_t src_row = semi16 ? ((static_cast<uint64_t>(pl.src_w) + 1) / 2) * 4
                                 : ch.src_format == FKB_PIX_Y210 ? ((static_cast<uint64_t>(pl.src_w) + 1) / 2) * 8
                                 : nv12 ? ((static_cast<uint64_t>(pl.src_w) + 1) / 2) * 2
                                 : uyvy ? ((static_cast<uint64_t>(pl.src_w) + 1) / 2) * 4
                                 : static_cast<uint64_t>(pl.src_w) * (ch.src_format == FKB_PIX_F32C3 ? 12 : (ch.src_format == FKB_PIX_U8C4 || ch.src_format == FKB_PIX_F32P3) ? 4 : 3);
        if (pl.src_pitch < src_row) return FKB_ERR_INVALID;
        if (pl.crop_w <= 0 || pl.crop_h <= 0) return FKB_ERR_INVALID;
        if (ch.border) {
            // the rectangle may leave the frame; its origin is signed (crop.h:36-39).  Bounded so that the index maps
            // of the border modes cannot overflow.
            const int64_t lim = 1 << 24;
            const int64_t x = static_cast<int32_t>(pl.crop_x), y = static_cast<int32_t>(pl.crop_y);
            if (x < -lim || x > lim || y < -lim || y > lim || pl.crop_w > lim || pl.crop_h > lim || pl.src_w > lim || pl.src_h > lim)
                return FKB_ERR_INVALID;
        } else if (static_cast<uint64_t>(pl.crop_x) + static_cast<uint64_t>(pl.crop_w) > pl.src_w ||
                   static_cast<uint64_t>(pl.crop_y) + static_cast<uint64_t>(pl.crop_h) > pl.src_h) {
            return FKB_ERR_INVALID;
        }
    } else if (ch.geometry == FKB_GEOM_NONE) {
        for (int c = 0; c < 3; ++c)  // a uchar3 default
            if (!(pl.bg[c] >= 0.f && pl.bg[c] <= 255.f) || pl.bg[c] != std::floor(pl.bg[c])) return FKB_ERR_INVALID;
        if ((ch.dst_format == FKB_PIX_U8C4 || ch.dst_format == FKB_PIX_F32C4) &&
            (!(pl.bg_w >= 0.f && pl.bg_w <= 255.f) || pl.bg_w != std::floor(pl.bg_w))) return FKB_ERR_INVALID;
    }
    if (pl.dst_w == 0 || pl.dst_h == 0) return FKB_ERR_INVALID;
    const bool four = ch.dst_format == FKB_PIX_U8C4 || ch.dst_format == FKB_PIX_F32C4;
    const bool one = ch.dst_format == FKB_PIX_U8C1 || ch.dst_format == FKB_PIX_F32C1;
    const bool f32 = ch.dst_format == FKB_PIX_F32C3 || ch.dst_format == FKB_PIX_F32C4 || ch.dst_format == FKB_PIX_F32C1;
    const bool planes3 = ch.write_kind == FKB_WRITE_SPLIT_PLANES;
    if (planes3 && (!pl.dst_y || !pl.dst_z)) return FKB_ERR_NULL;
    const bool split = ch.write_kind == FKB_WRITE_SPLIT || planes3;
    const bool semi = ch.write_kind == FKB_WRITE_NV12 || ch.write_kind == FKB_WRITE_NV21;
    if (semi && !pl.dst_y) return FKB_ERR_NULL;
    const uint64_t dst_row = semi ? ((static_cast<uint64_t>(pl.dst_w) + 1) / 2) * 2
                             : ch.write_kind == FKB_WRITE_UYVY ? ((static_cast<uint64_t>(pl.dst_w) + 1) / 2) * 4
                             : four ? static_cast<uint64_t>(pl.dst_w) * (f32 ? 16 : 4)
                             : one ? static_cast<uint64_t>(pl.dst_w) * (f32 ? 4 : 1)
                             : static_cast<uint64_t>(pl.dst_w) * (split ? (f32 ? 4 : 1) : (f32 ? 12 : 3));
    if (pl.dst_pitch < dst_row) return FKB_ERR_INVALID;
    if (f32 && ((reinterpret_cast<uintptr_t>(pl.dst) & 3) || (pl.dst_pitch & 3) || (pl.dst_channel_stride & 3))) return FKB_ERR_INVALID;
    if (f32 && planes3 && ((reinterpret_cast<uintptr_t>(pl.dst_y) & 3) || (reinterpret_cast<uintptr_t>(pl.dst_z) & 3))) return FKB_ERR_INVALID;
    if (split && !planes3 && pl.dst_channel_stride < static_cast<uint64_t>(pl.dst_pitch) * (pl.dst_h - 1) + dst_row) return FKB_ERR_INVALID;
    if (dflt) return FKB_OK;
    if (ch.geometry == FKB_GEOM_NONE) {
        if (pl.dst_w > static_cast<uint32_t>(pl.crop_w) || pl.dst_h > static_cast<uint32_t>(pl.crop_h)) return FKB_ERR_INVALID;
    } else {
        // A PRESERVE_AR target that rounds to zero width or height (x2 < x1 or y2 < y1) is legal in the reference:
        // no pixel is inside, the whole plane is background, and the scale factors (then infinite) are never used.
        const bool empty = ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR && (pl.x2 < pl.x1 || pl.y2 < pl.y1);
        if (!empty && (!(pl.fx > 0.f) || !(pl.fy > 0.f) || !std::isfinite(pl.fx) || !std::isfinite(pl.fy))) return FKB_ERR_INVALID;
        // source coordinates stay below 2^22 (the kernels take their floor without a conversion instruction)
        if (!empty && (!(pl.fx * static_cast<float>(pl.dst_w) < 4194304.f) || !(pl.fy * static_cast<float>(pl.dst_h) < 4194304.f))) return FKB_ERR_UNSUPPORTED;
        if (ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR && !empty) {
            if (pl.x1 < 0 || pl.y1 < 0 || pl.x2 >= static_cast<int>(pl.dst_w) || pl.y2 >= static_cast<int>(pl.dst_h)) return FKB_ERR_INVALID;
        }
    }
    return FKB_OK;
}

int validate(const fkb_chain_desc* chains, uint32_t n_chains, const fkb_plane_desc* planes, uint32_t n_planes) {
    if (!chains || !planes) return FKB_ERR_NULL;
    if (n_chains == 0 || n_chains > FKB_MAX_CHAINS || n_planes == 0) return FKB_ERR_INVALID;
    for (uint32_t c = 0; c < n_chains; ++c) {
        const int rc = check_chain(chains[c]);
        if (rc != FKB_OK) return rc;
    }
    for (uint32_t z = 0; z < n_planes; ++z) {
        if ((planes[z].chain & ~FKB_PLANE_DEFAULT) >= n_chains) return FKB_ERR_INVALID;
        const int rc = check_plane(chains[planes[z].chain & ~FKB_PLANE_DEFAULT], planes[z]);
        if (rc != FKB_OK) return rc;
    }
    return FKB_OK;
}

// -------------------------------------------------------------------------------------------------------
// lowering
// -------------------------------------------------------------------------------------------------------
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Debugging and tuning switches, read from the environment once per lowering (not once per plane):
//   FKB_FORCE_GATHER=1       routes every plane through gather_kernel, which lets the kernel paths check each other;
//   FKB_TINY_PIXELS=n        launches below n output pixels take the one-pixel-per-thread kernels (0 switches that off, and
//                            the joining of small pipelined planes to a general kernel with it, which the tests use to
//                            drive small cases through the pipelined kernels);
//   FKB_ROWS_PER_ITEM=n      output rows per item of the staged kernel (default: chosen from the launch size);
//   FKB_SPLIT_ITEMS=0        the staged kernel's last items are dealt whole (default: in two halves, see lower());
//   FKB_TEST_EXTRA_TX=n      test hook: the staged kernel's resize loads announce n bytes more than they deliver, so its
//                            bounded waits run out and the launch ends with FKB_ERR_DEVICE_WAIT in the status word;
//   FKB_WAIT_LIMIT_US=n      how long such a wait lasts before it gives up (default one second);
//   FKB_TEST_SHRINK_FRAME=1  test hook for the self-checking build: the plane records claim source frames of one row, so that
//                            build's range checks fail, record FKB_ERR_DEVICE_CHECK and skip the copies (the release build
//                            does not read that field on its pipelined paths).
struct Tuning {
    bool force_gather = false;
    uint64_t tiny_pixels = kTinyLaunchPixels;
    uint32_t rows_per_item = 0, test_extra_tx = 0, wait_limit_ns = 1000000000u;
    bool test_shrink_frame = false;
    bool split_items = true;  // FKB_SPLIT_ITEMS=0: the staged kernel's last items are not dealt in halves
};
Tuning read_tuning() {
    Tuning t;
    const char* e = std::getenv("FKB_FORCE_GATHER");
    t.force_gather = e && e[0] == '1';
    if ((e = std::getenv("FKB_TINY_PIXELS")) && e[0]) t.tiny_pixels = std::strtoull(e, nullptr, 10);
    if ((e = std::getenv("FKB_ROWS_PER_ITEM")) && e[0]) t.rows_per_item = static_cast<uint32_t>(std::strtoul(e, nullptr, 10));
    if ((e = std::getenv("FKB_TEST_EXTRA_TX")) && e[0]) t.test_extra_tx = static_cast<uint32_t>(std::strtoul(e, nullptr, 10));
    if ((e = std::getenv("FKB_SPLIT_ITEMS")) && e[0] == '0') t.split_items = false;
    if ((e = std::getenv("FKB_TEST_SHRINK_FRAME")) && e[0] == '1') t.test_shrink_frame = true;
    if ((e = std::getenv("FKB_WAIT_LIMIT_US")) && e[0]) t.wait_limit_ns = static_cast<uint32_t>(std::min<unsigned long>(std::strtoul(e, nullptr, 10), 4000000ul) * 1000ul);
    return t;
}

uint32_t post_kind_of(const fkb_chain_desc& ch);

// Chooses the kernel path and tile shape of one plane.
void classify(const fkb_chain_desc& ch, PlaneRec& r, const Tuning& tune) {
    r.kclass = KCLASS_GATHER;
    r.tile_w = r.tile_h = r.tiles_x = 0;
    if (ch.dst_format == FKB_PIX_U8C4 || ch.dst_format == FKB_PIX_F32C4) { r.kclass = KCLASS_GATHER4; return; }
    if (ch.dst_format == FKB_PIX_U8C1 || ch.dst_format == FKB_PIX_F32C1) return;  // one-channel chains: the general kernel
    if (tune.force_gather) return;
    if (ch.border) {
        // a rectangle inside the frame never meets the border: it takes the usual paths; one that leaves it is
        // remapped tap by tap in the general kernel
        const int64_t x = static_cast<int32_t>(r.crop_x), y = static_cast<int32_t>(r.crop_y);
        if (x < 0 || y < 0 || x + r.crop_w > static_cast<int64_t>(r.src_w) || y + r.crop_h > static_cast<int64_t>(r.src_h)) return;
    }
    // what nv12_kernel's aligned tap loads need: 16-bit UV pairs (NV12 / NV21), one word per pixel pair (UYVY, and the
    // chroma of P010 / P210), one 64-bit group per pixel pair (Y210)
    const uintptr_t sa = reinterpret_cast<uintptr_t>(r.src), ca = reinterpret_cast<uintptr_t>(r.src_chroma);
    bool yuv_aligned = false;
    switch (ch.src_format) {
    case FKB_PIX_NV12: case FKB_PIX_NV21: yuv_aligned = (ca & 1) == 0 && (r.src_pitch & 1) == 0; break;
    case FKB_PIX_UYVY: yuv_aligned = (sa & 3) == 0 && (r.src_pitch & 3) == 0; break;
    case FKB_PIX_P010: case FKB_PIX_P210: yuv_aligned = (ca & 3) == 0 && (r.src_pitch & 3) == 0; break;
    case FKB_PIX_Y210: yuv_aligned = (sa & 7) == 0 && (r.src_pitch & 7) == 0; break;
    default: break;
    }
    if (yuv_aligned && ch.geometry != FKB_GEOM_NONE && ch.n_pre_ops == 1 && ch.ops[0].code == FKB_OP_YUV2RGB &&
        ch.write_kind <= FKB_WRITE_SPLIT_PLANES && post_kind_of(ch) != 8u && !(ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR && (r.x2 < r.x1 || r.y2 < r.y1))) {
        r.kclass = KCLASS_NV12;  // NV12 -> RGB on the taps -> resize -> [Mul][Add|Sub][Div][SaturateCast]: nv12_kernel
        return;
    }
    const bool f32 = ch.dst_format == FKB_PIX_F32C3;
    // planar float destinations (tensor, transposed tensor, three planes) have a staged path for resampling chains
    const bool planar = (ch.write_kind == FKB_WRITE_SPLIT || ch.write_kind == FKB_WRITE_SPLIT_PLANES) && f32 && ch.geometry != FKB_GEOM_NONE;
    // uchar4 sources (alpha skipped) have a staged path for resampling chains with a float destination
    const bool src4 = ch.src_format == FKB_PIX_U8C4;
    if (src4 && (!f32 || ch.geometry == FKB_GEOM_NONE)) return;
    if ((ch.src_format != FKB_PIX_U8C3 && !src4) || (ch.write_kind != FKB_WRITE_PACKED && !planar)) return;
    if (!aligned16(r.src) || !aligned16(r.dst) || (r.src_pitch & 15) || (r.dst_pitch & 15)) return;
    if (planar && ((r.dst_cstride & 15) || (r.dst_cstride2 & 15))) return;
    const uint32_t elt = f32 ? 12u : 3u;

    (void)elt;
    if (ch.geometry == FKB_GEOM_NONE) {
        if ((r.crop_x * 3u) & 15u) return;  // the staged row must start on a 16-byte boundary
        // one row segment per step: 16 pixels per lane (uchar3 out) or 4 pixels per lane in two passes (float3 out)
        r.tile_w = std::min(r.dst_w, f32 ? kMaxTileW : kPointTileU8);
        r.kclass = KCLASS_POINT;
        if (!f32) {  // uchar3 -> uchar3 through per-channel ops only: table lookups (lut_kernel)
            bool per_channel = true;
            for (uint32_t i = 0; i < ch.n_ops; ++i) per_channel = per_channel && ch.ops[i].code != FKB_OP_YUV2RGB;
            if (per_channel) r.kclass = KCLASS_LUT;
        }
    } else {
        for (uint32_t i = 0; i < ch.n_pre_ops; ++i)
            if (ch.ops[i].code != FKB_OP_CAST_F32) return;  // taps are transformed before interpolation: general path
        if (ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR && (r.x2 < r.x1 || r.y2 < r.y1)) {
            // a crop so thin that its resized image has no pixel: every row of the plane is background, which the staged
            // kernel writes without touching the source (its scale factors may be infinite and are not used)
            r.x1 = 0; r.x2 = -1;  // (an empty row range is recorded as an empty column range: no column has a footprint)
            r.tile_w = std::min(r.dst_w, kMaxTileW);
            r.kclass = KCLASS_RESIZE;
            r.tiles_x = (r.dst_w + r.tile_w - 1) / r.tile_w;
            return;
        }
        if (!(r.fx <= 32.f) || !(r.fy <= 4096.f)) return;
        for (uint32_t i = ch.n_pre_ops; i < ch.n_ops; ++i)  // (a per-plane Mul operand takes a factor of 2^22 there, too)
            if (ch.ops[i].code == FKB_OP_MUL && ch.ops[i].plane_slot >= 0)
                for (int c = 0; c < 3; ++c)
                    if (!(std::fabs(r.params[ch.ops[i].plane_slot][c]) < 0x1p100f)) return;
        // the staged kernel reads tap bytes as subnormal floats and scales them by powers of two; with scale factors
        // this small (an enlargement by 2^24) a weight could underflow there
        if (!(r.fx >= 5.9604645e-8f) || !(r.fy >= 5.9604645e-8f)) return;
        // widest segment (at most 8 columns per lane) whose source columns fit one staged row
        uint32_t tw = std::min(r.dst_w, kMaxTileW);
        for (;;) {
            const uint32_t cols = std::min<uint32_t>(r.crop_w, static_cast<uint32_t>(std::ceil((tw - 1) * static_cast<double>(r.fx))) + 3u);
            if (cols * (src4 ? 4u : 3u) + 63u <= kInRowBytes) break;
            if (tw <= 16) return;  // too sparse to stage: general path
            tw = tw > 32 ? ((tw - 1) & ~15u) : 16u;
        }
        r.tile_w = tw;
        r.kclass = KCLASS_RESIZE;
    }
    r.tiles_x = (r.dst_w + r.tile_w - 1) / r.tile_w;  // tile_h is chosen per launch (rows_per_item)
}

// Whether a plane can run on rgb_kernel (one pixel per thread, post-ops specialised): a packed byte source, a resampling
// geometry with nothing but casts ahead of it, a specialisable op shape behind it, and a rectangle inside the frame.
bool rgb_kernel_takes(const fkb_chain_desc& ch, const PlaneRec& r) {
    if (ch.src_format != FKB_PIX_U8C3 && ch.src_format != FKB_PIX_U8C4) return false;
    if (ch.dst_format != FKB_PIX_U8C3 && ch.dst_format != FKB_PIX_F32C3) return false;
    if (ch.geometry == FKB_GEOM_NONE || ch.write_kind > FKB_WRITE_SPLIT_PLANES || post_kind_of(ch) == 8u || r.src == nullptr) return false;
    for (uint32_t i = 0; i < ch.n_pre_ops; ++i)
        if (ch.ops[i].code != FKB_OP_CAST_F32) return false;
    if (ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR && (r.x2 < r.x1 || r.y2 < r.y1)) return false;
    const int64_t x = static_cast<int32_t>(r.crop_x), y = static_cast<int32_t>(r.crop_y);
    return x >= 0 && y >= 0 && x + r.crop_w <= static_cast<int64_t>(r.src_w) && y + r.crop_h <= static_cast<int64_t>(r.src_h);
}

// Output rows a warp processes per item.  An item costs a set-up (about as much as a row and a half), and inside an
// item the source rows of the rows after next are already in flight, so longer items run better; shorter ones balance
// better (warps claim them from a counter, the next one a few rows before the current one ends) and leave a shorter
// tail when the launch ends.  Measured on crop-resize launches of 224 x 224 planes (rows per warp in brackets): 2048
// planes (194) 12 rows per item 242 us, 8: 255, 10: 245, 16: 245, 24: 251; 1024 planes (97) 12: 126, 8: 132, 16: 127;
// 512 planes (48) 12: 68.3, 8: 70.5, 20: 72; 256 planes (24) 10: 39.1, 8: 40.0, 12: 41.3, 14: 46.6; 128 planes (12): items
// of 13 or 14 rows, one per warp, 24-25 us, against 25.7-26.3 us for 6 to 8 rows; 192 planes (18): 8 rows 31.0 us, 10 rows
// 33.8 us (fewer than two items per warp, which are then dealt by position).  So: a launch too small to give every
// resident warp sixteen rows gets items of just the length that spreads its rows over all warps in one round; up to
// twenty-one rows per warp items have eight rows (enough items for the counter), up to forty ten, beyond that twelve.
uint32_t rows_per_item(uint64_t row_segments, uint32_t resident_warps) {
    if (row_segments < 16ull * resident_warps)
        return static_cast<uint32_t>(std::max<uint64_t>((row_segments + resident_warps - 1) / resident_warps, 1));
    return row_segments < 21ull * resident_warps ? 8u : row_segments < 40ull * resident_warps ? 10u : 12u;
}

// Shape of the ops that follow the read / the interpolation: bit 0 Mul, bit 1 Add or Sub, bit 2 SaturateCast when the
// chain is [Cast]* [Mul] [Add|Sub] [Div] [SaturateCast] in this order (bit 4 = Div; the kernels specialise those shapes),
// else 8 (interpreted).
uint32_t post_kind_of(const fkb_chain_desc& ch) {
    uint32_t i = ch.geometry == FKB_GEOM_NONE ? 0 : ch.n_pre_ops, kind = 0;
    while (i < ch.n_ops && ch.ops[i].code == FKB_OP_CAST_F32) ++i;
    if (i < ch.n_ops && ch.ops[i].code == FKB_OP_MUL) {
        // (the staged kernel folds a factor of 2^22 into this operand: a huge one goes through the interpreter instead)
        if (ch.ops[i].plane_slot < 0)
            for (int c = 0; c < 3; ++c)
                if (!(std::fabs(ch.ops[i].v[c]) < 0x1p100f)) return 8u;
        kind |= 1; ++i;
    }
    if (i < ch.n_ops && (ch.ops[i].code == FKB_OP_ADD || ch.ops[i].code == FKB_OP_SUB)) { kind |= 2; ++i; }
    if (i < ch.n_ops && ch.ops[i].code == FKB_OP_DIV) { kind |= 16; ++i; }  // only nv12_kernel specialises this part
    if (i < ch.n_ops && ch.ops[i].code == FKB_OP_SATCAST_U8) { kind |= 4; ++i; }
    return i == ch.n_ops ? kind : 8u;
}

// Immediate operands of a chain's [Mul][Add|Sub][Div] post-ops (see PostImm).
PostImm post_imm_of(const fkb_chain_desc& ch) {
    PostImm q{};
    for (int c = 0; c < 3; ++c) { q.m[c] = 1.f; q.a[c] = 0.f; q.d[c] = 1.f; }
    for (uint32_t i = ch.geometry == FKB_GEOM_NONE ? 0 : ch.n_pre_ops; i < ch.n_ops; ++i) {
        const fkb_op& op = ch.ops[i];
        if (op.code != FKB_OP_MUL && op.code != FKB_OP_ADD && op.code != FKB_OP_SUB && op.code != FKB_OP_DIV) continue;
        if (op.plane_slot >= 0) q.slots = 1;
        for (int c = 0; c < 3; ++c) {
            if (op.code == FKB_OP_MUL) q.m[c] = op.v[c];
            if (op.code == FKB_OP_ADD) q.a[c] = op.v[c];
            if (op.code == FKB_OP_SUB) q.a[c] = -op.v[c];
            if (op.code == FKB_OP_DIV) q.d[c] = op.v[c];
        }
    }
    return q;
}

struct Lowered {
    PlaneRec* recs = nullptr;        // one record per plane: the caller's fixed array, or `storage`
    std::vector<PlaneRec> storage;   // used only when the caller gave no array (never by the no-allocation entry point)
    LaunchParams lp;
    uint32_t staged_grid = 0;
    uint32_t lut_grid = 0;
    dim3 gather_grid{0, 0, 0};
    dim3 gather4_grid{0, 0, 0};
    dim3 nv12_grid{0, 0, 0};
    int gather_ppt = 4;
    uint32_t kernels = 0;
};

int device_sm_count(int& sms) {
    static int cached[64] = {0};
    int dev = 0;
    FKB_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && cached[dev]) { sms = cached[dev]; return FKB_OK; }
    FKB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (dev < 64) cached[dev] = sms;
    return FKB_OK;
}

int status_word(int** out) {
    static std::mutex m;
    static int* cached[64] = {nullptr};
    int dev = 0;
    FKB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> g(m);
    if (dev < 64 && cached[dev]) { *out = cached[dev]; return FKB_OK; }
    int* p = nullptr;
    FKB_CUDA(status_word_address(&p));
    if (dev < 64) cached[dev] = p;
    *out = p;
    return FKB_OK;
}

// Fills L.lp.four when every four-channel plane of the launch runs one chain that rgba_kernel can take: no per-plane
// operands, nothing but casts ahead of the interpolation, at most kFourMaxSteps steps behind it, no plane that yields its
// default value or whose rectangle leaves the frame, word-aligned sources and destinations.  Mul / Add / Sub become one
// fused multiply-add per channel, reorders a permutation of the operands and of the final store (see FourConsts).
void flatten_four_channel_chain(const fkb_chain_desc* chains, Lowered& L) {
    FourConsts& k = L.lp.four;
    k.enabled = 0;
    uint32_t chain = 0xffffffffu;
    for (uint32_t z = L.lp.gather4_z0; z < L.lp.gather4_z1; ++z) {
        const PlaneRec& r = L.recs[z];
        if (r.kclass != KCLASS_GATHER4) continue;
        if (chain == 0xffffffffu) chain = r.chain;
        const fkb_chain_desc& ch = chains[r.chain];
        if (r.chain != chain || r.src == nullptr) return;
        const int64_t x = static_cast<int32_t>(r.crop_x), y = static_cast<int32_t>(r.crop_y);
        if (x < 0 || y < 0 || x + r.crop_w > static_cast<int64_t>(r.src_w) || y + r.crop_h > static_cast<int64_t>(r.src_h)) return;
        const bool f32 = ch.dst_format == FKB_PIX_F32C4;
        const uintptr_t align = f32 ? 15u : 3u;
        if ((reinterpret_cast<uintptr_t>(r.dst) & align) || (r.dst_pitch & align)) return;
        if (ch.src_format == FKB_PIX_U8C4 && ((reinterpret_cast<uintptr_t>(r.src) & 3u) || (r.src_pitch & 3u))) return;
        if (ch.geometry != FKB_GEOM_NONE) {
            if (ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR && (r.x2 < r.x1 || r.y2 < r.y1)) return;
            if (!(r.fx >= 5.9604645e-8f) || !(r.fy >= 5.9604645e-8f) || !(r.fx <= 16777216.f) || !(r.fy <= 16777216.f)) return;
        }
    }
    if (chain == 0xffffffffu) return;
    const fkb_chain_desc& ch = chains[chain];
    uint32_t first = 0;
    if (ch.geometry != FKB_GEOM_NONE) {
        for (uint32_t i = 0; i < ch.n_pre_ops; ++i)
            if (ch.ops[i].code != FKB_OP_CAST_F32) return;
        first = ch.n_pre_ops;
    }
    uint32_t pi[4] = {0, 1, 2, 3};  // actual channel c is held in stored channel pi[c]
    bool have4 = ch.src_format == FKB_PIX_U8C4;
    uint32_t n = 0, kinds = 0;
    for (uint32_t i = first; i < ch.n_ops; ++i) {
        const fkb_op& op = ch.ops[i];
        if (op.code == FKB_OP_CAST_F32) continue;
        if (op.code == FKB_OP_REORDER_ZYX) { std::swap(pi[0], pi[2]); continue; }
        if (op.plane_slot >= 0 || n == kFourMaxSteps) return;
        const float operand[4] = {op.v[0], op.v[1], op.v[2], ch.op_w[i]};
        for (int c = 0; c < 4; ++c) { k.m[n][c] = 1.f; k.a[n][c] = -0.0f; }  // the identity: fma(x, 1, -0) = x
        const int nc = have4 ? 4 : 3;
        switch (op.code) {
        case FKB_OP_MUL: for (int c = 0; c < nc; ++c) k.m[n][pi[c]] = operand[c]; break;
        case FKB_OP_ADD: for (int c = 0; c < nc; ++c) k.a[n][pi[c]] = operand[c]; break;
        case FKB_OP_SUB: for (int c = 0; c < nc; ++c) k.a[n][pi[c]] = -operand[c]; break;
        case FKB_OP_DIV: for (int c = 0; c < nc; ++c) k.m[n][pi[c]] = operand[c]; kinds |= 1u << (2 * n); break;
        case FKB_OP_SATCAST_U8: kinds |= 2u << (2 * n); break;
        case FKB_OP_ADD_ALPHA: k.m[n][pi[3]] = 0.f; k.a[n][pi[3]] = op.v[0]; have4 = true; break;  // (the channel holds a finite value)
        default: return;
        }
        ++n;
    }
    k.n_steps = n; k.kinds = kinds;
    k.perm = pi[0] | (pi[1] << 2) | (pi[2] << 4) | (pi[3] << 6);
    k.src3 = ch.src_format == FKB_PIX_U8C3;
    k.f32 = ch.dst_format == FKB_PIX_F32C4;
    k.resize = ch.geometry != FKB_GEOM_NONE;
    k.preserve_ar = ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR;
    k.enabled = 1;
}

int lower(const fkb_chain_desc* chains, uint32_t n_chains, const fkb_plane_desc* planes, uint32_t n_planes, Lowered& L) {
    const int rc = validate(chains, n_chains, planes, n_planes);
    if (rc != FKB_OK) return rc;
    if (!L.recs) { L.storage.resize(n_planes); L.recs = L.storage.data(); }
    const Tuning tune = read_tuning();
    std::memset(&L.lp, 0, sizeof(L.lp));
    std::memcpy(L.lp.chains, chains, sizeof(fkb_chain_desc) * n_chains);
    uint32_t n_tiles = 0, gw = 0, gh = 0, n_gather = 0, g4w = 0, g4h = 0, n_gather4 = 0;
    uint32_t first_count = 0;
    int sms = 0;
    {
        const int e = device_sm_count(sms);
        if (e != FKB_OK) return e;
    }
    uint64_t row_segments = 0, lut_rows = 0, total_pixels = 0, gather_pixels = 0;
    uint32_t n_nv12 = 0, nw = 0, nh = 0, nv12_chain = 0xffffffffu;
    uint32_t lut_min_tiles_x = 0xffffffffu;
    // Order of the records.  A record is self-contained (it carries its own destination), so the table may hold the
    // planes in any order, and the pipelined kernel deals its items in table order.  Planes of different chains cost
    // different things — a resize plane is arithmetic, a pointwise float plane is memory traffic — and a launch that
    // runs first all planes of one chain and then all of the other (as a divergent launch lists them) is short of HBM
    // bandwidth in one phase and leaves it idle in the other.  The planes of a launch of several chains are therefore
    // dealt chain by chain in turn, each chain at its own rate, so that at any time items of all chains are in flight
    // (the divergent configuration: 110.9 -> 102.6 us).  Within a chain the caller's order is kept.
    std::vector<uint32_t> order;
    if (n_chains > 1 && n_planes > 2) {
        uint32_t count[FKB_MAX_CHAINS] = {0}, first[FKB_MAX_CHAINS] = {0}, taken[FKB_MAX_CHAINS] = {0};
        for (uint32_t z = 0; z < n_planes; ++z) ++count[planes[z].chain & ~FKB_PLANE_DEFAULT];
        for (uint32_t c = 1; c < n_chains; ++c) first[c] = first[c - 1] + count[c - 1];
        std::vector<uint32_t> by_chain(n_planes);
        for (uint32_t z = 0; z < n_planes; ++z) {
            const uint32_t c = planes[z].chain & ~FKB_PLANE_DEFAULT;
            by_chain[first[c] + taken[c]++] = z;
        }
        std::memset(taken, 0, sizeof(taken));
        order.resize(n_planes);
        for (uint32_t i = 0; i < n_planes; ++i) {
            uint32_t best = 0;
            uint64_t best_num = 1, best_den = 0;  // the chain whose next plane comes earliest, (taken + 1) / count smallest
            for (uint32_t c = 0; c < n_chains; ++c) {
                if (taken[c] == count[c]) continue;
                const uint64_t num = taken[c] + 1ull, den = count[c];
                if (best_den == 0 || num * best_den < best_num * den) { best = c; best_num = num; best_den = den; }
            }
            order[i] = by_chain[first[best] + taken[best]++];
        }
    }
    for (uint32_t z = 0; z < n_planes; ++z) {
        const fkb_plane_desc& s = planes[order.empty() ? z : order[z]];
        PlaneRec& r = L.recs[z];
        std::memset(&r, 0, sizeof(r));
        r.src = static_cast<const uint8_t*>(s.src);
        r.src_chroma = static_cast<const uint8_t*>(s.src_chroma);
        r.dst = static_cast<uint8_t*>(s.dst);
        const uint32_t wk = chains[s.chain & ~FKB_PLANE_DEFAULT].write_kind;
        if (wk == FKB_WRITE_NV12 || wk == FKB_WRITE_NV21) {  // luma plane + chroma rows: one address difference
            r.dst_cstride = static_cast<uint64_t>(static_cast<const uint8_t*>(s.dst_y) - static_cast<const uint8_t*>(s.dst));
        } else if (wk == FKB_WRITE_SPLIT_PLANES) {  // three separate planes: address differences
            r.dst_cstride = static_cast<uint64_t>(static_cast<const uint8_t*>(s.dst_y) - static_cast<const uint8_t*>(s.dst));
            r.dst_cstride2 = static_cast<uint64_t>(static_cast<const uint8_t*>(s.dst_z) - static_cast<const uint8_t*>(s.dst));
        } else {
            r.dst_cstride = s.dst_channel_stride; r.dst_cstride2 = 2 * s.dst_channel_stride;
        }
        r.src_pitch = s.src_pitch; r.src_w = s.src_w; r.src_h = s.src_h;
        r.crop_x = s.crop_x; r.crop_y = s.crop_y; r.crop_w = s.crop_w; r.crop_h = s.crop_h;
        r.dst_w = s.dst_w; r.dst_h = s.dst_h; r.dst_pitch = s.dst_pitch;
        r.fx = s.fx; r.fy = s.fy; r.x1 = s.x1; r.y1 = s.y1; r.x2 = s.x2; r.y2 = s.y2;
        std::memcpy(r.bg, s.bg, sizeof(r.bg));
        r.chain = s.chain & ~FKB_PLANE_DEFAULT;
        std::memcpy(r.params, s.params, sizeof(r.params));
        r.bg_w = s.bg_w;
        std::memcpy(r.params_w, s.params_w, sizeof(r.params_w));
        if (s.chain & FKB_PLANE_DEFAULT) {  // the kernels know such a plane by its null source; the general kernels fill it
            r.src = r.src_chroma = nullptr;
            const fkb_chain_desc& ch = chains[r.chain];
            const uint32_t df = ch.dst_format;
            r.kclass = (df == FKB_PIX_U8C4 || df == FKB_PIX_F32C4) ? KCLASS_GATHER4 : KCLASS_GATHER;
            // Under a Resize such a plane is `bg` put through the ops behind the interpolation, pixel for pixel: what the
            // pipelined kernel writes for a plane without a single pixel inside its resized image.  Where a plane of this
            // chain with a source would take that kernel (asked of classify() with a stand-in source), this one does too,
            // as an all-background plane; the launch then needs no second kernel for it.
            if (ch.geometry != FKB_GEOM_NONE && !tune.force_gather && ch.src_format == FKB_PIX_U8C3) {
                PlaneRec probe = r;
                probe.src = reinterpret_cast<const uint8_t*>(uintptr_t{4096});  // (never read: classify() looks at its alignment only)
                probe.src_pitch = 16; probe.src_w = probe.src_h = 1;
                probe.crop_x = probe.crop_y = 0; probe.crop_w = probe.crop_h = 1;
                probe.fx = probe.fy = 1.f; probe.x1 = probe.y1 = 0; probe.x2 = probe.y2 = 0;
                classify(ch, probe, tune);
                if (probe.kclass == KCLASS_RESIZE) {
                    r.kclass = KCLASS_RESIZE;
                    r.tile_w = std::min(r.dst_w, kMaxTileW); r.tiles_x = (r.dst_w + r.tile_w - 1) / r.tile_w;
                    r.all_background = 1u;
                    r.crop_x = r.crop_y = 0; r.crop_w = r.crop_h = 1; r.src_pitch = 16; r.fx = r.fy = 1.f;
                    r.x1 = 0; r.x2 = -1; r.y1 = 0; r.y2 = -1;
                }
            }
        } else {
            classify(chains[r.chain], r, tune);
        }
        if (tune.test_shrink_frame) r.src_h = 1;
        total_pixels += static_cast<uint64_t>(r.dst_w) * r.dst_h;
    }
    // A launch of a few ten thousand pixels is pure latency: the pipelined paths would spend it filling their stages,
    // so it goes through the general kernel, one pixel per thread.
    if (total_pixels < tune.tiny_pixels)
        for (uint32_t z = 0; z < n_planes; ++z)
            if (L.recs[z].kclass != KCLASS_NV12 && L.recs[z].kclass != KCLASS_GATHER4) {
                // (the one-pixel-per-thread kernel where its conditions hold, else the general kernel)
                L.recs[z].kclass = (!tune.force_gather && rgb_kernel_takes(chains[L.recs[z].chain], L.recs[z])) ? KCLASS_NV12 : KCLASS_GATHER;
                L.recs[z].tiles_x = 0;
            }
    // A launch that needs the general kernel anyway (say, for crops that leave the frame under a BorderReader) and whose
    // other planes are small runs them there too: a second kernel costs more than the pipelined path saves on so few pixels.
    {
        uint64_t general = 0, pipelined = 0;
        for (uint32_t z = 0; z < n_planes; ++z) {
            const uint64_t px = static_cast<uint64_t>(L.recs[z].dst_w) * L.recs[z].dst_h;
            if (L.recs[z].kclass == KCLASS_GATHER) general += px;
            else if (L.recs[z].kclass == KCLASS_POINT || L.recs[z].kclass == KCLASS_RESIZE || L.recs[z].kclass == KCLASS_LUT) pipelined += px;
        }
        if (tune.tiny_pixels != 0 && general && pipelined && pipelined < kJoinGeneralPixels)  // (FKB_TINY_PIXELS=0 switches this routing off, too)
            for (uint32_t z = 0; z < n_planes; ++z)
                if (L.recs[z].kclass == KCLASS_POINT || L.recs[z].kclass == KCLASS_RESIZE || L.recs[z].kclass == KCLASS_LUT) {
                    L.recs[z].kclass = KCLASS_GATHER;
                    L.recs[z].tiles_x = 0;
                }
    }
    for (uint32_t z = 0; z < n_planes; ++z) {
        const PlaneRec& r = L.recs[z];
        if (r.kclass == KCLASS_POINT || r.kclass == KCLASS_RESIZE) row_segments += static_cast<uint64_t>(r.tiles_x) * r.dst_h;
        if (r.kclass == KCLASS_LUT) { lut_rows += r.dst_h; lut_min_tiles_x = std::min(lut_min_tiles_x, r.tiles_x); }
        if (r.kclass == KCLASS_GATHER) gather_pixels += static_cast<uint64_t>(r.dst_w) * r.dst_h;
        if (r.kclass == KCLASS_NV12) {
            if (nv12_chain == 0xffffffffu) nv12_chain = r.chain;
            if (r.chain == nv12_chain) { ++n_nv12; nw = std::max(nw, r.dst_w); nh = std::max(nh, r.dst_h); }
            else { L.recs[z].kclass = KCLASS_GATHER; gather_pixels += static_cast<uint64_t>(r.dst_w) * r.dst_h; }
        }
    }
    // LUT units: a block of rows of one plane per CTA visit; about one unit per resident CTA, at least eight row segments
    const uint32_t lut_rpu = lut_rows ? std::max<uint32_t>(static_cast<uint32_t>((lut_rows + 1ull * kLutCtasPerSm * sms - 1) / (1ull * kLutCtasPerSm * sms)),
                                                           (kLutWarps + lut_min_tiles_x - 1) / lut_min_tiles_x) : 1u;
    uint32_t n_lut_units = 0;
    // The records of the general kernels' planes move to the end of the table (a record is self-contained, so the order
    // of the table is free): each of those kernels then gets a grid that covers exactly its own planes, however they were
    // scattered among the others.  In place, no allocation: [other classes | one pixel per thread | four-channel | general].
    {
        auto to_back = [&](uint32_t cls, uint32_t end) {
            uint32_t lo = 0, hi = end;
            while (lo < hi) {
                if (L.recs[lo].kclass != cls) { ++lo; continue; }
                if (L.recs[hi - 1].kclass == cls) { --hi; continue; }
                std::swap(L.recs[lo], L.recs[hi - 1]);
                ++lo; --hi;
            }
            return hi;  // first record of class `cls`
        };
        const uint32_t first_general = to_back(KCLASS_GATHER, n_planes);
        const uint32_t first_four = to_back(KCLASS_GATHER4, first_general);
        const uint32_t first_pixel = to_back(KCLASS_NV12, first_four);
        L.lp.pixel_z0 = first_pixel; L.lp.pixel_z1 = first_four;
    }
    // Items of the staged kernel; when every plane of the launch has the same shape (the batched crop-resize case) the
    // kernel finds an item's plane by division instead of a search.
    const uint32_t resident_warps = kStagedCtasPerSm * kStagedWarps * static_cast<uint32_t>(sms);
    const uint32_t rpi = tune.rows_per_item ? std::min(tune.rows_per_item, kMaxRowsPerItem) : rows_per_item(row_segments, resident_warps);
    bool same_shape = n_planes > 0;
    for (uint32_t z = 0; z < n_planes && same_shape; ++z) {
        const PlaneRec& r = L.recs[z];
        same_shape = (r.kclass == KCLASS_POINT || r.kclass == KCLASS_RESIZE) && r.tiles_x == L.recs[0].tiles_x && r.dst_h == L.recs[0].dst_h;
    }
    for (uint32_t z = 0; z < n_planes; ++z) {
        PlaneRec& r = L.recs[z];
        r.lut_base = n_lut_units;
        if (r.kclass == KCLASS_LUT) {
            r.tile_h = std::min(r.dst_h, lut_rpu);
            n_lut_units += (r.dst_h + r.tile_h - 1) / r.tile_h;
        } else if (r.kclass != KCLASS_GATHER) {
            r.tile_h = std::min(r.dst_h, rpi);
        }
        r.tile_base = n_tiles;
        const uint32_t count = (r.kclass == KCLASS_POINT || r.kclass == KCLASS_RESIZE) ? r.tiles_x * ((r.dst_h + r.tile_h - 1) / r.tile_h) : 0u;
        if (z == 0) first_count = count;
        if (static_cast<uint64_t>(n_tiles) + count > 0xfffffff0ull) return FKB_ERR_TOO_LARGE;
        n_tiles += count;
        if (r.kclass == KCLASS_GATHER) {
            if (!n_gather++) L.lp.gather_z0 = z;
            L.lp.gather_z1 = z + 1;
            gw = std::max(gw, r.dst_w); gh = std::max(gh, r.dst_h);
        }
        if (r.kclass == KCLASS_GATHER4) {
            if (!n_gather4++) L.lp.gather4_z0 = z;
            L.lp.gather4_z1 = z + 1;
            g4w = std::max(g4w, r.dst_w); g4h = std::max(g4h, r.dst_h);
        }
    }
    L.lp.n_planes = n_planes;
    L.lp.neg_zero = -0.0f;
    L.lp.test_extra_tx = tune.test_extra_tx;
    L.lp.wait_limit_ns = tune.wait_limit_ns;
    L.lp.pdl = total_pixels >= kPdlMinPixels;
    for (uint32_t c = 0; c < n_chains; ++c) {
        L.lp.post_kind[c] = post_kind_of(chains[c]);
        L.lp.post_imm[c] = post_imm_of(chains[c]);
        uint32_t reorders = 0;
        for (uint32_t i = 0; i < chains[c].n_ops; ++i) reorders += chains[c].ops[i].code == FKB_OP_REORDER_ZYX;
        L.lp.lut_swap |= (reorders & 1u) << c;
    }
    L.lp.n_tiles = n_tiles;
    {
        // A launch whose warps claim their items ends when the last claimed items do.  The last items — half as many as
        // there are resident warps — are therefore dealt as two halves each (their first rows, their other rows): the end
        // of the launch then waits for half an item, at the price of one more item set-up for those.  FKB_SPLIT_ITEMS=0
        // switches it off.
        const uint32_t resident = kStagedCtasPerSm * kStagedWarps * static_cast<uint32_t>(sms);
        L.lp.n_split = (tune.split_items && n_tiles > 2u * resident) ? std::min(n_tiles - 2u * resident, resident / 2u) : 0u;
    }
    L.lp.tiles_per_plane = (same_shape && first_count) ? first_count : 0;
    if (n_tiles) {
        L.staged_grid = std::min<uint32_t>(n_tiles, kStagedCtasPerSm * static_cast<uint32_t>(sms));
        ++L.kernels;
    }
    L.lp.n_lut_units = n_lut_units;
    if (n_lut_units) {
        L.lut_grid = std::min<uint32_t>(n_lut_units, kLutCtasPerSm * static_cast<uint32_t>(sms));
        ++L.kernels;
    }
    if (n_nv12) {
        // nv12_kernel is specialised on one chain; planes of any other NV12 chain of the launch take the general kernel
        const uint32_t c = nv12_chain;
        const fkb_chain_desc& ch = chains[c];
        Nv12Consts& k = L.lp.nv12;
        std::memcpy(k.ccm, ch.ccm, sizeof(k.ccm));
        std::memcpy(k.sub, ch.yuv_sub, sizeof(k.sub));
        const PostImm imm = post_imm_of(ch);
        std::memcpy(k.m, imm.m, sizeof(k.m)); std::memcpy(k.a, imm.a, sizeof(k.a)); std::memcpy(k.d, imm.d, sizeof(k.d));
        k.kind = post_kind_of(ch); k.chain = c; k.slots = imm.slots;
        k.preserve_ar = ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR; k.f32 = ch.dst_format == FKB_PIX_F32C3; k.split = ch.write_kind != FKB_WRITE_PACKED;
        // nv12_pair_kernel's conditions: the colour matrix of the YCbCr standards ([s 0 r; s g1 g2; s b 0]), integer
        // offsets, immediate operands, and plane offsets that fit 32 bits
        k.vu = ch.src_format == FKB_PIX_NV21;
        k.yuv_fmt = ch.src_format;
        k.src_px = ch.src_format == FKB_PIX_U8C3 ? 3u : ch.src_format == FKB_PIX_U8C4 ? 4u : 0u;
        bool pair = (ch.src_format == FKB_PIX_NV12 || ch.src_format == FKB_PIX_NV21) && !imm.slots && k.ccm[0] > 0.f && std::isfinite(k.ccm[0]) && k.ccm[3] == k.ccm[0] && k.ccm[6] == k.ccm[0] &&
                    k.ccm[1] == 0.f && k.ccm[8] == 0.f;
        for (int i = 0; i < 3; ++i) {
            pair = pair && k.sub[i] >= 0.f && k.sub[i] <= 255.f && k.sub[i] == std::floor(k.sub[i]);
            k.kmag[i] = 8388608.f + (pair ? k.sub[i] : 0.f);
        }
        for (int i : {2, 4, 5, 7}) pair = pair && std::isfinite(k.ccm[i]);
        bool wide = true;
        for (uint32_t z = 0; z < n_planes && pair; ++z) {
            const PlaneRec& r = L.recs[z];
            if (r.kclass != KCLASS_NV12) continue;
            const uint64_t src_end = static_cast<uint64_t>(r.src_pitch) * (static_cast<uint64_t>(r.crop_y) + r.crop_h) + r.crop_x + r.crop_w;
            const uint64_t dst_end = static_cast<uint64_t>(r.dst_pitch) * r.dst_h;
            pair = src_end < (1ull << 31) && dst_end < (1ull << 31);
            wide = wide && (reinterpret_cast<uintptr_t>(r.dst) & 7) == 0 && (r.dst_pitch & 7) == 0 && (r.dst_cstride & 7) == 0 && (r.dst_cstride2 & 7) == 0;
        }
        k.pair = pair; k.wide_store = wide;
        L.nv12_grid = dim3((nw + (pair ? 63 : 31)) / (pair ? 64 : 32), (nh + 7) / 8, std::min<uint32_t>(L.lp.pixel_z1 - L.lp.pixel_z0, 65535u));
        ++L.kernels;
    }
    if (n_gather4) {
        if (!tune.force_gather) flatten_four_channel_chain(chains, L);  // (FKB_FORCE_GATHER keeps the interpreting kernel)
        // (grid.z spans only the planes from the first to the last of this class: a stray plane costs one layer of CTAs)
        L.gather4_grid = dim3((g4w + 31) / 32, (g4h + 7) / 8, std::min<uint32_t>(L.lp.gather4_z1 - L.lp.gather4_z0, 65535u));
        ++L.kernels;
    }
    if (n_gather) {
        // small launches are latency-bound: one pixel per thread puts four times as many threads on the taps.  Writes of a
        // YCbCr image go four pixels per thread much earlier: that turns their byte stores into word stores.
        bool yuv_write = false;
        for (uint32_t z = 0; z < n_planes; ++z)
            yuv_write = yuv_write || (L.recs[z].kclass == KCLASS_GATHER && chains[L.recs[z].chain].write_kind >= FKB_WRITE_NV12);
        L.gather_ppt = gather_pixels < (yuv_write ? (1u << 17) : (2u << 20)) ? 1 : 4;
        L.gather_grid = dim3((gw + 32 * L.gather_ppt - 1) / (32 * L.gather_ppt), (gh + 7) / 8, std::min<uint32_t>(L.lp.gather_z1 - L.lp.gather_z0, 65535u));
        ++L.kernels;
    }
    return status_word(&L.lp.status);
}

// Whether the staged kernel of this launch gets a work counter.  With one, every warp takes its first item by position
// and claims the rest; without, it takes every n-th item.  Up to two items per warp the positions do as well as claims
// would (measured: 128 planes of 224 x 224, 1.5 items per warp, 25.1 us by position against 27.7 us with claims, which
// all arrive at the counter at once when the kernel starts).
bool wants_work_counter(const Lowered& L) {
    return L.staged_grid != 0 && L.lp.n_tiles > 2u * L.staged_grid * kStagedWarps;  // (n_split is zero below that)
}

int run(const Lowered& L, const LaunchParams& lp, cudaStream_t stream) {
    if (L.staged_grid) FKB_CUDA(launch_staged(lp, L.staged_grid, stream));
    if (L.lut_grid) FKB_CUDA(launch_lut(lp, L.lut_grid, stream));
    if (L.nv12_grid.x) FKB_CUDA(launch_nv12(lp, L.nv12_grid, stream));
    if (L.gather_grid.x) FKB_CUDA(launch_gather(lp, L.gather_grid, L.gather_ppt, stream));
    if (L.gather4_grid.x) FKB_CUDA(launch_gather4(lp, L.gather4_grid, stream));
    return FKB_OK;
}

// -------------------------------------------------------------------------------------------------------
// descriptor arena: plane records of launches too large for the kernel parameters travel through a ring of
// pinned-host / device slots; a slot is reused only after the launch that read it has finished.
// -------------------------------------------------------------------------------------------------------
struct Arena {
    static constexpr int kSlots = 4;
    std::mutex m;
    int device = -1;
    size_t slot_bytes = 0;
    uint8_t* pinned = nullptr;
    uint8_t* dev = nullptr;
    uint32_t* work = nullptr;
    cudaEvent_t ev[kSlots] = {};
    bool used[kSlots] = {};
    int next = 0;

    int ensure(size_t bytes) {
        if (bytes <= slot_bytes) return FKB_OK;
        for (int i = 0; i < kSlots; ++i)
            if (used[i]) { FKB_CUDA(cudaEventSynchronize(ev[i])); used[i] = false; }
        // the old buffers go first and the arena counts as empty until both new ones exist: a failed allocation must not
        // leave a slot size behind that no buffer backs
        slot_bytes = 0;
        if (pinned) { uint8_t* q = pinned; pinned = nullptr; FKB_CUDA(cudaFreeHost(q)); }
        if (dev) { uint8_t* q = dev; dev = nullptr; FKB_CUDA(cudaFree(q)); }
        size_t want = 1u << 20;
        while (want < bytes) want <<= 1;
        uint8_t* new_pinned = nullptr;
        uint8_t* new_dev = nullptr;
        FKB_CUDA(cudaMallocHost(reinterpret_cast<void**>(&new_pinned), want * kSlots));
        {
            const cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&new_dev), want * kSlots);
            if (e != cudaSuccess) {
                (void)cudaFreeHost(new_pinned);
                t_last_cuda_error = static_cast<int>(e);
                (void)cudaGetLastError();
                return FKB_ERR_CUDA;
            }
        }
        pinned = new_pinned; dev = new_dev;
        if (!work) {  // one pair of item counters per slot; a kernel leaves its pair at zero
            FKB_CUDA(cudaMalloc(reinterpret_cast<void**>(&work), sizeof(uint32_t) * 2 * kSlots));
            FKB_CUDA(cudaMemset(work, 0, sizeof(uint32_t) * 2 * kSlots));
        }
        if (!ev[0])
            for (int i = 0; i < kSlots; ++i) FKB_CUDA(cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming));
        slot_bytes = want;
        return FKB_OK;
    }
};

Arena& arena_for_current_device(int& rc) {
    static std::mutex m;
    static Arena arenas[64];
    static Arena overflow;
    int dev = 0;
    const cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { t_last_cuda_error = static_cast<int>(e); rc = FKB_ERR_CUDA; return overflow; }
    rc = FKB_OK;
    std::lock_guard<std::mutex> g(m);
    Arena& a = dev < 64 ? arenas[dev] : overflow;
    a.device = dev;
    return a;
}

// A launch that stages its plane records through host memory owned by the library (an arena slot, the fixed array of
// the no-allocation entry point) cannot be recorded into a CUDA graph: the recorded copy would read that memory again at
// every replay, long after another launch has overwritten it, and the arena's event waits are illegal on a capturing
// stream.  Such launches are refused while the stream is capturing; launches whose records travel in the kernel
// parameters, and plans, record fine.
int refuse_if_capturing(cudaStream_t stream) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    FKB_CUDA(cudaStreamIsCapturing(stream, &st));
    return st == cudaStreamCaptureStatusNone ? FKB_OK : FKB_ERR_UNSUPPORTED;
}

int launch_once(const fkb_chain_desc* chains, uint32_t n_chains, const fkb_plane_desc* planes, uint32_t n_planes,
                cudaStream_t stream) {
    Lowered L;
    int rc;
    if (n_planes <= kInlinePlanes) {
        // a few planes: the records are lowered on the stack and travel in the kernel parameters
        PlaneRec local[kInlinePlanes];
        L.recs = local;
        if ((rc = lower(chains, n_chains, planes, n_planes, L)) != FKB_OK) return rc;
        std::memcpy(L.lp.inline_planes, local, sizeof(PlaneRec) * n_planes);
        L.recs = nullptr;
        L.lp.table = nullptr;
        if (!wants_work_counter(L)) return run(L, L.lp, stream);
        // (a few planes large enough for the kernel to claim its items: a slot of the arena lends its pair of counters)
        if ((rc = refuse_if_capturing(stream)) != FKB_OK) return rc;
        Arena& a = arena_for_current_device(rc);
        if (rc != FKB_OK) return rc;
        std::lock_guard<std::mutex> g(a.m);
        if ((rc = a.ensure(1)) != FKB_OK) return rc;
        const int slot = a.next;
        a.next = (a.next + 1) % Arena::kSlots;
        if (a.used[slot]) { FKB_CUDA(cudaEventSynchronize(a.ev[slot])); a.used[slot] = false; }
        L.lp.work = a.work + 2 * slot;
        if ((rc = run(L, L.lp, stream)) != FKB_OK) return rc;
        FKB_CUDA(cudaEventRecord(a.ev[slot], stream));
        a.used[slot] = true;
        return FKB_OK;
    }
    // Many planes: the records are lowered straight into a pinned slot of the arena (no intermediate array, no second
    // copy) and uploaded from there; the slot also lends the launch its pair of item counters.
    if (planes == nullptr || chains == nullptr) return FKB_ERR_NULL;
    if ((rc = refuse_if_capturing(stream)) != FKB_OK) return rc;
    Arena& a = arena_for_current_device(rc);
    if (rc != FKB_OK) return rc;
    std::lock_guard<std::mutex> g(a.m);
    const size_t bytes = sizeof(PlaneRec) * n_planes;
    if ((rc = a.ensure(bytes)) != FKB_OK) return rc;
    const int slot = a.next;
    if (a.used[slot]) { FKB_CUDA(cudaEventSynchronize(a.ev[slot])); a.used[slot] = false; }
    uint8_t* h = a.pinned + static_cast<size_t>(slot) * a.slot_bytes;
    uint8_t* d = a.dev + static_cast<size_t>(slot) * a.slot_bytes;
    L.recs = reinterpret_cast<PlaneRec*>(h);
    if ((rc = lower(chains, n_chains, planes, n_planes, L)) != FKB_OK) return rc;  // (the slot stays free)
    a.next = (a.next + 1) % Arena::kSlots;
    FKB_CUDA(cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, stream));
    L.lp.table = reinterpret_cast<const PlaneRec*>(d);
    if (wants_work_counter(L)) L.lp.work = a.work + 2 * slot;
    rc = run(L, L.lp, stream);
    // (even if a kernel launch failed, the copy above may be in flight: the slot counts as used either way)
    FKB_CUDA(cudaEventRecord(a.ev[slot], stream));
    a.used[slot] = true;
    return rc;
}

// -------------------------------------------------------------------------------------------------------
// fkb_launch_transform_noalloc: the plane-record table lives in a fixed array inside the library image
// -------------------------------------------------------------------------------------------------------
// Device-side table of the allocation-free entry point.  Every GPU that loads this library carries these
// FKB_NOALLOC_MAX_PLANES * sizeof(PlaneRec) bytes (896 KB) until the process exits.  In host code this name is only a
// handle for cudaGetSymbolAddress, never an address a kernel may be given.
static __device__ __align__(256) unsigned char g_noalloc_table[FKB_NOALLOC_MAX_PLANES * sizeof(PlaneRec)];

struct NoAllocState {
    std::mutex m;
    PlaneRec* device_table[64] = {nullptr};  // per device: where g_noalloc_table lives on that device
    PlaneRec host_recs[FKB_NOALLOC_MAX_PLANES];  // lowering target; ordinary (pageable) memory of the library image
};
NoAllocState& noalloc_state() {
    static NoAllocState s;
    return s;
}

// The lowering of lower(), writing into a caller-provided array instead of a growing vector.
int launch_noalloc(const fkb_chain_desc* chain, const fkb_plane_desc* planes, uint32_t n_planes, cudaStream_t stream) {
    if (!chain || !planes) return FKB_ERR_NULL;
    if (n_planes > FKB_NOALLOC_MAX_PLANES) return FKB_ERR_TOO_LARGE;  // the fixed table holds no more
    for (uint32_t z = 0; z < n_planes; ++z)
        if ((planes[z].chain & ~FKB_PLANE_DEFAULT) != 0) return FKB_ERR_INVALID;
    {
        const int rc = refuse_if_capturing(stream);
        if (rc != FKB_OK) return rc;
    }
    NoAllocState& st = noalloc_state();
    std::lock_guard<std::mutex> g(st.m);
    int dev = 0;
    FKB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return FKB_ERR_UNSUPPORTED;
    if (!st.device_table[dev]) {
        // set-up, once per device, with that device current: ask the runtime where the array lives on it
        PlaneRec* ptr = nullptr;
        FKB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_table));
        st.device_table[dev] = ptr;
    }
    // the same lowering as every other launch, writing its records into the fixed host array (no container grows)
    Lowered L;
    L.recs = st.host_recs;
    const int rc = lower(chain, 1, planes, n_planes, L);
    if (rc != FKB_OK) return rc;
    // Every record the kernels will read is rewritten by this copy; nothing in the table has to start at zero.  The
    // source is pageable memory: outside a stream capture (refused above) the runtime has taken the records out of
    // st.host_recs by the time the call returns, so the next call may overwrite them.
    FKB_CUDA(cudaMemcpyAsync(st.device_table[dev], st.host_recs, sizeof(PlaneRec) * n_planes, cudaMemcpyHostToDevice, stream));
    L.lp.table = st.device_table[dev];
    return run(L, L.lp, stream);  // (no work counter: items are dealt round-robin)
}

}  // namespace
}  // namespace fkb

// Item counters of a plan's staged kernel: a ring of pairs, one pair per launch in turn.  A kernel leaves its pair at
// zero, so a pair is ready again when the launch that used it has finished; launches of one plan may therefore overlap
// on the GPU (different streams) as long as fewer than kPlanCounterPairs of them are in flight at once.
constexpr uint32_t kPlanCounterPairs = 64;
struct fkb_plan {
    fkb::Lowered L;
    fkb::PlaneRec* table = nullptr;
    uint32_t* work = nullptr;
    mutable std::atomic<uint32_t> launches{0};
    int device = 0;
};

using namespace fkb;

extern "C" {

int fkb_resize_params(uint32_t geometry, fkb_plane_desc* pl) {
    if (!pl) return FKB_ERR_NULL;
    const int sw = pl->crop_w, sh = pl->crop_h;
    const int dw = static_cast<int>(pl->dst_w), dh = static_cast<int>(pl->dst_h);
    if (sw <= 0 || sh <= 0 || dw <= 0 || dh <= 0) return FKB_ERR_INVALID;
    int tw = dw, th = dh;
    if (geometry >= FKB_GEOM_RESIZE_PRESERVE_AR && geometry <= FKB_GEOM_RESIZE_PRESERVE_AR_LEFT) {
        // compute_target_size: fit the height first, fall back to fitting the width; RN_EVEN rounds the fitted
        // dimension down to an even number (and tests the evened width against the destination)
        const bool even = geometry == FKB_GEOM_RESIZE_PRESERVE_AR_RN_EVEN;
        const float by_height = static_cast<float>(dh) / static_cast<float>(sh);
        tw = static_cast<int>(std::round(by_height * static_cast<float>(sw)));
        if (even) tw -= tw % 2;
        if (tw > dw) {
            const float by_width = static_cast<float>(dw) / static_cast<float>(sw);
            tw = dw;
            th = static_cast<int>(std::round(by_width * static_cast<float>(sh)));
            if (even) th -= th % 2;
        }
    } else if (geometry != FKB_GEOM_RESIZE_IGNORE_AR) {
        return FKB_ERR_INVALID;
    }
    const double cfx = static_cast<double>(tw) / static_cast<double>(sw);
    const double cfy = static_cast<double>(th) / static_cast<double>(sh);
    pl->fx = static_cast<float>(1.0 / cfx);
    pl->fy = static_cast<float>(1.0 / cfy);
    pl->x1 = geometry == FKB_GEOM_RESIZE_PRESERVE_AR_LEFT ? 0 : (dw - tw) / 2;
    pl->y1 = (dh - th) / 2;
    pl->x2 = pl->x1 + tw - 1;
    pl->y2 = pl->y1 + th - 1;
    return FKB_OK;
}

int fkb_ycbcr_to_rgb(uint32_t range, uint32_t primitives, float ccm[9], float yuv_sub[3]) {
    return fkb_ycbcr_to_rgb_bits(8, range, primitives, ccm, yuv_sub);
}

int fkb_ycbcr_to_rgb_bits(uint32_t bits, uint32_t range, uint32_t primitives, float ccm[9], float yuv_sub[3]) {
    if (!ccm || !yuv_sub) return FKB_ERR_NULL;
    if (range > FKB_RANGE_FULL || primitives > FKB_PRIMITIVES_BT2020 || (bits != 8 && bits != 10 && bits != 12)) return FKB_ERR_INVALID;
    // per depth: the largest code, the luma and chroma offsets, the luma and chroma spans of limited range
    const float max_v = bits == 8 ? 255.f : bits == 10 ? 1023.f : 4095.f;
    const float sub_y = bits == 8 ? 16.f : bits == 10 ? 64.f : 256.f, sub_c = bits == 8 ? 128.f : bits == 10 ? 512.f : 2048.f;
    const float lim_y = bits == 8 ? 219.f : bits == 10 ? 876.f : 3504.f, lim_c = bits == 8 ? 224.f : bits == 10 ? 896.f : 3584.f;
    // luma weights of Rec. BT.601 / BT.709 / BT.2020; every step below is an fp32 operation, in this order
    static const float kKr[3] = {0.299f, 0.2126f, 0.2627f}, kKb[3] = {0.114f, 0.0722f, 0.0593f};
    const float Kr = kKr[primitives], Kb = kKb[primitives];
    const float Kg = 1.0f - Kr - Kb;
    float m[3][3] = {{1.0f, 0.0f, 2.0f * (1.0f - Kr)},
                     {1.0f, -2.0f * Kb * (1.0f - Kb) / Kg, -2.0f * Kr * (1.0f - Kr) / Kg},
                     {1.0f, 2.0f * (1.0f - Kb), 0.0f}};
    if (range == FKB_RANGE_LIMITED) {  // (8 bit: luma spans 219 codes from 16, chroma 224 around 128)
        const float scale_y = max_v / lim_y, scale_c = max_v / lim_c;
        for (int i = 0; i < 3; ++i) { m[i][0] *= scale_y; m[i][1] *= scale_c; m[i][2] *= scale_c; }
    }
    for (int i = 0; i < 9; ++i) ccm[i] = m[i / 3][i % 3];
    yuv_sub[0] = range == FKB_RANGE_LIMITED ? sub_y : 0.f;  // full range subtracts nothing from the luma
    yuv_sub[1] = yuv_sub[2] = sub_c;
    return FKB_OK;
}

int fkb_rgb_to_ycbcr(uint32_t range, uint32_t primitives, float ccm2[9], float yuv_add[3]) {
    if (!ccm2 || !yuv_add) return FKB_ERR_NULL;
    if (range > FKB_RANGE_FULL || primitives > FKB_PRIMITIVES_BT2020) return FKB_ERR_INVALID;
    static const float kKr[3] = {0.299f, 0.2126f, 0.2627f}, kKb[3] = {0.114f, 0.0722f, 0.0593f};
    const float Kr = kKr[primitives], Kb = kKb[primitives];
    const float Kg = 1.0f - Kr - Kb;
    float m[3][3] = {{Kr, Kg, Kb},
                     {-Kr / (2.0f * (1.0f - Kb)), -Kg / (2.0f * (1.0f - Kb)), 0.5f},
                     {0.5f, -Kg / (2.0f * (1.0f - Kr)), -Kb / (2.0f * (1.0f - Kr))}};
    if (range == FKB_RANGE_LIMITED) {  // 8 bit: 219 luma codes, 224 chroma codes out of 255
        const float scale_y = 219.f / 255.f, scale_c = 224.f / 255.f;
        for (int i = 0; i < 3; ++i) { m[0][i] *= scale_y; m[1][i] *= scale_c; m[2][i] *= scale_c; }
    }
    for (int i = 0; i < 9; ++i) ccm2[i] = m[i / 3][i % 3];
    yuv_add[0] = range == FKB_RANGE_LIMITED ? 16.f : 0.f;
    yuv_add[1] = yuv_add[2] = 128.f;
    return FKB_OK;
}

int fkb_validate(const fkb_chain_desc* chains, uint32_t n_chains, const fkb_plane_desc* planes, uint32_t n_planes) {
    return validate(chains, n_chains, planes, n_planes);
}

int fkb_launch_transform(const fkb_chain_desc* chain, const fkb_plane_desc* planes, uint32_t n_planes, void* cuda_stream) {
    const NvtxRange range("fkb_launch_transform");
    if (!chain || !planes) return FKB_ERR_NULL;
    for (uint32_t z = 0; z < n_planes; ++z)
        if ((planes[z].chain & ~FKB_PLANE_DEFAULT) != 0) return FKB_ERR_INVALID;
    return launch_once(chain, 1, planes, n_planes, static_cast<cudaStream_t>(cuda_stream));
}

int fkb_launch_transform_noalloc(const fkb_chain_desc* chain, const fkb_plane_desc* planes, uint32_t n_planes, void* cuda_stream) {
    const NvtxRange range("fkb_launch_transform_noalloc");
    return launch_noalloc(chain, planes, n_planes, static_cast<cudaStream_t>(cuda_stream));
}

int fkb_launch_divergent(const fkb_chain_desc* chains, uint32_t n_chains, const fkb_plane_desc* planes,
                         uint32_t n_planes, void* cuda_stream) {
    const NvtxRange range("fkb_launch_divergent");
    return launch_once(chains, n_chains, planes, n_planes, static_cast<cudaStream_t>(cuda_stream));
}

int fkb_plan_create(const fkb_chain_desc* chains, uint32_t n_chains, const fkb_plane_desc* planes, uint32_t n_planes,
                    fkb_plan** out) {
    if (!out) return FKB_ERR_NULL;
    *out = nullptr;
    fkb_plan* plan = new (std::nothrow) fkb_plan();
    if (!plan) return FKB_ERR_TOO_LARGE;
    int rc = lower(chains, n_chains, planes, n_planes, plan->L);
    if (rc != FKB_OK) { delete plan; return rc; }
    cudaError_t e = cudaGetDevice(&plan->device);
    if (e == cudaSuccess && wants_work_counter(plan->L)) {
        e = cudaMalloc(reinterpret_cast<void**>(&plan->work), 2 * sizeof(uint32_t) * kPlanCounterPairs);
        if (e == cudaSuccess) e = cudaMemset(plan->work, 0, 2 * sizeof(uint32_t) * kPlanCounterPairs);
        plan->L.lp.work = plan->work;
    }
    if (n_planes <= kInlinePlanes) {
        // a few planes travel in the kernel parameters, as in fkb_launch_transform: no table read before the first tap
        if (e != cudaSuccess) { t_last_cuda_error = static_cast<int>(e); (void)cudaGetLastError(); if (plan->work) cudaFree(plan->work); delete plan; return FKB_ERR_CUDA; }
        std::memcpy(plan->L.lp.inline_planes, plan->L.recs, sizeof(PlaneRec) * n_planes);
        plan->L.lp.table = nullptr;
        *out = plan;
        return FKB_OK;
    }
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&plan->table), sizeof(PlaneRec) * n_planes);
    if (e == cudaSuccess) e = cudaMemcpy(plan->table, plan->L.recs, sizeof(PlaneRec) * n_planes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        t_last_cuda_error = static_cast<int>(e);
        (void)cudaGetLastError();
        if (plan->table) cudaFree(plan->table);
        if (plan->work) cudaFree(plan->work);
        delete plan;
        return FKB_ERR_CUDA;
    }
    plan->L.lp.table = plan->table;
    *out = plan;
    return FKB_OK;
}

int fkb_plan_launch(const fkb_plan* plan, void* cuda_stream) {
    const NvtxRange range("fkb_plan_launch");
    if (!plan) return FKB_ERR_NULL;
    // a plan belongs to the device it was created on (its plane table and its status word live there)
    int dev = -1;
    FKB_CUDA(cudaGetDevice(&dev));
    if (dev != plan->device) return FKB_ERR_INVALID;
    if (!plan->work) return run(plan->L, plan->L.lp, static_cast<cudaStream_t>(cuda_stream));
    LaunchParams lp = plan->L.lp;  // this launch's own pair of item counters
    lp.work = plan->work + 2u * (plan->launches.fetch_add(1u, std::memory_order_relaxed) % kPlanCounterPairs);
    return run(plan->L, lp, static_cast<cudaStream_t>(cuda_stream));
}

void fkb_plan_destroy(fkb_plan* plan) {
    if (!plan) return;
    if (plan->table) cudaFree(plan->table);
    if (plan->work) cudaFree(plan->work);
    delete plan;
}

uint32_t fkb_plan_kernel_launches(const fkb_plan* plan) { return plan ? plan->L.kernels : 0; }

int fkb_device_status(void) {
    int* w = nullptr;
    const int rc = status_word(&w);
    if (rc != FKB_OK) return rc;
    FKB_CUDA(cudaDeviceSynchronize());
    int v = 0;
    FKB_CUDA(cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) {
        const int zero = 0;
        FKB_CUDA(cudaMemcpy(w, &zero, sizeof(int), cudaMemcpyHostToDevice));
    }
    return v;
}

int fkb_last_cuda_error(void) { return t_last_cuda_error; }

const char* fkb_status_string(int status) {
    switch (status) {
    case FKB_OK: return "ok";
    case FKB_ERR_NULL: return "a required pointer is null";
    case FKB_ERR_INVALID: return "invalid descriptor";
    case FKB_ERR_UNSUPPORTED: return "unsupported chain";
    case FKB_ERR_CUDA: return "CUDA runtime error";
    case FKB_ERR_TOO_LARGE: return "launch too large";
    case FKB_ERR_DEVICE_WAIT: return "a bounded device-side wait ran out";
    case FKB_ERR_DEVICE_CHECK: return "the self-checking build found an access outside its buffer and skipped it";
    default: return "unknown status";
    }
}

uint32_t fkb_abi_version(void) { return FKB_ABI_VERSION; }

}  // extern "C"
