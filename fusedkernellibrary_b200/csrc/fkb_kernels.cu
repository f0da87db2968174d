// The two sm_100a kernels behind fkb_launch_*:
//
//   staged_kernel  — persistent CTAs (two per SM) of autonomous warps.  Each warp walks a strided list of items
//                    (a block of output rows of one plane) and runs its own pipeline per output row: (1) the
//                    row's bounded source footprint (one or two source rows) is staged into the warp's slice of
//                    shared memory with non-multicast bulk async copies (cp.async.bulk, completion on the
//                    warp's mbarrier), double-buffered so the next row is in flight while this one is computed,
//                    (2) the row is computed from shared memory into a shared output row and (3) leaves with a
//                    bulk async store (full 16-byte-aligned lines, no partial sectors).  No __syncthreads
//                    anywhere: warps never wait for each other.  Two item kinds: POINT (no resampling, 16 or 4
//                    pixels per lane, 128-bit shared accesses) and RESIZE (bilinear from the staged rows).  The
//                    chain of a plane is picked once per item, so a divergent launch never diverges in a warp.
//   gather_kernel  — the general path: any source format (uchar3, NV12), ops before the interpolation, planar
//                    writes, unaligned buffers, or footprints too sparse/large to stage (heavy decimation).
//                    Four pixels per thread, read-only global loads, vector stores when aligned.
//
// Replaces launchTransformDPP_Kernel / launchDivergentBatchTransformDPP_Kernel of the reference
// (core/execution_model/executor_details/executor_kernels.h:20-30).  No tensor cores: nothing here is a
// contraction; the bound is HBM bandwidth.
#include <cstdlib>
#include "fkb_device.cuh"
#include "fkb_launch.h"

namespace fkb {

__device__ int g_status_word;  // what fkb_device_status() reads; LaunchParams::status points here

// ---------------------------------------------------------------------------------------------------------
// shared helpers
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ const PlaneRec* plane_table(const LaunchParams& p) {
    return p.table ? p.table : p.inline_planes;
}

// Frame pixel (X,Y) as three floats (uchar3 channels, or Y / Cb / Cr).
__device__ __forceinline__ void read_frame_global(const fkb_chain_desc& ch, const PlaneRec& pl, size_t X, size_t Y, float (&o)[3]) {
    if (kSelfChecking && !self_check(&g_status_word, X < pl.src_w && Y < pl.src_h)) { o[0] = o[1] = o[2] = 0.f; return; }
    switch (ch.src_format) {
    case FKB_PIX_NV12: case FKB_PIX_NV21: {
        const uint8_t* uv = pl.src_chroma + (Y >> 1) * pl.src_pitch + (X >> 1) * 2;
        const uint32_t vu = ch.src_format == FKB_PIX_NV21;  // V first
        o[0] = static_cast<float>(__ldg(pl.src + Y * pl.src_pitch + X));
        o[1] = static_cast<float>(__ldg(uv + vu));
        o[2] = static_cast<float>(__ldg(uv + (vu ^ 1u)));
        break;
    }
    case FKB_PIX_UYVY: {
        const uint8_t* g = pl.src + Y * pl.src_pitch + (X >> 1) * 4;  // U Y0 V Y1
        o[0] = static_cast<float>(__ldg(g + 1 + 2 * (X & 1)));
        o[1] = static_cast<float>(__ldg(g));
        o[2] = static_cast<float>(__ldg(g + 2));
        break;
    }
    case FKB_PIX_P010: case FKB_PIX_P210: {  // ushort luma plane, ushort2 chroma rows (every second row for 4:2:0)
        const size_t cy = ch.src_format == FKB_PIX_P010 ? (Y >> 1) : Y;
        const unsigned short* uv = reinterpret_cast<const unsigned short*>(pl.src_chroma + cy * pl.src_pitch) + (X >> 1) * 2;
        o[0] = static_cast<float>(__ldg(reinterpret_cast<const unsigned short*>(pl.src + Y * pl.src_pitch) + X));
        o[1] = static_cast<float>(__ldg(uv));
        o[2] = static_cast<float>(__ldg(uv + 1));
        break;
    }
    case FKB_PIX_Y210: {  // ushort4 groups Y0 U Y1 V
        const unsigned short* g = reinterpret_cast<const unsigned short*>(pl.src + Y * pl.src_pitch) + (X >> 1) * 4;
        o[0] = static_cast<float>(__ldg(g + 2 * (X & 1)));
        o[1] = static_cast<float>(__ldg(g + 1));
        o[2] = static_cast<float>(__ldg(g + 3));
        break;
    }
    case FKB_PIX_F32C3: {
        const float* q = reinterpret_cast<const float*>(pl.src + Y * pl.src_pitch) + X * 3;
        o[0] = __ldg(q); o[1] = __ldg(q + 1); o[2] = __ldg(q + 2);
        break;
    }
    case FKB_PIX_F32P3: {
        const size_t step = static_cast<size_t>(pl.src_chroma - pl.src);  // bytes between channel planes
        const uint8_t* q = pl.src + Y * pl.src_pitch + X * 4;
        o[0] = __ldg(reinterpret_cast<const float*>(q)); o[1] = __ldg(reinterpret_cast<const float*>(q + step));
        o[2] = __ldg(reinterpret_cast<const float*>(q + 2 * step));
        break;
    }
    default: {  // uchar3, or uchar4 whose alpha byte is not read
        const uint8_t* q = pl.src + Y * pl.src_pitch + X * (ch.src_format == FKB_PIX_U8C4 ? 4u : 3u);
        o[0] = static_cast<float>(__ldg(q));
        o[1] = static_cast<float>(__ldg(q + 1));
        o[2] = static_cast<float>(__ldg(q + 2));
        break;
    }
    }
}
// Index maps of the reference's BorderReader modes (border_reader.h:211-330), idx = low(high(i)); n is the frame extent.
__device__ __forceinline__ int border_index(uint32_t mode, int i, int n) {
    const int last = n - 1;
    switch (mode) {
    case FKB_BORDER_REPLICATE: return max(min(i, last), 0);
    case FKB_BORDER_REFLECT: {
        const int hi = last - abs(last - i) + (i > last ? 1 : 0);
        return (abs(hi) - (hi < 0 ? 1 : 0)) % n;
    }
    case FKB_BORDER_WRAP: {
        const int hi = i < n ? i : i % n;
        return hi >= 0 ? hi : hi - ((hi - n + 1) / n) * n;
    }
    case FKB_BORDER_REFLECT_101: return abs(abs(last - abs(last - i)) % n) % n;
    default: return i;
    }
}
// Crop-relative pixel (cx,cy) of a plane: the Crop adds its (signed) origin, a BorderReader maps what leaves the frame.
// Returns true when the tap lies outside the frame of a CONSTANT border: nothing is read and the caller substitutes
// the chain's border value.
__device__ __forceinline__ bool read_tap_global(const fkb_chain_desc& ch, const PlaneRec& pl, int cx, int cy, float (&o)[3]) {
    int X = cx + static_cast<int>(pl.crop_x), Y = cy + static_cast<int>(pl.crop_y);
    if (ch.border) {
        const int w = static_cast<int>(pl.src_w), h = static_cast<int>(pl.src_h);
        if (ch.border == FKB_BORDER_CONSTANT) {
            if (X < 0 || X >= w || Y < 0 || Y >= h) { o[0] = o[1] = o[2] = 0.f; return true; }
        } else {
            X = border_index(ch.border, X, w);
            Y = border_index(ch.border, Y, h);
        }
    }
    read_frame_global(ch, pl, static_cast<size_t>(X), static_cast<size_t>(Y), o);
    return false;
}
// ops[first..last) on N values of which some (mask bit n) are constant-border taps: those take the border value after
// the ops that precede the BorderReader.
template <int N>
__device__ __forceinline__ void apply_ops_bordered(float (&v)[N][3], const fkb_chain_desc& ch, const PlaneRec& pl, uint32_t last, uint32_t outside) {
    if (outside == 0u) { apply_ops<N>(v, ch, pl, 0, last); return; }
    apply_ops<N>(v, ch, pl, 0, ch.border_at);
#pragma unroll
    for (int n = 0; n < N; ++n)
        if ((outside >> n) & 1u) { v[n][0] = ch.border_value[0]; v[n][1] = ch.border_value[1]; v[n][2] = ch.border_value[2]; }
    apply_ops<N>(v, ch, pl, ch.border_at, last);
}

// ---------------------------------------------------------------------------------------------------------
// gather_kernel
// ---------------------------------------------------------------------------------------------------------
// PPT pixels per thread: 4 for large launches (vector stores), 1 for small ones (more threads hide the tap latency).
// INLINE: the plane records are kernel parameters (launches of a few planes): they are read where they lie, through the
// constant bank, instead of being copied to shared memory first — two block-wide barriers less per plane, which is most
// of what a launch of a few ten thousand pixels can save.
template <int PPT, bool INLINE>
__global__ void __launch_bounds__(256) gather_kernel(const __grid_constant__ LaunchParams p) {
    pdl_signal();
    pdl_wait();
    __shared__ PlaneRec s_pl;
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (uint32_t z = p.gather_z0 + blockIdx.z; z < p.gather_z1; z += gridDim.z) {
        if (!INLINE) {
            __syncthreads();
            if (threadIdx.x < sizeof(PlaneRec) / 16)
                reinterpret_cast<uint4*>(&s_pl)[threadIdx.x] = reinterpret_cast<const uint4*>(p.table + z)[threadIdx.x];
            __syncthreads();
        }
        const PlaneRec& pl = INLINE ? p.inline_planes[z] : s_pl;
        if (pl.kclass != KCLASS_GATHER) continue;
        const fkb_chain_desc& ch = p.chains[pl.chain];
        const uint32_t y = blockIdx.y * 8 + ty;
        const uint32_t x0 = (blockIdx.x * 32 + tx) * PPT;
        if (y >= pl.dst_h || x0 >= pl.dst_w) continue;
        const uint32_t nvalid = min(static_cast<uint32_t>(PPT), pl.dst_w - x0);

        float v[PPT][3];
        if (pl.src == nullptr) {
            // a plane whose read yields its default value (beyond usedPlanes of a conditional batch read)
#pragma unroll
            for (int n = 0; n < PPT; ++n) { v[n][0] = pl.bg[0]; v[n][1] = pl.bg[1]; v[n][2] = pl.bg[2]; }
            apply_ops<PPT>(v, ch, pl, ch.geometry == FKB_GEOM_NONE ? 0 : ch.n_pre_ops, ch.n_ops);
        } else if (ch.geometry == FKB_GEOM_NONE) {
            uint32_t outside = 0;
            const uint8_t* q12 = pl.src + static_cast<size_t>(pl.crop_y + y) * pl.src_pitch + static_cast<size_t>(pl.crop_x + x0) * 3;
            if (PPT == 4 && nvalid == 4 && ch.src_format == FKB_PIX_U8C3 && !ch.border && (reinterpret_cast<uintptr_t>(q12) & 3) == 0) {
                // four packed byte pixels = three aligned words
                const uint32_t* q4 = reinterpret_cast<const uint32_t*>(q12);
                const uint32_t w3[3] = {__ldg(q4), __ldg(q4 + 1), __ldg(q4 + 2)};
#pragma unroll
                for (int b = 0; b < 12; ++b) v[(b / 3) % PPT][b % 3] = static_cast<float>((w3[b >> 2] >> (8 * (b & 3))) & 0xffu);
            } else {
#pragma unroll
                for (int n = 0; n < PPT; ++n) {
                    if (n < nvalid) outside |= static_cast<uint32_t>(read_tap_global(ch, pl, static_cast<int>(x0) + n, static_cast<int>(y), v[n])) << n;
                    else { v[n][0] = v[n][1] = v[n][2] = 0.f; }
                }
            }
            apply_ops_bordered<PPT>(v, ch, pl, ch.n_ops, outside);
        } else {
            const bool par = ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR;
            const int ox = par ? pl.x1 : 0, oy = par ? pl.y1 : 0;
            const bool row_in = !par || (static_cast<int>(y) >= pl.y1 && static_cast<int>(y) <= pl.y2);
            const AxisTap ay = axis_tap(row_in ? static_cast<int>(y) - oy : 0, pl.fy, pl.crop_h);
#pragma unroll
            for (int n = 0; n < PPT; ++n) {
                const int x = static_cast<int>(x0) + n;
                const bool inside = n < nvalid && row_in && (!par || (x >= pl.x1 && x <= pl.x2));
                if (inside) {
                    const AxisTap ax = axis_tap(x - ox, pl.fx, pl.crop_w);
                    float t[4][3];
                    uint32_t outside = read_tap_global(ch, pl, ax.i0, ay.i0, t[0]) ? 1u : 0u;
                    outside |= read_tap_global(ch, pl, ax.i1, ay.i0, t[1]) ? 2u : 0u;
                    outside |= read_tap_global(ch, pl, ax.i0, ay.i1, t[2]) ? 4u : 0u;
                    outside |= read_tap_global(ch, pl, ax.i1, ay.i1, t[3]) ? 8u : 0u;
                    apply_ops_bordered<4>(t, ch, pl, ch.n_pre_ops, outside);
                    const float w00 = __fmul_rn(ax.w0, ay.w0), w10 = __fmul_rn(ax.w1, ay.w0);
                    const float w01 = __fmul_rn(ax.w0, ay.w1), w11 = __fmul_rn(ax.w1, ay.w1);
#pragma unroll
                    for (int c = 0; c < 3; ++c) v[n][c] = bilerp(t[0][c], t[1][c], t[2][c], t[3][c], w00, w10, w01, w11);
                } else {
                    v[n][0] = pl.bg[0]; v[n][1] = pl.bg[1]; v[n][2] = pl.bg[2];
                }
            }
            apply_ops<PPT>(v, ch, pl, ch.n_pre_ops, ch.n_ops);
        }

        uint8_t* row = pl.dst + static_cast<size_t>(y) * pl.dst_pitch;
        if (ch.dst_format == FKB_PIX_U8C1 || ch.dst_format == FKB_PIX_F32C1) {
            // one channel (after FKB_OP_RGB2GRAY): channel 0 of each pixel
            if (ch.dst_format == FKB_PIX_F32C1) {
                float* f = reinterpret_cast<float*>(row) + x0;
                if (PPT == 4 && nvalid == 4 && (reinterpret_cast<uintptr_t>(f) & 15) == 0) *reinterpret_cast<float4*>(f) = make_float4(v[0][0], v[1 % PPT][0], v[2 % PPT][0], v[3 % PPT][0]);
                else for (uint32_t n = 0; n < nvalid; ++n) f[n] = v[n][0];
            } else {
                uint8_t* q = row + x0;
                if (PPT == 4 && nvalid == 4 && (reinterpret_cast<uintptr_t>(q) & 3) == 0)
                    *reinterpret_cast<uint32_t*>(q) = static_cast<uint32_t>(v[0][0]) | (static_cast<uint32_t>(v[1 % PPT][0]) << 8) |
                                                      (static_cast<uint32_t>(v[2 % PPT][0]) << 16) | (static_cast<uint32_t>(v[3 % PPT][0]) << 24);
                else for (uint32_t n = 0; n < nvalid; ++n) q[n] = static_cast<uint8_t>(v[n][0]);
            }
        } else if (ch.write_kind >= FKB_WRITE_NV12 && PPT == 4 && nvalid == 4 && (pl.dst_pitch & 7u) == 0 &&
            (reinterpret_cast<uintptr_t>(pl.dst) & 7u) == 0 && (pl.dst_cstride & 3u) == 0) {
            // four pixels of a YCbCr image with word stores (x0 is a multiple of four: two whole chroma pairs)
            uint32_t b[4][3];
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int c = 0; c < 3; ++c) b[n][c] = static_cast<uint32_t>(v[n % PPT][c]);
            if (ch.write_kind == FKB_WRITE_UYVY) {
                *reinterpret_cast<uint2*>(row + static_cast<size_t>(x0) * 2) =
                    make_uint2(b[0][1] | (b[0][0] << 8) | (b[0][2] << 16) | (b[1][0] << 24), b[2][1] | (b[2][0] << 8) | (b[2][2] << 16) | (b[3][0] << 24));
            } else {
                *reinterpret_cast<uint32_t*>(row + x0) = b[0][0] | (b[1][0] << 8) | (b[2][0] << 16) | (b[3][0] << 24);
                uint32_t* uv = reinterpret_cast<uint32_t*>(pl.dst + pl.dst_cstride + static_cast<size_t>(y >> 1) * pl.dst_pitch + x0);
                if (ch.write_kind == FKB_WRITE_NV12) {
                    if (!(y & 1u)) *uv = b[0][1] | (b[0][2] << 8) | (b[2][1] << 16) | (b[2][2] << 24);   // the block's first pixel
                } else if (y == min(y | 1u, pl.dst_h - 1u)) {
                    *uv = b[1][2] | (b[1][1] << 8) | (b[3][2] << 16) | (b[3][1] << 24);                  // the block's last pixel, V first
                }
            }
        } else if (ch.write_kind >= FKB_WRITE_NV12) {
            // (Y,Cb,Cr) byte triples into a YCbCr image; the chroma rows of NV12 / NV21 start dst_cstride bytes after dst
            for (uint32_t n = 0; n < nvalid; ++n) {
                const uint32_t x = x0 + n;
                const uint8_t yy = static_cast<uint8_t>(v[n][0]), cb = static_cast<uint8_t>(v[n][1]), cr = static_cast<uint8_t>(v[n][2]);
                if (ch.write_kind == FKB_WRITE_UYVY) {
                    uint8_t* g = row + static_cast<size_t>(x >> 1) * 4;
                    if (x & 1u) g[3] = yy; else { g[0] = cb; g[1] = yy; g[2] = cr; }
                } else {
                    row[x] = yy;
                    uint8_t* uv = pl.dst + pl.dst_cstride + static_cast<size_t>(y >> 1) * pl.dst_pitch + static_cast<size_t>(x >> 1) * 2;
                    if (ch.write_kind == FKB_WRITE_NV12) {
                        if (!(x & 1u) && !(y & 1u)) { uv[0] = cb; uv[1] = cr; }
                    } else if (x == min(x | 1u, pl.dst_w - 1u) && y == min(y | 1u, pl.dst_h - 1u)) {  // last pixel of the 2x2 block
                        uv[0] = cr; uv[1] = cb;
                    }
                }
            }
        } else if (ch.write_kind != FKB_WRITE_PACKED) {
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                uint8_t* q = row + channel_offset(pl, c);
                if (ch.dst_format == FKB_PIX_F32C3) {
                    float* f = reinterpret_cast<float*>(q) + x0;
                    if (PPT == 4 && nvalid == 4 && (reinterpret_cast<uintptr_t>(f) & 15) == 0) {
                        *reinterpret_cast<float4*>(f) = make_float4(v[0][c], v[1 % PPT][c], v[2 % PPT][c], v[3 % PPT][c]);
                    } else {
                        for (uint32_t n = 0; n < nvalid; ++n) f[n] = v[n][c];
                    }
                } else {
                    for (uint32_t n = 0; n < nvalid; ++n) q[x0 + n] = static_cast<uint8_t>(v[n][c]);
                }
            }
        } else if (ch.dst_format == FKB_PIX_F32C3) {
            float* f = reinterpret_cast<float*>(row) + static_cast<size_t>(x0) * 3;
            if (PPT == 4 && nvalid == 4 && (reinterpret_cast<uintptr_t>(f) & 15) == 0) {
                float4* f4 = reinterpret_cast<float4*>(f);
                f4[0] = make_float4(v[0][0], v[0][1], v[0][2], v[1 % PPT][0]);
                f4[1] = make_float4(v[1 % PPT][1], v[1 % PPT][2], v[2 % PPT][0], v[2 % PPT][1]);
                f4[2] = make_float4(v[2 % PPT][2], v[3 % PPT][0], v[3 % PPT][1], v[3 % PPT][2]);
            } else {
                for (uint32_t n = 0; n < nvalid; ++n) { f[3 * n] = v[n][0]; f[3 * n + 1] = v[n][1]; f[3 * n + 2] = v[n][2]; }
            }
        } else {
            uint8_t* q = row + static_cast<size_t>(x0) * 3;
            if (PPT == 4 && nvalid == 4 && (reinterpret_cast<uintptr_t>(q) & 3) == 0) {
                uint32_t b[12];
#pragma unroll
                for (int n = 0; n < 4; ++n)
#pragma unroll
                    for (int c = 0; c < 3; ++c) b[3 * n + c] = static_cast<uint32_t>(v[n % PPT][c]);
                uint32_t* q4 = reinterpret_cast<uint32_t*>(q);
#pragma unroll
                for (int k = 0; k < 3; ++k) q4[k] = b[4 * k] | (b[4 * k + 1] << 8) | (b[4 * k + 2] << 16) | (b[4 * k + 3] << 24);
            } else {
                for (uint32_t n = 0; n < nvalid; ++n) {
                    q[3 * n] = static_cast<uint8_t>(v[n][0]); q[3 * n + 1] = static_cast<uint8_t>(v[n][1]); q[3 * n + 2] = static_cast<uint8_t>(v[n][2]);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// gather4_kernel: chains that write four channels (uchar4 | uchar3 + opaque alpha -> ... -> uchar4 | float4)
// ---------------------------------------------------------------------------------------------------------
// One output pixel per thread; a source pixel is one 32-bit load.  The ops are Cast, Mul / Add / Sub / Div with four
// operands (the fourth in fkb_chain_desc::op_w or PlaneRec::params_w), the BGRA <-> RGBA reorder and SaturateCast.
__device__ __forceinline__ bool read_tap4(const fkb_chain_desc& ch, const PlaneRec& pl, int cx, int cy, float (&o)[4]) {
    int X = cx + static_cast<int>(pl.crop_x), Y = cy + static_cast<int>(pl.crop_y);
    if (ch.border) {
        const int w = static_cast<int>(pl.src_w), h = static_cast<int>(pl.src_h);
        if (ch.border == FKB_BORDER_CONSTANT) {
            if (X < 0 || X >= w || Y < 0 || Y >= h) { o[0] = o[1] = o[2] = o[3] = 0.f; return true; }
        } else {
            X = border_index(ch.border, X, w);
            Y = border_index(ch.border, Y, h);
        }
    }
    if (kSelfChecking && !self_check(&g_status_word, X >= 0 && Y >= 0 && static_cast<uint32_t>(X) < pl.src_w && static_cast<uint32_t>(Y) < pl.src_h)) {
        o[0] = o[1] = o[2] = o[3] = 0.f;
        return false;
    }
    if (ch.src_format == FKB_PIX_U8C3) {  // three channels until FKB_OP_ADD_ALPHA appends the fourth
        const uint8_t* q3 = pl.src + static_cast<size_t>(Y) * pl.src_pitch + static_cast<size_t>(X) * 3;
        o[0] = static_cast<float>(__ldg(q3)); o[1] = static_cast<float>(__ldg(q3 + 1)); o[2] = static_cast<float>(__ldg(q3 + 2));
        o[3] = 0.f;
        return false;
    }
    const uint8_t* q = pl.src + static_cast<size_t>(Y) * pl.src_pitch + static_cast<size_t>(X) * 4;
    uint32_t px;
    if ((reinterpret_cast<uintptr_t>(q) & 3) == 0) px = __ldg(reinterpret_cast<const uint32_t*>(q));
    else px = __ldg(q) | (__ldg(q + 1) << 8) | (__ldg(q + 2) << 16) | (__ldg(q + 3) << 24);
    o[0] = static_cast<float>(px & 0xffu); o[1] = static_cast<float>((px >> 8) & 0xffu);
    o[2] = static_cast<float>((px >> 16) & 0xffu); o[3] = static_cast<float>(px >> 24);
    return false;
}
template <int N>
__device__ __forceinline__ void apply_ops4(float (&v)[N][4], const fkb_chain_desc& ch, const PlaneRec& pl, uint32_t first, uint32_t last) {
    for (uint32_t i = first; i < last; ++i) {
        const int slot = ch.ops[i].plane_slot;
        float p[4];
        if (slot >= 0) { p[0] = pl.params[slot][0]; p[1] = pl.params[slot][1]; p[2] = pl.params[slot][2]; p[3] = pl.params_w[slot]; }
        else { p[0] = ch.ops[i].v[0]; p[1] = ch.ops[i].v[1]; p[2] = ch.ops[i].v[2]; p[3] = ch.op_w[i]; }
        switch (ch.ops[i].code) {
        case FKB_OP_MUL:
#pragma unroll
            for (int n = 0; n < N; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) v[n][c] = __fmul_rn(v[n][c], p[c]);
            break;
        case FKB_OP_ADD:
#pragma unroll
            for (int n = 0; n < N; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) v[n][c] = __fadd_rn(v[n][c], p[c]);
            break;
        case FKB_OP_SUB:
#pragma unroll
            for (int n = 0; n < N; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) v[n][c] = __fsub_rn(v[n][c], p[c]);
            break;
        case FKB_OP_DIV:
#pragma unroll
            for (int n = 0; n < N; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) v[n][c] = __fdiv_rn(v[n][c], p[c]);
            break;
        case FKB_OP_REORDER_ZYX:
#pragma unroll
            for (int n = 0; n < N; ++n) { const float t = v[n][0]; v[n][0] = v[n][2]; v[n][2] = t; }
            break;
        case FKB_OP_SATCAST_U8:
#pragma unroll
            for (int n = 0; n < N; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) v[n][c] = sat_u8_as_float(v[n][c]);
            break;
        case FKB_OP_ADD_ALPHA:
#pragma unroll
            for (int n = 0; n < N; ++n) v[n][3] = ch.ops[i].v[0];
            break;
        default: break;  // FKB_OP_CAST_F32: values are already carried as fp32
        }
    }
}
template <int N>
__device__ __forceinline__ void apply_ops4_bordered(float (&v)[N][4], const fkb_chain_desc& ch, const PlaneRec& pl, uint32_t last, uint32_t outside) {
    if (outside == 0u) { apply_ops4<N>(v, ch, pl, 0, last); return; }
    apply_ops4<N>(v, ch, pl, 0, ch.border_at);
#pragma unroll
    for (int n = 0; n < N; ++n)
        if ((outside >> n) & 1u) { v[n][0] = ch.border_value[0]; v[n][1] = ch.border_value[1]; v[n][2] = ch.border_value[2]; v[n][3] = ch.border_value_w; }
    apply_ops4<N>(v, ch, pl, ch.border_at, last);
}

__global__ void __launch_bounds__(256) gather4_kernel(const __grid_constant__ LaunchParams p) {
    pdl_signal();
    pdl_wait();
    const PlaneRec* table = plane_table(p);
    const uint32_t x = blockIdx.x * 32 + (threadIdx.x & 31), y = blockIdx.y * 8 + (threadIdx.x >> 5);
    for (uint32_t z = p.gather4_z0 + blockIdx.z; z < p.gather4_z1; z += gridDim.z) {
        const PlaneRec& pl = table[z];  // read in place: every thread of the CTA reads the same words (broadcast, cached)
        if (pl.kclass != KCLASS_GATHER4 || x >= pl.dst_w || y >= pl.dst_h) continue;
        const fkb_chain_desc& ch = p.chains[pl.chain];
        float v[1][4];
        if (pl.src == nullptr) {  // a plane whose read yields its default value
            v[0][0] = pl.bg[0]; v[0][1] = pl.bg[1]; v[0][2] = pl.bg[2]; v[0][3] = pl.bg_w;
            apply_ops4<1>(v, ch, pl, ch.geometry == FKB_GEOM_NONE ? 0 : ch.n_pre_ops, ch.n_ops);
        } else if (ch.geometry == FKB_GEOM_NONE) {
            const uint32_t outside = read_tap4(ch, pl, static_cast<int>(x), static_cast<int>(y), v[0]) ? 1u : 0u;
            apply_ops4_bordered<1>(v, ch, pl, ch.n_ops, outside);
        } else {
            const bool par = ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR;
            const int xi = static_cast<int>(x), yi = static_cast<int>(y);
            if (!par || (xi >= pl.x1 && xi <= pl.x2 && yi >= pl.y1 && yi <= pl.y2)) {
                const AxisTap ax = axis_tap(xi - (par ? pl.x1 : 0), pl.fx, pl.crop_w), ay = axis_tap(yi - (par ? pl.y1 : 0), pl.fy, pl.crop_h);
                float t[4][4];
                uint32_t outside = read_tap4(ch, pl, ax.i0, ay.i0, t[0]) ? 1u : 0u;
                outside |= read_tap4(ch, pl, ax.i1, ay.i0, t[1]) ? 2u : 0u;
                outside |= read_tap4(ch, pl, ax.i0, ay.i1, t[2]) ? 4u : 0u;
                outside |= read_tap4(ch, pl, ax.i1, ay.i1, t[3]) ? 8u : 0u;
                apply_ops4_bordered<4>(t, ch, pl, ch.n_pre_ops, outside);
                const float w00 = __fmul_rn(ax.w0, ay.w0), w10 = __fmul_rn(ax.w1, ay.w0);
                const float w01 = __fmul_rn(ax.w0, ay.w1), w11 = __fmul_rn(ax.w1, ay.w1);
#pragma unroll
                for (int c = 0; c < 4; ++c) v[0][c] = bilerp(t[0][c], t[1][c], t[2][c], t[3][c], w00, w10, w01, w11);
            } else {
                v[0][0] = pl.bg[0]; v[0][1] = pl.bg[1]; v[0][2] = pl.bg[2]; v[0][3] = pl.bg_w;
            }
            apply_ops4<1>(v, ch, pl, ch.n_pre_ops, ch.n_ops);
        }
        uint8_t* row = pl.dst + static_cast<size_t>(y) * pl.dst_pitch;
        if (ch.dst_format == FKB_PIX_F32C4) {
            float* f = reinterpret_cast<float*>(row) + static_cast<size_t>(x) * 4;
            if ((reinterpret_cast<uintptr_t>(f) & 15) == 0) *reinterpret_cast<float4*>(f) = make_float4(v[0][0], v[0][1], v[0][2], v[0][3]);
            else { f[0] = v[0][0]; f[1] = v[0][1]; f[2] = v[0][2]; f[3] = v[0][3]; }
        } else {
            uint8_t* q = row + static_cast<size_t>(x) * 4;
            const uint32_t px = static_cast<uint32_t>(v[0][0]) | (static_cast<uint32_t>(v[0][1]) << 8) | (static_cast<uint32_t>(v[0][2]) << 16) |
                                (static_cast<uint32_t>(v[0][3]) << 24);
            if ((reinterpret_cast<uintptr_t>(q) & 3) == 0) *reinterpret_cast<uint32_t*>(q) = px;
            else { q[0] = static_cast<uint8_t>(px); q[1] = static_cast<uint8_t>(px >> 8); q[2] = static_cast<uint8_t>(px >> 16); q[3] = static_cast<uint8_t>(px >> 24); }
        }
    }
}

// rgba_kernel: the same four-channel chains without an interpreter.  Two horizontally adjacent output pixels per thread,
// so that every arithmetic step is one packed f32x2 instruction per channel; the chain's ops after the interpolation
// arrive flattened as at most six steps (FourConsts), N of them, unrolled.  A tap byte becomes a float without a
// conversion: the byte, moved to the low end of a word, is the bit pattern of the subnormal b * 2^-149; the vertical
// weights carry a factor of 2^127, and one exact multiplication by 2^22 puts the scale right (see resize_item).
// Taps are computed for clamped coordinates, so that every address is valid; letterbox pixels are replaced afterwards.
template <int N, bool SRC3>
__global__ void __launch_bounds__(256) rgba_kernel(const __grid_constant__ LaunchParams p) {
    pdl_signal();
    pdl_wait();
    const PlaneRec* table = plane_table(p);
    const FourConsts& k = p.four;
    const float nz = p.neg_zero;
    const uint32_t xa = (blockIdx.x * 32 + (threadIdx.x & 31)) * 2, xb = xa + 1, y = blockIdx.y * 8 + (threadIdx.x >> 5);
    for (uint32_t z = p.gather4_z0 + blockIdx.z; z < p.gather4_z1; z += gridDim.z) {
        const PlaneRec& pl = table[z];
        if (pl.kclass != KCLASS_GATHER4 || xa >= pl.dst_w || y >= pl.dst_h) continue;
        const bool has_b = xb < pl.dst_w;
        f2 v[4];  // channel c of the two pixels
        constexpr uint32_t sp = SRC3 ? 3u : 4u;
        const uint32_t pitch = pl.src_pitch;
        auto tap = [&](const uint8_t* row, uint32_t X) -> uint32_t {  // the pixel's bytes in one word (byte 3 = 0 for a uchar3 source)
            const uint8_t* q = row + static_cast<size_t>(X) * sp;
            if (!SRC3) return __ldg(reinterpret_cast<const uint32_t*>(q));  // (the host checked the alignment)
            return __ldg(q) | (__ldg(q + 1) << 8) | (__ldg(q + 2) << 16);
        };
        if (!k.resize) {
            const uint8_t* row = pl.src + static_cast<size_t>(pl.crop_y + y) * pitch;
            const uint32_t pa = tap(row, pl.crop_x + xa), pb = tap(row, pl.crop_x + (has_b ? xb : xa));
#pragma unroll
            for (int c = 0; c < 4; ++c) v[c] = f2{FKB_BYTE_F32(pa, c), FKB_BYTE_F32(pb, c)};
        } else {
            const bool par = k.preserve_ar != 0;
            const int ox = par ? pl.x1 : 0, oy = par ? pl.y1 : 0;
            const AxisTap ta = axis_tap(max(static_cast<int>(xa) - ox, 0), pl.fx, pl.crop_w);
            const AxisTap tb = axis_tap(max(static_cast<int>(xb) - ox, 0), pl.fx, pl.crop_w);
            const AxisTap ty = axis_tap(max(static_cast<int>(y) - oy, 0), pl.fy, pl.crop_h);
            const uint8_t* r0 = pl.src + static_cast<size_t>(ty.i0 + pl.crop_y) * pitch;
            const uint8_t* r1 = pl.src + static_cast<size_t>(ty.i1 + pl.crop_y) * pitch;
            // tap order: (x0,y0) (x1,y0) (x0,y1) (x1,y1); all eight pixel loads are requested before any is used
            const uint32_t a00 = tap(r0, ta.i0 + pl.crop_x), a10 = tap(r0, ta.i1 + pl.crop_x), a01 = tap(r1, ta.i0 + pl.crop_x), a11 = tap(r1, ta.i1 + pl.crop_x);
            const uint32_t b00 = tap(r0, tb.i0 + pl.crop_x), b10 = tap(r0, tb.i1 + pl.crop_x), b01 = tap(r1, tb.i0 + pl.crop_x), b11 = tap(r1, tb.i1 + pl.crop_x);
            const float wy0s = __fmul_rn(ty.w0, kTapScale), wy1s = __fmul_rn(ty.w1, kTapScale);
            const f2 wy0{wy0s, wy0s}, wy1{wy1s, wy1s}, wx0{ta.w0, tb.w0}, wx1{ta.w1, tb.w1};
            const f2 w00 = mul2(wx0, wy0), w10 = mul2(wx1, wy0), w01 = mul2(wx0, wy1), w11 = mul2(wx1, wy1);
            const f2 unscale{kTapUnscale, kTapUnscale};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t sel = 0x4440u | c;  // byte c to the low end, zeros above it
                const f2 p00{__uint_as_float(__byte_perm(a00, 0u, sel)), __uint_as_float(__byte_perm(b00, 0u, sel))};
                const f2 p10{__uint_as_float(__byte_perm(a10, 0u, sel)), __uint_as_float(__byte_perm(b10, 0u, sel))};
                const f2 p01{__uint_as_float(__byte_perm(a01, 0u, sel)), __uint_as_float(__byte_perm(b01, 0u, sel))};
                const f2 p11{__uint_as_float(__byte_perm(a11, 0u, sel)), __uint_as_float(__byte_perm(b11, 0u, sel))};
                const f2 s = add2(add2(add2(mul2_unfusable(p00, w00, nz), mul2_unfusable(p10, w10, nz)), mul2_unfusable(p01, w01, nz)),
                                  mul2_unfusable(p11, w11, nz));
                v[c] = mul2(s, unscale);  // (exact, and followed by no addition it could fuse with: the steps are FMAs already)
            }
            if (par) {
                const int xi = static_cast<int>(xa), yi = static_cast<int>(y);
                const bool row_in = yi >= pl.y1 && yi <= pl.y2;
                const bool in_a = row_in && xi >= pl.x1 && xi <= pl.x2, in_b = row_in && xi + 1 >= pl.x1 && xi + 1 <= pl.x2;
                const float bg[4] = {pl.bg[0], pl.bg[1], pl.bg[2], pl.bg_w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (!in_a) v[c].x = bg[c];
                    if (!in_b) v[c].y = bg[c];
                }
            }
        }
        // A SaturateCast that ends the chain of a byte destination leaves its results as 2^23 + n, the integer in the low
        // byte, ready to be packed (the same rounding as the step itself: clamp, then one addition that rounds to even).
        bool biased = false;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const uint32_t kind = (k.kinds >> (2 * i)) & 3u;
            if (kind == 0u) {
#pragma unroll
                for (int c = 0; c < 4; ++c) v[c] = fma2(v[c], f2{k.m[i][c], k.m[i][c]}, f2{k.a[i][c], k.a[i][c]});
            } else if (kind == 1u) {
#pragma unroll
                for (int c = 0; c < 4; ++c) v[c] = f2{__fdiv_rn(v[c].x, k.m[i][c]), __fdiv_rn(v[c].y, k.m[i][c])};
            } else if (i == N - 1 && !k.f32) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    v[c] = add2(f2{fminf(fmaxf(v[c].x, 0.f), 255.f), fminf(fmaxf(v[c].y, 0.f), 255.f)}, f2{kMagic, kMagic});
                biased = true;
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) v[c] = f2{sat_u8_as_float(v[c].x), sat_u8_as_float(v[c].y)};
            }
        }
        // the channel order of the destination: as computed, red and blue exchanged, or (never produced by the host's
        // flattening so far) any other permutation
        constexpr uint32_t kAsIs = 0u | (1u << 2) | (2u << 4) | (3u << 6), kSwapped = 2u | (1u << 2) | (0u << 4) | (3u << 6);
        f2 o[4];
        if (k.perm == kAsIs) {
#pragma unroll
            for (int c = 0; c < 4; ++c) o[c] = v[c];
        } else if (k.perm == kSwapped) {
            o[0] = v[2]; o[1] = v[1]; o[2] = v[0]; o[3] = v[3];
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t from = (k.perm >> (2 * c)) & 3u;
                o[c] = from == 0u ? v[0] : from == 1u ? v[1] : from == 2u ? v[2] : v[3];
            }
        }
        uint8_t* row = pl.dst + static_cast<size_t>(y) * pl.dst_pitch;
        if (k.f32) {
            float4* q = reinterpret_cast<float4*>(row + static_cast<size_t>(xa) * 16);
            q[0] = make_float4(o[0].x, o[1].x, o[2].x, o[3].x);
            if (has_b) q[1] = make_float4(o[0].y, o[1].y, o[2].y, o[3].y);
        } else {
            // (the values are integers in [0, 255] held exactly, or already 2^23 + n: the low byte of the sum is the byte)
            uint32_t ba[4], bb[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const f2 t = biased ? o[c] : add2(o[c], f2{kMagic, kMagic});
                ba[c] = __float_as_uint(t.x); bb[c] = __float_as_uint(t.y);
            }
            const uint32_t wa = __byte_perm(__byte_perm(ba[0], ba[1], 0x0040u), __byte_perm(ba[2], ba[3], 0x0040u), 0x5410u);
            const uint32_t wb = __byte_perm(__byte_perm(bb[0], bb[1], 0x0040u), __byte_perm(bb[2], bb[3], 0x0040u), 0x5410u);
            uint32_t* q = reinterpret_cast<uint32_t*>(row + static_cast<size_t>(xa) * 4);
            if (has_b && (reinterpret_cast<uintptr_t>(q) & 7u) == 0) *reinterpret_cast<uint2*>(q) = make_uint2(wa, wb);
            else { q[0] = wa; if (has_b) q[1] = wb; }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// staged_kernel: every warp runs its own load -> compute -> store pipeline; warps never wait for one another
// ---------------------------------------------------------------------------------------------------------
// Shared memory of one warp (kSliceBytes): two mbarriers, the plane record of the item being processed, two
// source stages (two source rows each) and two output rows.
// All shared-memory accesses go through 32-bit offsets into this array, so that the address arithmetic is 32-bit
// integer adds and the accesses are plain LDS/STS with immediate offsets.
extern __shared__ __align__(128) uint8_t smem_raw[];
#ifdef FKB_PHASE_CLOCKS
constexpr uint32_t kPhaseSlots = 8192;  // one per warp of the grid (2 CTAs x 8 warps on each of at most 512 SMs)
__device__ unsigned long long g_phase_clocks[kPhaseSlots][kPhaseCount];
#endif
__device__ __forceinline__ void phase_clock_flush(const PhaseClock& pc, uint32_t lane) {
#ifdef FKB_PHASE_CLOCKS
    const uint32_t slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (lane == 0 && slot < kPhaseSlots) {
#pragma unroll
        for (int i = 0; i < kPhaseCount; ++i) g_phase_clocks[slot][i] += static_cast<unsigned long long>(pc.acc[i]);
    }
#endif
}


struct WarpSlice {
    uint32_t base;  // offset of this warp's slice in smem_raw
    const PlaneRec* pl;
    // mbarriers 0..3: the (up to four) stages of RESIZE items; 4..7: the four stages of POINT items
    __device__ __forceinline__ uint64_t* bar(uint32_t s) const { return reinterpret_cast<uint64_t*>(smem_raw + base) + s; }
    __device__ __forceinline__ uint32_t in0() const { return base + kSliceHeader; }
    __device__ __forceinline__ uint32_t in4(uint32_t s) const { return base + kSliceHeader + s * kInRowBytes; }
    __device__ __forceinline__ uint32_t out(uint32_t s) const { return base + kSliceHeader + kInRegionBytes + s * kOutSlotBytes; }
};
__device__ __forceinline__ WarpSlice warp_slice(uint32_t base) {
    WarpSlice w;
    w.base = base;
    w.pl = reinterpret_cast<const PlaneRec*>(smem_raw + base + 64);
    return w;
}
static_assert(64 + sizeof(PlaneRec) <= kSliceHeader, "slice header");

// Plane of staged tile t (warp-uniform t; called by all lanes of a warp).
__device__ __forceinline__ uint32_t tile_to_plane(const LaunchParams& p, uint32_t t, uint32_t& local) {
    if (p.tiles_per_plane) { const uint32_t z = t / p.tiles_per_plane; local = t - z * p.tiles_per_plane; return z; }
    const PlaneRec* table = plane_table(p);
    if (p.n_planes <= 32) {
        // lane i looks at plane i; first tiles never decrease, so the planes starting at or before t form a prefix
        const uint32_t lane = threadIdx.x & 31;
        const uint32_t base = lane < p.n_planes ? table[lane].tile_base : 0xffffffffu;
        const uint32_t z = __popc(__ballot_sync(0xffffffffu, base <= t)) - 1u;
        local = t - __shfl_sync(0xffffffffu, base, z);
        return z;
    }
    uint32_t lo = 0, hi = p.n_planes;  // the last plane whose first tile is <= t (planes without tiles are skipped over)
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (table[mid].tile_base <= t) lo = mid; else hi = mid;
    }
    local = t - table[lo].tile_base;
    return lo;
}

// The item a warp processes after the current one.  Its number is either known by position or claimed from the launch's
// counter.  The item functions call claim_now() four rows before the end of the current item and fetch() two rows
// before its end: by then the claim has returned, and the plane record requested there (14 lanes x 16 bytes, into
// registers) arrives while the last rows are computed.  Claiming this late matters at the end of a launch: an item
// claimed earlier than necessary waits for its warp while other warps have run out of work.
constexpr uint32_t kRecLanes = sizeof(PlaneRec) / 16;
struct NextItem {
    const PlaneRec* table;
    uint32_t* work;    // the launch's counter, or null: every item is dealt by position
    uint32_t base;     // what is added to a claimed value: the number of items dealt by position
    uint32_t item;     // the next item's number (numbers run to n_tiles + n_split: the last n_split items have two each)
    uint32_t local;    // ... its index among the items of its plane
    uint32_t half;     // ... and which part of it the number stands for: 0 all rows, 1 the first half, 2 the rest
    uint32_t claim;    // (lane 0) what the counter returned
    bool pending;      // `item` is to be replaced by the claim
    uint4 rec;         // the next item's plane record, 16 bytes per lane
    __device__ __forceinline__ void claim_now(uint32_t lane) {
        if (work) {
            if (lane == 0) claim = atomicAdd(work, 1u);
            pending = true;
        }
    }
    __device__ __forceinline__ void fetch(const LaunchParams& p, uint32_t lane) {
        if (pending) item = base + __shfl_sync(0xffffffffu, claim, 0);
        pending = false;
        if (item < p.n_tiles + p.n_split) {
            const uint32_t n_whole = p.n_tiles - p.n_split;
            uint32_t real = item;
            half = 0u;
            if (item >= n_whole) { real = n_whole + ((item - n_whole) >> 1); half = 1u + ((item - n_whole) & 1u); }
            const uint32_t z = tile_to_plane(p, real, local);
            if (lane < kRecLanes) rec = reinterpret_cast<const uint4*>(table + z)[lane];
        }
    }
};
// the rows of an item before which the next item is looked up and, two rows earlier, claimed
__device__ __forceinline__ uint32_t fetch_row(uint32_t nr) { return nr > 2u ? nr - 2u : nr - 1u; }
__device__ __forceinline__ uint32_t claim_row(uint32_t nr) { const uint32_t fr = fetch_row(nr); return fr > 2u ? fr - 2u : 0u; }

// One output row segment leaves through the TMA engine: lane 0 issues a bulk store of the 16-byte multiple,
// the (row_bytes mod 16) tail bytes go out with plain byte stores.
__device__ __forceinline__ void store_row(uint8_t* gdst, uint32_t srow, uint32_t row_bytes, uint32_t lane, const PlaneRec& pl) {
    const uint32_t bulk = row_bytes & ~15u;
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
        bool store = bulk != 0;
        if (kSelfChecking && store)
            store = self_check(&g_status_word, bulk_range_ok(gdst, bulk, pl.dst, static_cast<size_t>(pl.dst_pitch) * pl.dst_h) && (srow & 15u) == 0);
        if (store) bulk_store(gdst, smem_raw + srow, bulk);
        bulk_commit();
    }
    if (row_bytes != bulk) {  // rare: a row whose byte length is not a multiple of 16
        if (lane < row_bytes - bulk) gdst[bulk + lane] = smem_raw[srow + bulk + lane];
    }
}

// --- post-ops ---------------------------------------------------------------------------------------------
// The ops that follow the read (POINT) or the interpolation (RESIZE).  Chains of the shape [Mul] [Add|Sub] [SaturateCast]
// (each part optional, in this order) are specialised at compile time: KIND is a bit mask of the parts present and the
// operands sit in registers for the whole item.  x - s is computed as x + (-s), which is the same IEEE operation.  Every
// other chain runs through the op interpreter (KIND = kPostGeneric).
constexpr int kPostMul = 1, kPostAdd = 2, kPostSat = 4, kPostGeneric = 8, kPostDiv = 16;  // Div: nv12_kernel only

struct PostParams {
    float m[3], a[3], d[3];
};
__device__ __forceinline__ PostParams load_post(const fkb_chain_desc& ch, const PlaneRec& pl, uint32_t first) {
    PostParams q;
#pragma unroll
    for (int c = 0; c < 3; ++c) { q.m[c] = 1.f; q.a[c] = 0.f; q.d[c] = 1.f; }
    for (uint32_t i = first; i < ch.n_ops; ++i) {
        const fkb_op& op = ch.ops[i];
        const float* v = op.plane_slot >= 0 ? pl.params[op.plane_slot] : op.v;
        if (op.code == FKB_OP_MUL) { q.m[0] = v[0]; q.m[1] = v[1]; q.m[2] = v[2]; }
        else if (op.code == FKB_OP_ADD) { q.a[0] = v[0]; q.a[1] = v[1]; q.a[2] = v[2]; }
        else if (op.code == FKB_OP_SUB) { q.a[0] = -v[0]; q.a[1] = -v[1]; q.a[2] = -v[2]; }
        else if (op.code == FKB_OP_DIV) { q.d[0] = v[0]; q.d[1] = v[1]; q.d[2] = v[2]; }
    }
    return q;
}
// Applies the post-ops to one channel of a pixel pair.  With a SaturateCast the result is left as 2^23 + n (the
// integer n sits in the low byte of the bit pattern), ready to be stored as a byte.
template <int KIND>
__device__ __forceinline__ f2 post_channel(f2 r, const PostParams& q, int c, float nz) {
    if (KIND & kPostMul) r = (KIND & kPostAdd) ? mul2_unfusable(r, f2{q.m[c], q.m[c]}, nz) : mul2(r, f2{q.m[c], q.m[c]});
    if (KIND & kPostAdd) r = add2(r, f2{q.a[c], q.a[c]});
    if (KIND & kPostSat) {
        r.x = fminf(fmaxf(r.x, 0.f), 255.f);
        r.y = fminf(fmaxf(r.y, 0.f), 255.f);
        r = add2(r, f2{kMagic, kMagic});
    }
    return r;
}

// --- POINT items ------------------------------------------------------------------------------------------
// uchar3 -> uchar3: each lane owns 16 pixels (48 B): three 128-bit shared loads and stores; lane chunks are 48 B
// apart, which maps the eight lanes of a quarter-warp onto disjoint bank groups.
// uchar3 -> float3: each lane owns 4 pixels per pass: three 32-bit shared loads (12 B apart), three 128-bit stores.
// Their rows are short (at most 1.5 KB in), so three rows are kept in flight ahead of the one being computed.
template <bool F32, int KIND>
__device__ __forceinline__ bool point_item(const LaunchParams& p, const WarpSlice& w, uint32_t ox, uint32_t oy0,
                                           uint32_t ow, uint32_t nr, uint32_t& k, uint32_t lane, NextItem& next) {
    const PlaneRec& pl = *w.pl;
    const fkb_chain_desc& ch = p.chains[pl.chain];
    const float nz = p.neg_zero;
    // Mul / Add operands in the order the channels appear in a run of byte pairs: (c0,c1) (c2,c0) (c1,c2)
    const PostParams post = load_post(ch, pl, 0);
    f2 mp[3], ap[3];
#pragma unroll
    for (int kk = 0; kk < 3; ++kk) {
        mp[kk] = f2{__fmul_rn(post.m[(2 * kk) % 3], kByteScale), __fmul_rn(post.m[(2 * kk + 1) % 3], kByteScale)};
        ap[kk] = f2{post.a[(2 * kk) % 3], post.a[(2 * kk + 1) % 3]};
    }
    const uint32_t in_bytes = (ow * 3u + 15u) & ~15u;
    const uint8_t* gsrc = pl.src + static_cast<size_t>(pl.crop_y + oy0) * pl.src_pitch + static_cast<size_t>(pl.crop_x + ox) * 3u;
    const uint32_t src_pitch = pl.src_pitch;
    uint8_t* gdst = pl.dst + static_cast<size_t>(oy0) * pl.dst_pitch + static_cast<size_t>(ox) * (F32 ? 12u : 3u);
    auto issue = [&](uint32_t r, uint32_t s) {
        if (lane == 0) {
            bool good = true;
            if (kSelfChecking)
                good = self_check(p.status, bulk_range_ok(gsrc + static_cast<size_t>(r) * src_pitch, in_bytes, pl.src, static_cast<size_t>(pl.src_pitch) * pl.src_h) &&
                                                in_bytes <= kInRowBytes);
            mbar_arrive_expect_tx(w.bar(4 + s), good ? in_bytes : 0u);
            if (good) bulk_load(smem_raw + w.in4(s), gsrc + static_cast<size_t>(r) * src_pitch, in_bytes, w.bar(4 + s));
        }
    };
    auto compute = [&](uint32_t in_s, uint32_t out_s) {
        if (F32) {
            // 4 pixels = 12 source bytes = 6 byte pairs per lane step.  A pair (two neighbouring bytes of one word)
            // becomes two half-subnormals with one byte permute, is widened to fp32 (b * 2^-24) and multiplied by the
            // Mul operand pre-scaled by 2^24 (or by 2^24 alone), all exact; pair k holds channels (2k mod 3, 2k+1 mod 3).
            for (uint32_t c = lane; c * 4u < ow; c += 32) {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(smem_raw + in_s + c * 12u);
                const uint32_t q[3] = {src[0], src[1], src[2]};
                f2 v[6];
#pragma unroll
                for (int i = 0; i < 3; ++i) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t two = __byte_perm(q[i], 0u, h ? 0x4342u : 0x4140u);
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&two));
                        const int kk = (2 * i + h) % 3;
                        f2 t = {f.x, f.y};
                        if (KIND == kPostGeneric) t = mul2(t, f2{kByteScale, kByteScale});
                        else t = (KIND & kPostAdd) ? mul2_unfusable(t, mp[kk], nz) : mul2(t, mp[kk]);
                        if (KIND != kPostGeneric && (KIND & kPostAdd)) t = add2(t, ap[kk]);
                        v[2 * i + h] = t;
                    }
                }
                if (KIND == kPostGeneric) {
                    float t[4][3] = {{v[0].x, v[0].y, v[1].x}, {v[1].y, v[2].x, v[2].y}, {v[3].x, v[3].y, v[4].x}, {v[4].y, v[5].x, v[5].y}};
                    apply_ops<4>(t, ch, pl, 0, ch.n_ops);
                    v[0] = f2{t[0][0], t[0][1]}; v[1] = f2{t[0][2], t[1][0]}; v[2] = f2{t[1][1], t[1][2]};
                    v[3] = f2{t[2][0], t[2][1]}; v[4] = f2{t[2][2], t[3][0]}; v[5] = f2{t[3][1], t[3][2]};
                }
                float4* dst = reinterpret_cast<float4*>(smem_raw + out_s + c * 48u);
                dst[0] = make_float4(v[0].x, v[0].y, v[1].x, v[1].y);
                dst[1] = make_float4(v[2].x, v[2].y, v[3].x, v[3].y);
                dst[2] = make_float4(v[4].x, v[4].y, v[5].x, v[5].y);
            }
        } else {
            for (uint32_t c = lane; c * 16u < ow; c += 32) {
                const uint4* src = reinterpret_cast<const uint4*>(smem_raw + in_s + c * 48u);
                uint32_t q[12];
#pragma unroll
                for (int i = 0; i < 3; ++i) { const uint4 t = src[i]; q[4 * i] = t.x; q[4 * i + 1] = t.y; q[4 * i + 2] = t.z; q[4 * i + 3] = t.w; }
                float v[16][3];
#pragma unroll
                for (int b = 0; b < 48; ++b) v[b / 3][b % 3] = FKB_BYTE_F32(q[b >> 2], b & 3);
                apply_ops<16>(v, ch, pl, 0, ch.n_ops);
#pragma unroll
                for (int i = 0; i < 12; ++i) q[i] = 0;
#pragma unroll
                for (int b = 0; b < 48; ++b) q[b >> 2] |= u8_of_exact(v[b / 3][b % 3]) << (8 * (b & 3));
                uint4* dst = reinterpret_cast<uint4*>(smem_raw + out_s + c * 48u);
#pragma unroll
                for (int i = 0; i < 3; ++i) dst[i] = make_uint4(q[4 * i], q[4 * i + 1], q[4 * i + 2], q[4 * i + 3]);
            }
        }
    };
    constexpr uint32_t AHEAD = 3;
    const uint32_t dst_pitch = pl.dst_pitch, row_bytes = ow * (F32 ? 12u : 3u);
    // the previous item may have ended on either output buffer: start from a state where no store reads them
    if (lane == 0) bulk_wait_read_all();
    __syncwarp();
    for (uint32_t i = 0; i < AHEAD && i < nr; ++i) issue(i, (k + i) & 3u);
    const uint32_t fr = fetch_row(nr), cr = claim_row(nr);
    for (uint32_t r = 0; r < nr; ++r, ++k) {
        if (r == cr) next.claim_now(lane);
        if (r == fr) next.fetch(p, lane);
        const uint32_t s = k & 3u, o = k & 1u;
        if (lane == 0) bulk_wait_read_1();  // the store that read w.out(o) two rows ago is done with it
        if (r + AHEAD < nr) issue(r + AHEAD, (k + AHEAD) & 3u);  // into the stage of the row computed just before
        const bool landed = mbar_wait_bounded(w.bar(4 + s), (k >> 2) & 1u, p.wait_limit_ns);
        if (__any_sync(0xffffffffu, !landed)) return false;
        compute(w.in4(s), w.out(o));
        store_row(gdst + static_cast<size_t>(r) * dst_pitch, w.out(o), row_bytes, lane, pl);
    }
    return true;
}

// --- RESIZE items -----------------------------------------------------------------------------------------
// The columns of the item that lie inside the resized image (PRESERVE_AR leaves bars of background left and right)
// are dealt to the lanes in groups of 32: lane l owns columns xa+l, xa+32+l, ...; the last group is shifted left so
// that it is full too (a few columns are then computed twice, with identical results).  Everything that depends only
// on the column — the byte offset of its tap pair in a staged row and the two horizontal weights — is computed once
// per item and kept in registers for all rows; what depends only on the row — the two source rows and the vertical
// weights — is computed once per item too, row r by lane r, and handed round with shuffles.  A tap pair (x1, x1+1) is
// six consecutive bytes; the column one past the crop is made a copy of the last column after the row lands, which is
// exactly the reference's clamp of x2.
//
// A tap byte needs no conversion instruction at all: the zero-extended byte b, read as an fp32 bit pattern, is the
// subnormal number b * 2^-149, and the FMA pipe takes subnormal operands at full rate.  The vertical weights are
// pre-multiplied by 2^127 (exact), so every product is fl(b * w) * 2^-22 — the correctly rounded product, scaled by a
// power of two — and so is every partial sum (all terms are non-negative, nothing cancels, nothing underflows: the
// host sends planes whose scale factors are below 2^-24 elsewhere).  The 2^22 that is still missing is folded into the
// Mul operand when the chain has one (fl((v * 2^-22) * (m * 2^22)) = fl(v * m)), else it is one exact multiplication.
// Groups are computed two at a time with packed f32x2 instructions; an odd last group runs as scalars.
// The background bars are written into the two output-row buffers once per item.
static_assert(kMaxRowsPerItem <= 32, "one lane per row of an item");

__device__ __forceinline__ float tap_subnormal(uint32_t smem_off) {
    return __uint_as_float(static_cast<uint32_t>(smem_raw[smem_off]));
}
// [Mul][Add][Sat] on one scalar; with a SaturateCast the result is 2^23 + n (the integer in the low byte)
template <int KIND>
__device__ __forceinline__ float post_scalar(float r, float m, float a) {
    if (KIND & kPostMul) r = __fmul_rn(r, m);
    if (KIND & kPostAdd) r = __fadd_rn(r, a);
    if (KIND & kPostSat) r = __fadd_rn(fminf(fmaxf(r, 0.f), 255.f), kMagic);
    return r;
}

template <bool F32, int KIND, bool PLANAR = false, bool SRC4 = false>
__device__ __forceinline__ bool resize_item(const LaunchParams& p, const WarpSlice& w, uint32_t ox, uint32_t oy0,
                                            uint32_t ow, uint32_t nr, uint32_t& ph, uint32_t lane, NextItem& next) {
    static_assert(F32 || !PLANAR, "planar rows are float rows");
    PhaseClock pc;
    constexpr uint32_t FULL = 0xffffffffu;
    constexpr uint32_t SP = SRC4 ? 4u : 3u;                           // bytes per source pixel (uchar4: the alpha byte is skipped)
    constexpr uint32_t ELT = PLANAR ? 4u : F32 ? 12u : 3u;            // bytes between columns of a staged output row
    constexpr uint32_t DEAD = PLANAR ? kMaxTileW * 4u : kOutRowBytes;          // where columns that do not exist are stored
    const PlaneRec& pl = *w.pl;
    const fkb_chain_desc& ch = p.chains[pl.chain];
    // (an all-background plane carries an empty rectangle x1..x2, whatever the chain's geometry)
    const bool par = ch.geometry >= FKB_GEOM_RESIZE_PRESERVE_AR || pl.all_background != 0u;
    const int X1 = par ? pl.x1 : 0, Y1 = par ? pl.y1 : 0;
    const int X2 = par ? pl.x2 : static_cast<int>(pl.dst_w) - 1, Y2 = par ? pl.y2 : static_cast<int>(pl.dst_h) - 1;
    const int crop_w = pl.crop_w, crop_h = pl.crop_h;
    const float fx = pl.fx, fy = pl.fy, nz = p.neg_zero;
    const int xa = max(static_cast<int>(ox), X1), xb = min(static_cast<int>(ox + ow) - 1, X2);
    const int n_in = xb >= xa ? xb - xa + 1 : 0;     // columns of this item inside the resized image
    const int nj = (n_in + 31) >> 5;                 // groups of 32 columns
    const int c_lo = n_in ? axis_tap(xa - X1, fx, crop_w).i0 : 0;
    const int c_hi = n_in ? axis_tap(xb - X1, fx, crop_w).i0 + 1 : 0;  // highest column a tap pair touches
    const bool replicate = c_hi >= crop_w;
    const uint32_t g0 = (pl.crop_x + static_cast<uint32_t>(c_lo)) * SP;
    const uint32_t g1 = (pl.crop_x + static_cast<uint32_t>(min(c_hi, crop_w - 1)) + 1u) * SP;
    const uint32_t a0 = g0 & ~15u, shift = g0 - a0;
    const uint32_t row_bytes = ((g1 + 15u) & ~15u) - a0;
    if (row_bytes + 32u > kInRowBytes) return false;  // the host lowering guarantees the footprint fits
    // The staged-row region is cut into as many stages as this item's footprint lets fit, two to four, each of two rows
    // `rs` bytes apart: row r lands in stage r mod ns, and the source rows of row r + ns are requested as soon as row r
    // has been computed, so a load is in flight for ns - 1 row times before it is waited for.
    const uint32_t rs = row_bytes + 16u;
    const uint32_t ns = min(4u, kInRegionBytes / (2u * rs));
    const uint32_t in0 = w.in0();

    // per-row state, row r of the item in lane r: the two source rows (as an offset from the crop's first row, in
    // units of 16 bytes: staged sources have pitches that are multiples of 16) and the vertical weights times 2^127
    const uint32_t pitch16 = pl.src_pitch >> 4;
    const int y_l = static_cast<int>(oy0 + min(lane, nr - 1u));
    const bool in_l = n_in > 0 && y_l >= Y1 && y_l <= Y2;
    const AxisTap ay_l = axis_tap(in_l ? y_l - Y1 : 0, fy, crop_h);
    const uint32_t in_mask = __ballot_sync(FULL, in_l);
    const uint32_t row0_l = static_cast<uint32_t>(ay_l.i0) * pitch16;
    const uint32_t row1_l = static_cast<uint32_t>(ay_l.i1) * pitch16;
    const float wy0_l = __fmul_rn(ay_l.w0, kTapScale), wy1_l = __fmul_rn(ay_l.w1, kTapScale);

    const uint8_t* gsrc = pl.src + static_cast<size_t>(pl.crop_y) * pl.src_pitch + a0;
    // One lane requests row r's two source rows (r0, r1: offsets in units of 16 bytes) into stage s.  Always two staged
    // rows (the second repeats the first where the reference clamps y2), so that the second row sits at a fixed
    // distance from the first.
    auto load_rows = [&](uint32_t r, uint32_t s, uint32_t r0, uint32_t r1) {
        if (!((in_mask >> r) & 1u)) return;  // a row above or below the image reads nothing and waits for nothing
        bool in = true;
        const uint32_t at = in0 + s * (2u * rs);
        if (kSelfChecking) {
            const size_t frame = static_cast<size_t>(pl.src_pitch) * pl.src_h;
            in = self_check(p.status, bulk_range_ok(gsrc + static_cast<size_t>(r0) * 16u, row_bytes, pl.src, frame) &&
                                          bulk_range_ok(gsrc + static_cast<size_t>(r1) * 16u, row_bytes, pl.src, frame) &&
                                          at + 2u * rs <= in0 + kInRegionBytes && (at & 15u) == 0 && (rs & 15u) == 0);
        }
        mbar_arrive_expect_tx(w.bar(s), (in ? 2u * row_bytes : 0u) + p.test_extra_tx);
        if (in) {
            bulk_load(smem_raw + at, gsrc + static_cast<size_t>(r0) * 16u, row_bytes, w.bar(s));
            bulk_load(smem_raw + at + rs, gsrc + static_cast<size_t>(r1) * 16u, row_bytes, w.bar(s));
        }
    };
    // The source rows of the first ns output rows are requested before the rest of the set-up, which then overlaps their
    // latency (every stage was last read by a row this warp has finished): lane i requests row i, whose state it holds.
    if (lane < ns && lane < nr) load_rows(lane, lane, row0_l, row1_l);

    // per-column state of this lane: staged-row byte offset of the tap pair and the horizontal weights.  Where a column
    // goes in the output row follows from its group: group j starts 32 j columns after the lane's first column, except
    // the last group, which is shifted (or, when the item has fewer than 32 columns, partly missing: those lanes write
    // to the spare bytes behind the output row).
    uint32_t boff[8];
    float wx0[8], wx1[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // (all eight without a branch, so that their chains overlap; groups past nj are never used)
        int col = 32 * j + static_cast<int>(lane);                 // index among the inside columns
        if (j == nj - 1 && n_in >= 32) col = n_in - 32 + static_cast<int>(lane);  // last group, shifted to be full
        col = max(min(col, n_in - 1), 0);
        const AxisTap t = axis_tap(xa + col - X1, fx, crop_w);
        boff[j] = static_cast<uint32_t>(t.i0 - c_lo) * SP + shift;
        wx0[j] = t.w0; wx1[j] = t.w1;
    }
    const uint32_t obase = static_cast<uint32_t>(xa - static_cast<int>(ox) + static_cast<int>(lane)) * ELT;
    const uint32_t olast = n_in >= 32 ? static_cast<uint32_t>(xa - static_cast<int>(ox) + n_in - 32 + static_cast<int>(lane)) * ELT
                                      : (static_cast<int>(lane) < n_in ? obase : DEAD);
    // output-row offset of this lane's column of group j
    auto ocol = [&](int j) { return j + 1 == nj ? olast : obase + static_cast<uint32_t>(j) * (32u * ELT); };
    // Offset (in a staged row) of the crop's last column when a tap pair reaches one past it; that column is then
    // duplicated into the next three bytes (inside the 16 spare bytes every staged row has).
    const uint32_t rep_off = replicate ? static_cast<uint32_t>(crop_w - 1 - c_lo) * SP + shift : 0u;
    const uint32_t dst_pitch = pl.dst_pitch;
    uint8_t* gdst = pl.dst + static_cast<size_t>(oy0) * dst_pitch + static_cast<size_t>(ox) * ELT;

    // operands of the specialised post-ops; the Mul operand also takes the 2^22 the taps' scale leaves behind
    PostParams post;
    if (KIND != kPostGeneric) {
        const PostImm& imm = p.post_imm[pl.chain];
        if (imm.slots) post = load_post(ch, pl, ch.n_pre_ops);
        else {
#pragma unroll
            for (int c = 0; c < 3; ++c) { post.m[c] = imm.m[c]; post.a[c] = imm.a[c]; post.d[c] = 1.f; }
        }
    }
    // what a background pixel becomes, as the bit patterns that are stored
    uint32_t bgbits[3];
    if (KIND != kPostGeneric) {
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            const float b = post_scalar<KIND>(pl.bg[c], post.m[c], post.a[c]);
            bgbits[c] = (KIND & kPostSat) ? (__float_as_uint(b) & 0xffu) : __float_as_uint(b);
        }
    } else {
        float b[1][3] = {{pl.bg[0], pl.bg[1], pl.bg[2]}};
        apply_ops<1>(b, ch, pl, ch.n_pre_ops, ch.n_ops);
#pragma unroll
        for (int c = 0; c < 3; ++c) bgbits[c] = F32 ? __float_as_uint(b[0][c]) : u8_of_exact(b[0][c]);
    }
    float mq[3];  // Mul operand times 2^22 (or 2^22 alone)
#pragma unroll
    for (int c = 0; c < 3; ++c) mq[c] = (KIND != kPostGeneric && (KIND & kPostMul)) ? __fmul_rn(post.m[c], kTapUnscale) : kTapUnscale;

    auto put = [&](uint32_t q, uint32_t b0, uint32_t b1, uint32_t b2) {
        if (PLANAR) {
            *reinterpret_cast<uint32_t*>(smem_raw + q) = b0;
            *reinterpret_cast<uint32_t*>(smem_raw + q + kPlanarSegBytes) = b1;
            *reinterpret_cast<uint32_t*>(smem_raw + q + 2 * kPlanarSegBytes) = b2;
        }
        else if (F32) { uint32_t* f = reinterpret_cast<uint32_t*>(smem_raw + q); f[0] = b0; f[1] = b1; f[2] = b2; }
        else { smem_raw[q] = static_cast<uint8_t>(b0); smem_raw[q + 1] = static_cast<uint8_t>(b1); smem_raw[q + 2] = static_cast<uint8_t>(b2); }
    };
    // the bars left and right of the image are the same for every row of the item: fill them in both row buffers once
    // (after the bulk stores that still read those buffers have finished reading)
    if (lane == 0) bulk_wait_read_all();
    __syncwarp();
    if (static_cast<uint32_t>(n_in) < ow) {
        const int left = n_in ? xa - static_cast<int>(ox) : static_cast<int>(ow);  // columns of the left bar (all of them when nothing is inside)
        const int n_bar = static_cast<int>(ow) - n_in;
        for (int c = static_cast<int>(lane); c < n_bar; c += 32) {
            const uint32_t q = static_cast<uint32_t>(c < left ? c : c + n_in) * ELT;
            put(w.out(0) + q, bgbits[0], bgbits[1], bgbits[2]);
            put(w.out(1) + q, bgbits[0], bgbits[1], bgbits[2]);
        }
    }

    // the post-ops of one channel of a pixel pair and the bits to store
    auto finish = [&](const f2 (&v)[3], uint32_t (&bx)[3], uint32_t (&by)[3]) {
        if (KIND == kPostGeneric) {
            float t[2][3];
#pragma unroll
            for (int c = 0; c < 3; ++c) { const f2 u = mul2(v[c], f2{kTapUnscale, kTapUnscale}); t[0][c] = u.x; t[1][c] = u.y; }
            apply_ops<2>(t, ch, pl, ch.n_pre_ops, ch.n_ops);
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                bx[c] = F32 ? __float_as_uint(t[0][c]) : u8_of_exact(t[0][c]);
                by[c] = F32 ? __float_as_uint(t[1][c]) : u8_of_exact(t[1][c]);
            }
        } else {
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                // (a product by 2^22 alone is exact, so it may fuse with the addition that follows; a Mul operand's may not)
                f2 t = ((KIND & kPostMul) && (KIND & kPostAdd)) ? mul2_unfusable(v[c], f2{mq[c], mq[c]}, nz) : mul2(v[c], f2{mq[c], mq[c]});
                if (KIND & kPostAdd) t = add2(t, f2{post.a[c], post.a[c]});
                if (KIND & kPostSat) {
                    t.x = fminf(fmaxf(t.x, 0.f), 255.f);
                    t.y = fminf(fmaxf(t.y, 0.f), 255.f);
                    t = add2(t, f2{kMagic, kMagic});
                }
                bx[c] = __float_as_uint(t.x); by[c] = __float_as_uint(t.y);  // with SaturateCast: low byte = value
            }
        }
    };

    // two groups of columns (j, j+1) of the current row
    auto pair = [&](int j, uint32_t in_s, uint32_t out_s, f2 wy0, f2 wy1) {
        const uint32_t a0p = in_s + boff[j], a1p = in_s + boff[j + 1];
        const uint32_t a0q = a0p + rs, a1q = a1p + rs;  // the same columns in the second staged row
        const f2 wx0p = {wx0[j], wx0[j + 1]}, wx1p = {wx1[j], wx1[j + 1]};
        const f2 w00 = mul2(wx0p, wy0), w10 = mul2(wx1p, wy0), w01 = mul2(wx0p, wy1), w11 = mul2(wx1p, wy1);
        f2 v[3];
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            // taps of the two columns: (x1,y1) (x1+1,y1) (x1,y2) (x1+1,y2), each b * 2^-149
            const f2 p00 = {tap_subnormal(a0p + c), tap_subnormal(a1p + c)};
            const f2 p10 = {tap_subnormal(a0p + SP + c), tap_subnormal(a1p + SP + c)};
            const f2 p01 = {tap_subnormal(a0q + c), tap_subnormal(a1q + c)};
            const f2 p11 = {tap_subnormal(a0q + SP + c), tap_subnormal(a1q + SP + c)};
            v[c] = add2(add2(add2(mul2_unfusable(p00, w00, nz), mul2_unfusable(p10, w10, nz)), mul2_unfusable(p01, w01, nz)),
                        mul2_unfusable(p11, w11, nz));
        }
        uint32_t bx[3], by[3];
        finish(v, bx, by);
        put(out_s + obase + static_cast<uint32_t>(j) * (32u * ELT), bx[0], bx[1], bx[2]);  // (the first group of a pair is never the last)
        put(out_s + ocol(j + 1), by[0], by[1], by[2]);
    };
    // one group of columns: channels 0 and 1 as a packed pair, channel 2 with itself
    auto single = [&](int j, uint32_t in_s, uint32_t out_s, f2 wy0, f2 wy1) {
        const uint32_t ap = in_s + boff[j], aq = ap + rs;
        const f2 wx0p = {wx0[j], wx0[j]}, wx1p = {wx1[j], wx1[j]};
        const f2 w00 = mul2(wx0p, wy0), w10 = mul2(wx1p, wy0), w01 = mul2(wx0p, wy1), w11 = mul2(wx1p, wy1);
        const f2 p00 = {tap_subnormal(ap), tap_subnormal(ap + 1)}, p10 = {tap_subnormal(ap + SP), tap_subnormal(ap + SP + 1)};
        const f2 p01 = {tap_subnormal(aq), tap_subnormal(aq + 1)};
        const f2 p11 = {tap_subnormal(aq + SP), tap_subnormal(aq + SP + 1)};
        const f2 q00 = {tap_subnormal(ap + 2), 0.f}, q10 = {tap_subnormal(ap + SP + 2), 0.f};
        const f2 q01 = {tap_subnormal(aq + 2), 0.f}, q11 = {tap_subnormal(aq + SP + 2), 0.f};
        const f2 v01 = add2(add2(add2(mul2_unfusable(p00, w00, nz), mul2_unfusable(p10, w10, nz)), mul2_unfusable(p01, w01, nz)),
                            mul2_unfusable(p11, w11, nz));
        const f2 v2 = add2(add2(add2(mul2_unfusable(q00, w00, nz), mul2_unfusable(q10, w10, nz)), mul2_unfusable(q01, w01, nz)),
                           mul2_unfusable(q11, w11, nz));
        const f2 v[3] = {f2{v01.x, v2.y}, f2{v01.y, v2.y}, f2{v2.x, v2.y}};
        uint32_t bx[3], by[3];
        finish(v, bx, by);
        put(out_s + olast, bx[0], bx[1], bx[2]);  // (an odd group is the last one)
    };

    // Row loop.  Per row: wait for its source rows, compute it into an output-row buffer, and then — in lane 0's one
    // divergent stretch per row — send the row off with a bulk store, request the source rows of row r + ns into the
    // stage just read, and wait until the store of the previous row has finished reading the other buffer.
    // A row above or below the image is background from end to end: the first of a run of them is written into a buffer,
    // the others are stored from that same buffer again with nothing written and nothing waited for.  The two buffers
    // alternate by rows written, so a buffer is written only after wait_group.read has covered every store that read it.
    const uint32_t out_bytes = ow * ELT, out_bulk = out_bytes & ~15u;
    uint8_t* gout = gdst;
    uint32_t s = 0;         // stage of the row being computed: r mod ns
    uint32_t o = 0;         // the output-row buffer the next written row goes to
    bool bg_ready = false;  // the other buffer holds a background row (the previous row was one)
    pc.lap(kPhaseSetup);
    pc.count(kPhaseItems);
    bool first_wait = true;
    const uint32_t fr = fetch_row(nr), cr = claim_row(nr);
    for (uint32_t r = 0; r < nr; ++r, gout += dst_pitch) {
        if (r == cr) next.claim_now(lane);
        if (r == fr) next.fetch(p, lane);
        const uint32_t r0n = __shfl_sync(FULL, row0_l, (r + ns) & 31u), r1n = __shfl_sync(FULL, row1_l, (r + ns) & 31u);
        const bool row_in = (in_mask >> r) & 1u;
        const uint32_t in_s = in0 + s * (2u * rs);
        uint32_t out_s;
        if (!row_in) {
            if (bg_ready) out_s = w.out(o ^ 1u);
            else {
                out_s = w.out(o);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j < nj) put(out_s + ocol(j), bgbits[0], bgbits[1], bgbits[2]);
                o ^= 1u;
                bg_ready = true;
                fence_async_smem();
                __syncwarp();
            }
        } else {
            const float wy0s = __shfl_sync(FULL, wy0_l, r), wy1s = __shfl_sync(FULL, wy1_l, r);
            const bool ok = mbar_wait_bounded(w.bar(s), (ph >> s) & 1u, p.wait_limit_ns);
            if (__any_sync(FULL, !ok)) return false;  // (a convergence point for the whole warp, too)
            pc.lap(first_wait ? kPhaseFirstWait : kPhaseWait);
            first_wait = false;
            ph ^= 1u << s;
            out_s = w.out(o);
            o ^= 1u;
            bg_ready = false;
            if (replicate)
            {  // every lane writes the same three bytes (even lanes the first staged row, odd lanes the second)
                const uint32_t q = in_s + (lane & 1u) * rs + rep_off;
                const uint8_t c0 = smem_raw[q], c1 = smem_raw[q + 1], c2 = smem_raw[q + 2];
                smem_raw[q + SP] = c0; smem_raw[q + SP + 1] = c1; smem_raw[q + SP + 2] = c2;
                __syncwarp();
            }
            const f2 wy0 = {wy0s, wy0s}, wy1 = {wy1s, wy1s};
            switch (nj) {  // the odd group, if there is one ...
            case 7: single(6, in_s, out_s, wy0, wy1); break;
            case 5: single(4, in_s, out_s, wy0, wy1); break;
            case 3: single(2, in_s, out_s, wy0, wy1); break;
            case 1: single(0, in_s, out_s, wy0, wy1); break;
            default: break;
            }
            switch (nj >> 1) {  // ... and the pairs: one uniform jump instead of a test per pair
            case 4: pair(6, in_s, out_s, wy0, wy1);
            case 3: pair(4, in_s, out_s, wy0, wy1);
            case 2: pair(2, in_s, out_s, wy0, wy1);
            case 1: pair(0, in_s, out_s, wy0, wy1);
            default: break;
            }
            fence_async_smem();
            __syncwarp();
        }
        pc.lap(kPhaseCompute);
        pc.count(kPhaseRows);
        if (lane == 0) {
            bool store = out_bulk != 0;
            if (kSelfChecking && store)  // (a planar destination: the first channel's plane is the one the record describes)
                store = self_check(p.status, bulk_range_ok(gout, out_bulk, pl.dst, static_cast<size_t>(pl.dst_pitch) * pl.dst_h) && (out_s & 15u) == 0);
            if (store) {
                bulk_store(gout, smem_raw + out_s, out_bulk);
                if (PLANAR) {
                    bulk_store(gout + pl.dst_cstride, smem_raw + out_s + kPlanarSegBytes, out_bulk);
                    bulk_store(gout + pl.dst_cstride2, smem_raw + out_s + 2 * kPlanarSegBytes, out_bulk);
                }
            }
            pc.lap(kPhaseStore);
            bulk_commit();
            pc.lap(kPhaseCommit);
            if (r + ns < nr) load_rows(r + ns, s, r0n, r1n);
            pc.lap(kPhaseLoads);
            bulk_wait_read_1();  // the store of the row before has read its buffer: the next row may be written there
            pc.lap(kPhaseWaitRead);
        }
        s = s + 1u == ns ? 0u : s + 1u;
        if (out_bytes != out_bulk && lane < out_bytes - out_bulk) {  // rare: a row whose byte length is not a multiple of 16
            gout[out_bulk + lane] = smem_raw[out_s + out_bulk + lane];
            if (PLANAR) {
                gout[pl.dst_cstride + out_bulk + lane] = smem_raw[out_s + kPlanarSegBytes + out_bulk + lane];
                gout[pl.dst_cstride2 + out_bulk + lane] = smem_raw[out_s + 2 * kPlanarSegBytes + out_bulk + lane];
            }
        }
    }
    phase_clock_flush(pc, lane);
    return true;
}

template <bool F32, bool PLANAR = false, bool SRC4 = false>
__device__ __forceinline__ bool resize_dispatch(const LaunchParams& p, const WarpSlice& w, uint32_t kind, uint32_t ox,
                                                uint32_t oy0, uint32_t ow, uint32_t nr, uint32_t& ph, uint32_t lane, NextItem& next) {
    constexpr int S = F32 ? 0 : kPostSat;  // a uchar3 destination ends in a SaturateCast, a float3 one cannot
    switch (kind) {
    case S: return resize_item<F32, S, PLANAR, SRC4>(p, w, ox, oy0, ow, nr, ph, lane, next);
    case S | kPostMul: return resize_item<F32, S | kPostMul, PLANAR, SRC4>(p, w, ox, oy0, ow, nr, ph, lane, next);
    case S | kPostAdd: return resize_item<F32, S | kPostAdd, PLANAR, SRC4>(p, w, ox, oy0, ow, nr, ph, lane, next);
    case S | kPostMul | kPostAdd: return resize_item<F32, S | kPostMul | kPostAdd, PLANAR, SRC4>(p, w, ox, oy0, ow, nr, ph, lane, next);
    default: return resize_item<F32, kPostGeneric, PLANAR, SRC4>(p, w, ox, oy0, ow, nr, ph, lane, next);
    }
}

__global__ void __launch_bounds__(kStagedThreads, kStagedCtasPerSm) staged_kernel(const __grid_constant__ LaunchParams p) {
    pdl_signal();
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const WarpSlice w = warp_slice(warp * kSliceBytes);
    if (lane == 0) {
        for (uint32_t i = 0; i < 8; ++i) mbar_init(w.bar(i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const uint32_t warps_per_cta = blockDim.x >> 5;
    // Items are dealt in two ways.  By position, item i runs on warp (i / gridDim.x) % warps_per_cta of CTA i % gridDim.x
    // (a small launch spreads over all SMs).  With a work counter (launches of more than two items per warp), a warp takes
    // only its first item that way and claims every further one from the counter, so that warps whose items were cheap
    // (small crops, letterbox rows) take more of them.  The claim for the next item is issued four rows before the
    // current item ends and looked at two rows later (NextItem), so its latency is on nobody's critical path and no item
    // is held back by more than half an item's time.
    const uint32_t first = warp * gridDim.x + blockIdx.x, stride = gridDim.x * warps_per_cta;
    const bool dynamic = p.work != nullptr;
    uint32_t ph = 0, k4 = 0;  // phase bits of the RESIZE items' barriers; steps done so far by POINT items (four stages)
    bool ok = true;
    NextItem next;
    next.table = plane_table(p);
    next.work = p.work;
    next.base = stride;
    next.item = first; next.local = 0; next.half = 0; next.claim = 0; next.pending = false;
    next.rec = make_uint4(0, 0, 0, 0);
    // The first item's record is requested before the wait for the kernel before this one: the plane table is written by
    // the host (kernel parameters, a plan's table, or an upload that this launch follows in stream order), never by a
    // kernel, so reading it needs no ordering against one; everything else this kernel reads or writes comes after the wait.
    next.fetch(p, lane);
    pdl_wait();
    const uint32_t n_items = p.n_tiles + p.n_split;
    for (uint32_t item = first; item < n_items && ok;) {
        __syncwarp();
        if (lane < kRecLanes) reinterpret_cast<uint4*>(smem_raw + w.base + 64)[lane] = next.rec;
        __syncwarp();
        const uint32_t cur_local = next.local, cur_half = next.half;
        next.item = item + stride;  // by position, unless the launch has a counter
        const PlaneRec& pl = *w.pl;
        uint32_t tyi = cur_local, txi = 0;  // (most planes are one segment wide: no division then)
        if (pl.tiles_x != 1u) { tyi = cur_local / pl.tiles_x; txi = cur_local - tyi * pl.tiles_x; }
        const uint32_t ox = txi * pl.tile_w, ow = min(pl.tile_w, pl.dst_w - ox);
        uint32_t oy0 = tyi * pl.tile_h, nr = min(pl.tile_h, pl.dst_h - oy0);
        if (cur_half) {
            const uint32_t head = (nr + 1u) >> 1;  // rows of the first half
            if (cur_half == 1u) nr = head;
            else { oy0 += head; nr -= head; }
            if (nr == 0u) {  // (an item of one row has no second half; the next item is still to be found)
                next.claim_now(lane);
                next.fetch(p, lane);
                item = next.item;
                continue;
            }
        }
        const bool f32 = p.chains[pl.chain].dst_format == FKB_PIX_F32C3;
        if (pl.kclass == KCLASS_POINT) {
            if (!f32) ok = point_item<false, kPostGeneric>(p, w, ox, oy0, ow, nr, k4, lane, next);
            else switch (p.post_kind[pl.chain]) {
                case 0: ok = point_item<true, 0>(p, w, ox, oy0, ow, nr, k4, lane, next); break;
                case kPostMul: ok = point_item<true, kPostMul>(p, w, ox, oy0, ow, nr, k4, lane, next); break;
                case kPostAdd: ok = point_item<true, kPostAdd>(p, w, ox, oy0, ow, nr, k4, lane, next); break;
                case kPostMul | kPostAdd: ok = point_item<true, kPostMul | kPostAdd>(p, w, ox, oy0, ow, nr, k4, lane, next); break;
                default: ok = point_item<true, kPostGeneric>(p, w, ox, oy0, ow, nr, k4, lane, next); break;
            }
        }
        else if (p.chains[pl.chain].src_format == FKB_PIX_U8C4) {  // (float destinations only: the host lowering sees to it)
            ok = p.chains[pl.chain].write_kind != FKB_WRITE_PACKED ? resize_dispatch<true, true, true>(p, w, p.post_kind[pl.chain], ox, oy0, ow, nr, ph, lane, next)
                                                                   : resize_dispatch<true, false, true>(p, w, p.post_kind[pl.chain], ox, oy0, ow, nr, ph, lane, next);
        }
        else if (p.chains[pl.chain].write_kind != FKB_WRITE_PACKED) ok = resize_dispatch<true, true>(p, w, p.post_kind[pl.chain], ox, oy0, ow, nr, ph, lane, next);
        else ok = f32 ? resize_dispatch<true>(p, w, p.post_kind[pl.chain], ox, oy0, ow, nr, ph, lane, next)
                      : resize_dispatch<false>(p, w, p.post_kind[pl.chain], ox, oy0, ow, nr, ph, lane, next);
        item = next.item;
    }
    if (lane == 0) bulk_wait_all();  // shared memory must stay valid until the last bulk store has read it
    if (dynamic && lane == 0) {
        // the last warp to finish puts the counters back to zero for the next launch (every claim of this launch,
        // used or not, was issued before its warp's increment of the second counter)
        __threadfence();
        if (atomicAdd(p.work + 1, 1u) == stride - 1u) { p.work[0] = 0u; p.work[1] = 0u; __threadfence(); }
    }
    if (!ok) {
        // copies announced on the other stages may still be in flight: give them a bounded chance to land
        // (stages without a copy in flight never complete: the limit, shortened, ends those waits)
        const uint32_t grace = min(p.wait_limit_ns, 1000000u);
        for (uint32_t i = 0; i < 4; ++i) mbar_wait_bounded(w.bar(i), (ph >> i) & 1u, grace);
        for (uint32_t i = 1; i <= 3; ++i) mbar_wait_bounded(w.bar(4 + ((k4 + i) & 3u)), ((k4 + i) >> 2) & 1u, grace);
        if (lane == 0) atomicExch(p.status, FKB_ERR_DEVICE_WAIT);
    }
}

// ---------------------------------------------------------------------------------------------------------
// nv12_kernel: NV12 -> RGB on the taps -> bilinear resize -> [Mul][Add|Sub][Div][SaturateCast] -> any write
// ---------------------------------------------------------------------------------------------------------
// The DNN-preprocessing shape.  Such launches are small and decimate heavily (a 4K frame to 640x640 moves 8 MB), so they
// are bound by latency, not bandwidth: one thread per output pixel, all twelve tap bytes requested before any is used,
// the colour matrix and the chain's operands held in registers, no interpretation.  The conversion runs on each tap
// before the interpolation, which is what the reference computes when ConvertYUVToRGB is fused into the Read under the
// Resize (algorithms/image_processing/color_conversion.h:150-174, interpolation.h:70-104).
// The ops after the interpolation and the write of one pixel, shared by the one-pixel-per-thread kernels: operands from
// Nv12Consts (immediates) or from the plane record (per-plane operands).
__device__ __forceinline__ void pixel_tail(const LaunchParams& p, const PlaneRec& pl, uint32_t x, uint32_t y, float (&v)[3]) {
    const Nv12Consts& k = p.nv12;
    float m[3], a[3], d[3];
    if (k.slots) {
        const PostParams q = load_post(p.chains[k.chain], pl, p.chains[k.chain].n_pre_ops);
#pragma unroll
        for (int c = 0; c < 3; ++c) { m[c] = q.m[c]; a[c] = q.a[c]; d[c] = q.d[c]; }
    } else {
#pragma unroll
        for (int c = 0; c < 3; ++c) { m[c] = k.m[c]; a[c] = k.a[c]; d[c] = k.d[c]; }
    }
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        if (k.kind & kPostMul) v[c] = __fmul_rn(v[c], m[c]);
        if (k.kind & kPostAdd) v[c] = __fadd_rn(v[c], a[c]);
        if (k.kind & kPostDiv) v[c] = __fdiv_rn(v[c], d[c]);
        if (k.kind & kPostSat) v[c] = sat_u8_as_float(v[c]);
    }
    uint8_t* row = pl.dst + static_cast<size_t>(y) * pl.dst_pitch;
    if (k.split) {
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            uint8_t* q8 = row + channel_offset(pl, c);
            if (k.f32) reinterpret_cast<float*>(q8)[x] = v[c]; else q8[x] = static_cast<uint8_t>(u8_of_exact(v[c]));
        }
    } else if (k.f32) {
        float* f = reinterpret_cast<float*>(row) + static_cast<size_t>(x) * 3;
        f[0] = v[0]; f[1] = v[1]; f[2] = v[2];
    } else {
        uint8_t* q8 = row + static_cast<size_t>(x) * 3;
        q8[0] = static_cast<uint8_t>(u8_of_exact(v[0])); q8[1] = static_cast<uint8_t>(u8_of_exact(v[1])); q8[2] = static_cast<uint8_t>(u8_of_exact(v[2]));
    }
}

__device__ __forceinline__ void nv12_pixel(const LaunchParams& p, const PlaneRec& pl, uint32_t x, uint32_t y) {
    if (pl.kclass != KCLASS_NV12) return;
    if (x >= pl.dst_w || y >= pl.dst_h) return;
    const Nv12Consts& k = p.nv12;
    const bool par = k.preserve_ar != 0;
    const bool inside = !par || (static_cast<int>(x) >= pl.x1 && static_cast<int>(x) <= pl.x2 &&
                                 static_cast<int>(y) >= pl.y1 && static_cast<int>(y) <= pl.y2);
    float v[3] = {pl.bg[0], pl.bg[1], pl.bg[2]};
    if (inside) {
        const AxisTap ax = axis_tap(static_cast<int>(x) - (par ? pl.x1 : 0), pl.fx, pl.crop_w);
        const AxisTap ay = axis_tap(static_cast<int>(y) - (par ? pl.y1 : 0), pl.fy, pl.crop_h);
        const uint32_t Xs[2] = {ax.i0 + pl.crop_x, ax.i1 + pl.crop_x}, Ys[2] = {ay.i0 + pl.crop_y, ay.i1 + pl.crop_y};
        const size_t pitch = pl.src_pitch;
        // the loads of all four taps first; tap t = (Xs[t & 1], Ys[t >> 1])
        uint32_t lum[4], cbs[4], crs[4];
        switch (k.yuv_fmt) {
        case FKB_PIX_UYVY:  // one aligned word U Y0 V Y1 per pixel pair
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint32_t X = Xs[t & 1];
                const uint32_t g = __ldg(reinterpret_cast<const uint32_t*>(pl.src + Ys[t >> 1] * pitch) + (X >> 1));
                lum[t] = (g >> (8u + 16u * (X & 1u))) & 0xffu; cbs[t] = g & 0xffu; crs[t] = (g >> 16) & 0xffu;
            }
            break;
        case FKB_PIX_P010: case FKB_PIX_P210:  // ushort luma; one aligned word (U,V) per pixel pair, every second row for 4:2:0
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint32_t X = Xs[t & 1], Y = Ys[t >> 1], cy = k.yuv_fmt == FKB_PIX_P010 ? Y >> 1 : Y;
                lum[t] = __ldg(reinterpret_cast<const unsigned short*>(pl.src + Y * pitch) + X);
                const uint32_t g = __ldg(reinterpret_cast<const uint32_t*>(pl.src_chroma + cy * pitch) + (X >> 1));
                cbs[t] = g & 0xffffu; crs[t] = g >> 16;
            }
            break;
        case FKB_PIX_Y210:  // one aligned ushort4 Y0 U Y1 V per pixel pair
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint32_t X = Xs[t & 1];
                const uint2 g = __ldg(reinterpret_cast<const uint2*>(pl.src + Ys[t >> 1] * pitch) + (X >> 1));
                lum[t] = (X & 1u) ? g.y & 0xffffu : g.x & 0xffffu; cbs[t] = g.x >> 16; crs[t] = g.y >> 16;
            }
            break;
        default:  // NV12 / NV21: byte luma, one aligned 16-bit word per chroma pair
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint32_t X = Xs[t & 1], Y = Ys[t >> 1];
                lum[t] = __ldg(pl.src + Y * pitch + X);
                const uint32_t g = __ldg(reinterpret_cast<const unsigned short*>(pl.src_chroma + (Y >> 1) * pitch) + (X >> 1));
                cbs[t] = k.vu ? g >> 8 : g & 0xffu; crs[t] = k.vu ? g & 0xffu : g >> 8;
            }
            break;
        }
        const float w00 = __fmul_rn(ax.w0, ay.w0), w10 = __fmul_rn(ax.w1, ay.w0);
        const float w01 = __fmul_rn(ax.w0, ay.w1), w11 = __fmul_rn(ax.w1, ay.w1);
        const float w[4] = {w00, w10, w01, w11};
        float acc[3];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const float yy = static_cast<float>(lum[t]);
            const float a = k.sub[0] != 0.f ? __fsub_rn(yy, k.sub[0]) : yy;  // x - 0 is x
            const float b = __fsub_rn(static_cast<float>(cbs[t]), k.sub[1]);
            const float d = __fsub_rn(static_cast<float>(crs[t]), k.sub[2]);
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                const float rgb = __fadd_rn(__fadd_rn(__fmul_rn(a, k.ccm[3 * c]), __fmul_rn(b, k.ccm[3 * c + 1])), __fmul_rn(d, k.ccm[3 * c + 2]));
                const float term = __fmul_rn(rgb, w[t]);
                acc[c] = t == 0 ? term : __fadd_rn(acc[c], term);  // ((t0 + t1) + t2) + t3, the reference's order
            }
        }
#pragma unroll
        for (int c = 0; c < 3; ++c) v[c] = acc[c];
    }
    pixel_tail(p, pl, x, y, v);
}

// rgb_kernel: the same latency-oriented shape for packed byte sources (uchar3, or uchar4 whose alpha is skipped): one output
// pixel per thread, the twelve tap bytes requested before any is used, the post-ops' operands in registers.  It serves the
// launches of a few ten thousand pixels, where the general kernel's per-tap format dispatch and op interpreter are most of
// the time.
__device__ __forceinline__ void rgb_pixel(const LaunchParams& p, const PlaneRec& pl, uint32_t x, uint32_t y) {
    if (pl.kclass != KCLASS_NV12) return;
    if (x >= pl.dst_w || y >= pl.dst_h) return;
    const Nv12Consts& k = p.nv12;
    const bool par = k.preserve_ar != 0;
    const bool inside = !par || (static_cast<int>(x) >= pl.x1 && static_cast<int>(x) <= pl.x2 &&
                                 static_cast<int>(y) >= pl.y1 && static_cast<int>(y) <= pl.y2);
    float v[3] = {pl.bg[0], pl.bg[1], pl.bg[2]};
    if (inside) {
        const AxisTap ax = axis_tap(static_cast<int>(x) - (par ? pl.x1 : 0), pl.fx, pl.crop_w);
        const AxisTap ay = axis_tap(static_cast<int>(y) - (par ? pl.y1 : 0), pl.fy, pl.crop_h);
        const uint32_t sp = k.src_px, pitch = pl.src_pitch;
        const uint8_t* r0 = pl.src + static_cast<size_t>(ay.i0 + pl.crop_y) * pitch;
        const uint8_t* r1 = pl.src + static_cast<size_t>(ay.i1 + pl.crop_y) * pitch;
        const uint32_t o0 = (ax.i0 + pl.crop_x) * sp, o1 = (ax.i1 + pl.crop_x) * sp;
        uint32_t t[4][3];
#pragma unroll
        for (int c = 0; c < 3; ++c) { t[0][c] = __ldg(r0 + o0 + c); t[1][c] = __ldg(r0 + o1 + c); t[2][c] = __ldg(r1 + o0 + c); t[3][c] = __ldg(r1 + o1 + c); }
        const float w00 = __fmul_rn(ax.w0, ay.w0), w10 = __fmul_rn(ax.w1, ay.w0);
        const float w01 = __fmul_rn(ax.w0, ay.w1), w11 = __fmul_rn(ax.w1, ay.w1);
#pragma unroll
        for (int c = 0; c < 3; ++c)
            v[c] = bilerp(static_cast<float>(t[0][c]), static_cast<float>(t[1][c]), static_cast<float>(t[2][c]), static_cast<float>(t[3][c]), w00, w10, w01, w11);
    }
    pixel_tail(p, pl, x, y, v);
}

__global__ void __launch_bounds__(256, 4) rgb_kernel(const __grid_constant__ LaunchParams p) {
    pdl_signal();
    pdl_wait();
    const uint32_t x = blockIdx.x * 32 + (threadIdx.x & 31), y = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (p.table == nullptr) {
        for (uint32_t z = p.pixel_z0 + blockIdx.z; z < p.pixel_z1; z += gridDim.z) rgb_pixel(p, p.inline_planes[z], x, y);
    } else {
        for (uint32_t z = p.pixel_z0 + blockIdx.z; z < p.pixel_z1; z += gridDim.z) rgb_pixel(p, p.table[z], x, y);
    }
}

__global__ void __launch_bounds__(256, 8) nv12_kernel(const __grid_constant__ LaunchParams p) {
    pdl_signal();
    pdl_wait();
    const uint32_t x = blockIdx.x * 32 + (threadIdx.x & 31), y = blockIdx.y * 8 + (threadIdx.x >> 5);
    // Two copies of the body so that each knows where its plane records live: in the kernel parameters (constant-bank
    // reads, shared by all threads) for launches of a few planes, in the global table otherwise.
    if (p.table == nullptr) {
        for (uint32_t z = p.pixel_z0 + blockIdx.z; z < p.pixel_z1; z += gridDim.z) nv12_pixel(p, p.inline_planes[z], x, y);
    } else {
        for (uint32_t z = p.pixel_z0 + blockIdx.z; z < p.pixel_z1; z += gridDim.z) nv12_pixel(p, p.table[z], x, y);
    }
}

// nv12_pair_kernel: the same chain for the colour matrices every YCbCr standard uses, two output pixels per thread.
// Conditions (checked on the host): the matrix has the shape [s 0 r; s g1 g2; s b 0] with s > 0, the offsets are
// integers in [0,255], the operands are immediates, and every offset into a plane fits 32 bits.  Under them
//   * (Y*s + Cb*0) + Cr*r == Y*s + Cr*r bit for bit (a finite x times 0 is a zero, and adding a zero of either sign to
//     a value that is never -0 changes nothing: Y - offset is an exact integer difference, so its zero is +0, and so
//     is that zero times a positive s), and likewise for the blue row, which drops six of the fifteen operations per tap;
//   * byte - offset is computed as (2^23 + byte) - (2^23 + offset): one byte-permute and one exact subtraction;
//   * the two pixels of a thread share every coefficient, so the arithmetic runs as packed f32x2 operations.
// A product that feeds only a sum is written as fma(a, b, -0), which the assembler cannot contract with the sum.
struct PairTaps {
    uint32_t x0, x1;
    float w0, w1;
};
__device__ __forceinline__ f2 magic_pair(uint32_t wa, uint32_t wb, uint32_t sel) {
    return f2{__uint_as_float(__byte_perm(wa, 0x4B000000u, sel)), __uint_as_float(__byte_perm(wb, 0x4B000000u, sel))};
}
template <bool SCALED_LUMA, bool VU>
__device__ __forceinline__ void nv12_pair(const Nv12Consts& k, const float nz, const PlaneRec& pl, uint32_t xa, uint32_t y) {
    if (pl.kclass != KCLASS_NV12) return;
    if (xa >= pl.dst_w || y >= pl.dst_h) return;
    const bool par = k.preserve_ar != 0;
    const uint32_t xb = xa + 1;
    const bool has_b = xb < pl.dst_w;
    const int ox = par ? pl.x1 : 0, oy = par ? pl.y1 : 0;
    // taps are computed for clamped coordinates, so that every address is valid; letterbox pixels are replaced below
    const AxisTap ta = axis_tap(max(static_cast<int>(xa) - ox, 0), pl.fx, pl.crop_w);
    const AxisTap tb = axis_tap(max(static_cast<int>(xb) - ox, 0), pl.fx, pl.crop_w);
    const AxisTap ty = axis_tap(max(static_cast<int>(y) - oy, 0), pl.fy, pl.crop_h);
    const uint32_t pitch = pl.src_pitch;
    const uint32_t Y0 = ty.i0 + pl.crop_y, Y1 = ty.i1 + pl.crop_y;
    const uint32_t ry0 = Y0 * pitch + pl.crop_x, ry1 = Y1 * pitch + pl.crop_x;
    const uint32_t rc0 = (Y0 >> 1) * pitch, rc1 = (Y1 >> 1) * pitch;
    const uint32_t ua0 = (ta.i0 + pl.crop_x) & ~1u, ua1 = (ta.i1 + pl.crop_x) & ~1u;
    const uint32_t ub0 = (tb.i0 + pl.crop_x) & ~1u, ub1 = (tb.i1 + pl.crop_x) & ~1u;
    const uint8_t* __restrict__ lum = pl.src;
    const uint8_t* __restrict__ chr = pl.src_chroma;
    // tap order: (x0,y0) (x1,y0) (x0,y1) (x1,y1); all sixteen loads are requested before any is used
    uint32_t la[4], lb[4], ca[4], cb[4];
    la[0] = __ldg(lum + (ry0 + ta.i0)); la[1] = __ldg(lum + (ry0 + ta.i1)); la[2] = __ldg(lum + (ry1 + ta.i0)); la[3] = __ldg(lum + (ry1 + ta.i1));
    lb[0] = __ldg(lum + (ry0 + tb.i0)); lb[1] = __ldg(lum + (ry0 + tb.i1)); lb[2] = __ldg(lum + (ry1 + tb.i0)); lb[3] = __ldg(lum + (ry1 + tb.i1));
    ca[0] = __ldg(reinterpret_cast<const unsigned short*>(chr + (rc0 + ua0))); ca[1] = __ldg(reinterpret_cast<const unsigned short*>(chr + (rc0 + ua1)));
    ca[2] = __ldg(reinterpret_cast<const unsigned short*>(chr + (rc1 + ua0))); ca[3] = __ldg(reinterpret_cast<const unsigned short*>(chr + (rc1 + ua1)));
    cb[0] = __ldg(reinterpret_cast<const unsigned short*>(chr + (rc0 + ub0))); cb[1] = __ldg(reinterpret_cast<const unsigned short*>(chr + (rc0 + ub1)));
    cb[2] = __ldg(reinterpret_cast<const unsigned short*>(chr + (rc1 + ub0))); cb[3] = __ldg(reinterpret_cast<const unsigned short*>(chr + (rc1 + ub1)));
    const f2 wy0{ty.w0, ty.w0}, wy1{ty.w1, ty.w1};
    const f2 wx0{ta.w0, tb.w0}, wx1{ta.w1, tb.w1};
    const f2 w[4] = {mul2(wx0, wy0), mul2(wx1, wy0), mul2(wx0, wy1), mul2(wx1, wy1)};
    const f2 ky{-k.kmag[0], -k.kmag[0]}, ku{-k.kmag[1], -k.kmag[1]}, kv{-k.kmag[2], -k.kmag[2]};
    const f2 cr{k.ccm[2], k.ccm[2]}, cg1{k.ccm[4], k.ccm[4]}, cg2{k.ccm[5], k.ccm[5]}, cbl{k.ccm[7], k.ccm[7]}, cy{k.ccm[0], k.ccm[0]};
    constexpr uint32_t sel_u = VU ? 0x7441u : 0x7440u, sel_v = VU ? 0x7440u : 0x7441u;  // which byte of a chroma pair is Cb
    f2 acc[3];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const f2 yy = add2(magic_pair(la[t], lb[t], 0x7440u), ky);
        const f2 uu = add2(magic_pair(ca[t], cb[t], sel_u), ku);
        const f2 vv = add2(magic_pair(ca[t], cb[t], sel_v), kv);
        const f2 ys = SCALED_LUMA ? mul2_unfusable(yy, cy, nz) : yy;  // the luma column is 1 for full range, and x * 1 is x
        const f2 r = add2(ys, mul2_unfusable(vv, cr, nz));
        const f2 g = add2(add2(ys, mul2_unfusable(uu, cg1, nz)), mul2_unfusable(vv, cg2, nz));
        const f2 b = add2(ys, mul2_unfusable(uu, cbl, nz));
        const f2 tr = mul2_unfusable(r, w[t], nz), tg = mul2_unfusable(g, w[t], nz), tbb = mul2_unfusable(b, w[t], nz);
        acc[0] = t == 0 ? tr : add2(acc[0], tr);
        acc[1] = t == 0 ? tg : add2(acc[1], tg);
        acc[2] = t == 0 ? tbb : add2(acc[2], tbb);
    }
    if (par) {
        const bool row_in = static_cast<int>(y) >= pl.y1 && static_cast<int>(y) <= pl.y2;
        const bool in_a = row_in && static_cast<int>(xa) >= pl.x1 && static_cast<int>(xa) <= pl.x2;
        const bool in_b = row_in && static_cast<int>(xb) >= pl.x1 && static_cast<int>(xb) <= pl.x2;
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            if (!in_a) acc[c].x = pl.bg[c];
            if (!in_b) acc[c].y = pl.bg[c];
        }
    }
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        if (k.kind & kPostMul) acc[c] = mul2_unfusable(acc[c], f2{k.m[c], k.m[c]}, nz);
        if (k.kind & kPostAdd) acc[c] = add2(acc[c], f2{k.a[c], k.a[c]});
        if (k.kind & kPostDiv) { acc[c].x = __fdiv_rn(acc[c].x, k.d[c]); acc[c].y = __fdiv_rn(acc[c].y, k.d[c]); }
        if (k.kind & kPostSat) { acc[c].x = sat_u8_as_float(acc[c].x); acc[c].y = sat_u8_as_float(acc[c].y); }
    }
    uint8_t* __restrict__ row = pl.dst + y * pl.dst_pitch;
    if (k.f32) {
        if (k.split) {
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                float* q = reinterpret_cast<float*>(row + channel_offset(pl, c)) + xa;
                if (has_b && k.wide_store) *reinterpret_cast<float2*>(q) = make_float2(acc[c].x, acc[c].y);
                else { q[0] = acc[c].x; if (has_b) q[1] = acc[c].y; }
            }
        } else {
            float* q = reinterpret_cast<float*>(row) + xa * 3u;
            if (has_b && k.wide_store) {
                reinterpret_cast<float2*>(q)[0] = make_float2(acc[0].x, acc[1].x);
                reinterpret_cast<float2*>(q)[1] = make_float2(acc[2].x, acc[0].y);
                reinterpret_cast<float2*>(q)[2] = make_float2(acc[1].y, acc[2].y);
            } else {
                q[0] = acc[0].x; q[1] = acc[1].x; q[2] = acc[2].x;
                if (has_b) { q[3] = acc[0].y; q[4] = acc[1].y; q[5] = acc[2].y; }
            }
        }
    } else {
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            uint8_t* q = k.split ? row + channel_offset(pl, c) + xa : row + xa * 3u + c;
            const uint32_t step = k.split ? 1u : 3u;
            q[0] = static_cast<uint8_t>(u8_of_exact(acc[c].x));
            if (has_b) q[step] = static_cast<uint8_t>(u8_of_exact(acc[c].y));
        }
    }
}

template <int THREADS, int MINB, bool SCALED_LUMA, bool VU>
__global__ void __launch_bounds__(THREADS, MINB) nv12_pair_kernel(const __grid_constant__ LaunchParams p) {
    pdl_signal();
    pdl_wait();
    const uint32_t x = (blockIdx.x * 32 + (threadIdx.x & 31)) * 2, y = blockIdx.y * (THREADS / 32) + (threadIdx.x >> 5);
    // two copies of the body, so that each knows where its plane records live: a few kernel-parameter records, or a table
    if (p.table == nullptr) {
        for (uint32_t z = p.pixel_z0 + blockIdx.z; z < p.pixel_z1; z += gridDim.z) nv12_pair<SCALED_LUMA, VU>(p.nv12, p.neg_zero, p.inline_planes[z], x, y);
    } else {
        for (uint32_t z = p.pixel_z0 + blockIdx.z; z < p.pixel_z1; z += gridDim.z) nv12_pair<SCALED_LUMA, VU>(p.nv12, p.neg_zero, p.table[z], x, y);
    }
}
// The one-plane launch (a frame into a network's input tensor) carries only what it reads — the chain's constants and the
// plane's record, 0.4 KB instead of the 5.6 KB of LaunchParams: every field is a constant-bank operand at a fixed offset,
// and a launch this short feels the size of its parameter block.
struct PairParams1 {
    Nv12Consts nv12;
    float neg_zero;
    PlaneRec plane;
};
template <int THREADS, int MINB, bool SCALED_LUMA, bool VU>
__global__ void __launch_bounds__(THREADS, MINB) nv12_pair1_kernel(const __grid_constant__ PairParams1 q) {
    pdl_signal();
    pdl_wait();
    const uint32_t x = (blockIdx.x * 32 + (threadIdx.x & 31)) * 2, y = blockIdx.y * (THREADS / 32) + (threadIdx.x >> 5);
    nv12_pair<SCALED_LUMA, VU>(q.nv12, q.neg_zero, q.plane, x, y);
}

// ---------------------------------------------------------------------------------------------------------
// lut_kernel: uchar3 -> uchar3 chains without resampling
// ---------------------------------------------------------------------------------------------------------
// Every op of such a chain acts on one channel at a time (a channel reorder only renames channels), so output channel c
// is a function of one source byte: out[c] = T_c(in[perm(c)]).  Each CTA evaluates the chain — through the same op
// interpreter as every other path, so the table is exact by construction — once for the 256 possible bytes, and then
// every pixel costs three table reads instead of the whole chain (IEEE divisions and saturations included).  An entry
// is one 32-bit word holding the three channels' results for that byte value, and every lane reads its own copy of the
// table (copy l lives in bank l), so a table read is free of bank conflicts whatever the pixel values are.  The rows of
// the table are 256 bytes apart (the copies fill the first 128), so the address of a read — value * 256 + lane * 4 — is
// one byte-permute that drops the source byte into byte 1 of a word whose byte 0 is lane * 4.
// One CTA of 24 warps per SM.  Rows move like in staged_kernel — per-warp bulk loads into shared memory, bulk stores out —
// but a segment is transformed in place (a lane reads its 16 pixels, then writes them back), so each warp needs only one
// ring of four buffers: one being computed, two loads in flight, one store still being read.
__device__ __forceinline__ uint32_t unit_to_plane(const LaunchParams& p, uint32_t u, uint32_t& local) {
    const PlaneRec* table = plane_table(p);
    uint32_t lo = 0, hi = p.n_planes;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (table[mid].lut_base <= u) lo = mid; else hi = mid;
    }
    local = u - table[lo].lut_base;
    return lo;
}

template <bool SWAP>
__device__ __forceinline__ void lut_segment(uint32_t seg, uint32_t ow, uint32_t lane) {
    if (lane * 16u >= ow) return;
    uint4* buf = reinterpret_cast<uint4*>(smem_raw + seg + lane * 48u);
    uint32_t q[12];
#pragma unroll
    for (int i = 0; i < 3; ++i) { const uint4 t = buf[i]; q[4 * i] = t.x; q[4 * i + 1] = t.y; q[4 * i + 2] = t.z; q[4 * i + 3] = t.w; }
    const uint32_t lane_word = lane * 4u | kLutTableAddr;  // bytes 0, 2 and 3 of every table address
    uint32_t o[12];
#pragma unroll
    for (int i = 0; i < 12; ++i) {
        uint32_t e[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int b = 4 * i + t, c = b % 3;          // output byte b is channel c of pixel b / 3
            const int sb = SWAP ? b - c + (2 - c) : b;   // the source byte it is a function of
            // absolute shared address of lane's copy of the entry: 0x10000 | value << 8 | lane << 2, one byte permute
            const uint32_t at = __byte_perm(q[sb >> 2], lane_word, 0x7604u | ((sb & 3) << 4));
            asm("ld.shared.u32 %0, [%1];" : "=r"(e[t]) : "r"(at));
        }
        // byte (4i+t) % 3 of entry t is the channel this output byte wants
        const uint32_t c0 = (4 * i) % 3, c1 = (4 * i + 1) % 3, c2 = (4 * i + 2) % 3, c3 = (4 * i + 3) % 3;  // constants once unrolled
        o[i] = __byte_perm(__byte_perm(e[0], e[1], c0 | ((4u + c1) << 4)), __byte_perm(e[2], e[3], c2 | ((4u + c3) << 4)), 0x5410u);
    }
#pragma unroll
    for (int i = 0; i < 3; ++i) buf[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
}

__global__ void __launch_bounds__(kLutThreads, 1) lut_kernel(const __grid_constant__ LaunchParams p) {
    pdl_signal();
    __shared__ PlaneRec s_pl;
    __shared__ uint32_t s_entry[256];
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // tells the compiler the value is warp-uniform
    // Where things are: the table at the absolute shared address kLutTableAddr, warp slices below it as far as they fit
    // (from the first 128-byte boundary of the dynamic region) and above it for the rest.  Offsets are relative to smem_raw.
    const uint32_t sbase = smem_addr(smem_raw);
    const uint32_t low0 = ((sbase + 127u) & ~127u) - sbase;                       // first slice below the table
    const uint32_t n_low = sbase + low0 < kLutTableAddr ? (kLutTableAddr - sbase - low0) / kLutSliceBytes : 0u;
    const uint32_t table = kLutTableAddr - sbase;                                 // (offset of the table in smem_raw)
    if (sbase > kLutTableAddr || table + kLutBytes + (kLutWarps - min(n_low, kLutWarps)) * kLutSliceBytes > kLutSmemBytes) {
        pdl_wait();
        if (threadIdx.x == 0) atomicExch(p.status, FKB_ERR_DEVICE_WAIT);          // the layout does not fit: nothing is touched
        return;
    }
    const uint32_t slice = warp < n_low ? low0 + warp * kLutSliceBytes : table + kLutBytes + (warp - n_low) * kLutSliceBytes;
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw + slice);
    const uint32_t buf0 = slice + 64;
    if (lane == 0) {
        for (uint32_t i = 0; i < kLutStages; ++i) mbar_init(&bar[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    pdl_wait();  // nothing above touches global memory
    const PlaneRec* tbl = plane_table(p);
    uint32_t cur_plane = 0xffffffffu, k = 0;
    bool ok = true;
    for (uint32_t unit = blockIdx.x; unit < p.n_lut_units; unit += gridDim.x) {
        uint32_t local;
        const uint32_t z = unit_to_plane(p, unit, local);
        const bool rebuild = z != cur_plane;  // block-uniform
        if (rebuild) {
            __syncthreads();  // nobody reads the old table or plane record any more
            if (threadIdx.x < sizeof(PlaneRec) / 16)
                reinterpret_cast<uint4*>(&s_pl)[threadIdx.x] = reinterpret_cast<const uint4*>(tbl + z)[threadIdx.x];
            __syncthreads();
        }
        const PlaneRec& pl = s_pl;
        const bool swap = (p.lut_swap >> pl.chain) & 1u;
        const uint32_t row0 = local * pl.tile_h, nrows = min(pl.tile_h, pl.dst_h - row0);
        const uint32_t nseg = nrows * pl.tiles_x;
        const uint8_t* gsrc = pl.src + static_cast<size_t>(pl.crop_y + row0) * pl.src_pitch + static_cast<size_t>(pl.crop_x) * 3u;
        uint8_t* gdst = pl.dst + static_cast<size_t>(row0) * pl.dst_pitch;
        const uint32_t src_pitch = pl.src_pitch, dst_pitch = pl.dst_pitch, tiles_x = pl.tiles_x, tile_w = pl.tile_w, dst_w = pl.dst_w;
        // Segment g of the unit is (row g / tiles_x, column tile g % tiles_x); this warp takes g = warp, warp + 24, ...
        // Two cursors walk that list without dividing: `pf` for the loads, three segments ahead of `cu`, the one computed.
        struct Cursor { uint32_t g, r, tx; };
        const uint32_t step_r = kLutWarps / tiles_x, step_tx = kLutWarps % tiles_x;
        auto advance = [&](Cursor& c) {
            c.g += kLutWarps; c.tx += step_tx; c.r += step_r;
            if (c.tx >= tiles_x) { c.tx -= tiles_x; ++c.r; }
        };
        auto issue = [&](const Cursor& c, uint32_t s) {
            const uint32_t ow = min(tile_w, dst_w - c.tx * tile_w);
            const uint32_t bytes = (ow * 3u + 15u) & ~15u;
            const uint8_t* from = gsrc + static_cast<size_t>(c.r) * src_pitch + static_cast<size_t>(c.tx) * tile_w * 3u;
            bool good = true;
            if (kSelfChecking)
                good = self_check(&g_status_word, bulk_range_ok(from, bytes, pl.src, static_cast<size_t>(pl.src_pitch) * pl.src_h) && bytes <= kLutSegBytes);
            mbar_arrive_expect_tx(&bar[s], good ? bytes : 0u);
            if (good) bulk_load(smem_raw + buf0 + s * kLutSegBytes, from, bytes, &bar[s]);
        };
        Cursor cu{warp, warp / tiles_x, warp % tiles_x}, pf = cu;
        constexpr uint32_t AHEAD = kLutStages - 1;
        if (lane == 0) bulk_wait_read_all();  // the ring's earlier stores have been read out of their buffers
        for (uint32_t i = 0; i < AHEAD; ++i) {  // the first loads fly while the table is built
            if (lane == 0 && pf.g < nseg) issue(pf, (k + i) % kLutStages);
            advance(pf);
        }
        if (rebuild) {
            const fkb_chain_desc& ch = p.chains[pl.chain];
            if (threadIdx.x < 256) {
                const float t = static_cast<float>(threadIdx.x);
                float v[1][3] = {{t, t, t}};
                apply_ops<1>(v, ch, pl, 0, ch.n_ops);
                s_entry[threadIdx.x] = u8_of_exact(v[0][0]) | (u8_of_exact(v[0][1]) << 8) | (u8_of_exact(v[0][2]) << 16);
            }
            __syncthreads();
            // copy l of value v sits at v * 256 + l * 4: consecutive threads write consecutive words of a row
            for (uint32_t w = threadIdx.x; w < 256u * 32u; w += kLutThreads)
                *reinterpret_cast<uint32_t*>(smem_raw + table + (w >> 5) * 256u + (w & 31u) * 4u) = s_entry[w >> 5];
            __syncthreads();
            cur_plane = z;
        }
        // Per segment: wait for it, transform it in place, and then — lane 0's one divergent stretch — send it off, wait
        // until the store of the segment before has read its buffer, and request the segment three ahead into that buffer.
        for (; cu.g < nseg && ok; advance(cu), advance(pf), ++k) {
            const uint32_t s = k % kLutStages;
            const bool landed = mbar_wait_bounded(&bar[s], (k / kLutStages) & 1u, p.wait_limit_ns);
            if (__any_sync(0xffffffffu, !landed)) { ok = false; break; }
            const uint32_t ow = min(tile_w, dst_w - cu.tx * tile_w);
            const uint32_t seg = buf0 + s * kLutSegBytes;
            if (swap) lut_segment<true>(seg, ow, lane);
            else lut_segment<false>(seg, ow, lane);
            uint8_t* out = gdst + static_cast<size_t>(cu.r) * dst_pitch + static_cast<size_t>(cu.tx) * tile_w * 3u;
            const uint32_t out_bytes = ow * 3u, out_bulk = out_bytes & ~15u;
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                bool store = out_bulk != 0;
                if (kSelfChecking && store)
                    store = self_check(&g_status_word, bulk_range_ok(out, out_bulk, pl.dst, static_cast<size_t>(pl.dst_pitch) * pl.dst_h));
                if (store) bulk_store(out, smem_raw + seg, out_bulk);
                bulk_commit();
                bulk_wait_read_1();
                if (pf.g < nseg) issue(pf, (k + AHEAD) % kLutStages);
            }
            if (out_bytes != out_bulk && lane < out_bytes - out_bulk) out[out_bulk + lane] = smem_raw[seg + out_bulk + lane];  // rare
        }
        if (__syncthreads_or(ok ? 0 : 1)) { ok = false; break; }
    }
    if (lane == 0) bulk_wait_all();
    if (!ok) {
        for (uint32_t i = 1; i < kLutStages; ++i) mbar_wait_bounded(&bar[(k + i) % kLutStages], ((k + i) / kLutStages) & 1u, min(p.wait_limit_ns, 1000000u));
        if (threadIdx.x == 0) atomicExch(p.status, FKB_ERR_DEVICE_WAIT);
    }
}

// ---------------------------------------------------------------------------------------------------------
// host-callable launchers (the only symbols the host translation unit needs from this file)
// ---------------------------------------------------------------------------------------------------------
// Every kernel is launched with programmatic stream serialisation allowed: when the operation before it in the stream
// is one of this library's kernels (which all signal griddepcontrol.launch_dependents at their start), the GPU may set
// the new grid up — launch latency, CTA scheduling, the prologue that touches no global memory — while the earlier grid
// is still running; every kernel executes griddepcontrol.wait before its first access to global memory, and that
// instruction returns only when the earlier grid has completed and its writes are visible.  After any other kind of
// operation, or after a kernel that does not signal, the launch is ordered as usual.  Measured on chains of dependent
// launches: a kernel of four microseconds and more gains 0.5 to 0.9 us, one of two microseconds loses 0.9 us (the wait
// resolves later than a plain kernel boundary), so the host sets LaunchParams::pdl only for launches of 200 000 output
// pixels and more.  FKB_PDL=0 switches the attribute off altogether.
bool pdl_allowed() {
    static const bool on = [] { const char* e = std::getenv("FKB_PDL"); return !(e && e[0] == '0'); }();
    return on;
}
template <typename P>
cudaError_t launch_kernel(void (*kernel)(P), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, const P& params, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = (pdl && pdl_allowed()) ? 1u : 0u;
    return cudaLaunchKernelEx(&cfg, kernel, params);
}
cudaError_t launch_staged(const LaunchParams& p, uint32_t grid, cudaStream_t stream) {
    static thread_local int configured_device = -1;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (configured_device != dev) {
        e = cudaFuncSetAttribute(staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kStagedSmemBytes));
        if (e != cudaSuccess) return e;
        configured_device = dev;
    }
    launch_kernel(staged_kernel, grid, kStagedThreads, kStagedSmemBytes, stream, p, p.pdl != 0);
    return cudaGetLastError();
}

#ifdef FKB_PHASE_CLOCKS
}  // namespace fkb
// Only in the phase-clock build: the sums over all warps since the last reset (see PhaseClock) go to out[0 .. n), at most
// kPhaseCount of them.
extern "C" int fkb_debug_phase_clocks(unsigned long long* out, int n, int reset) {
    static unsigned long long host[fkb::kPhaseSlots][fkb::kPhaseCount];
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (out) {
        if (cudaMemcpyFromSymbol(host, fkb::g_phase_clocks, sizeof(host)) != cudaSuccess) return -1;
        for (int i = 0; i < n && i < fkb::kPhaseCount; ++i) {
            out[i] = 0;
            for (uint32_t s = 0; s < fkb::kPhaseSlots; ++s) out[i] += host[s][i];
        }
    }
    if (reset) {
        void* sym = nullptr;
        if (cudaGetSymbolAddress(&sym, fkb::g_phase_clocks) != cudaSuccess || cudaMemset(sym, 0, sizeof(host)) != cudaSuccess) return -1;
    }
    return 0;
}
namespace fkb {
#endif

cudaError_t launch_lut(const LaunchParams& p, uint32_t grid, cudaStream_t stream) {
    static thread_local int configured_device = -1;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (configured_device != dev) {
        e = cudaFuncSetAttribute(lut_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kLutSmemBytes));
        if (e != cudaSuccess) return e;
        configured_device = dev;
    }
    launch_kernel(lut_kernel, grid, kLutThreads, kLutSmemBytes, stream, p, p.pdl != 0);
    return cudaGetLastError();
}

cudaError_t launch_nv12(const LaunchParams& p, dim3 grid, cudaStream_t stream) {
    // the pair kernel runs 128-thread CTAs (four rows of 64 pixels), ten per SM: more, smaller CTAs shorten the tail
    if (p.nv12.pair) {
        const dim3 g(grid.x, grid.y * 2, grid.z);
        const bool scaled = p.nv12.ccm[0] != 1.f;
        if (p.table == nullptr && p.n_planes == 1) {
            PairParams1 q;
            q.nv12 = p.nv12; q.neg_zero = p.neg_zero; q.plane = p.inline_planes[0];
            if (scaled && p.nv12.vu) launch_kernel(nv12_pair1_kernel<128, 10, true, true>, g, 128, 0, stream, q, p.pdl != 0);
            else if (scaled) launch_kernel(nv12_pair1_kernel<128, 10, true, false>, g, 128, 0, stream, q, p.pdl != 0);
            else if (p.nv12.vu) launch_kernel(nv12_pair1_kernel<128, 10, false, true>, g, 128, 0, stream, q, p.pdl != 0);
            else launch_kernel(nv12_pair1_kernel<128, 10, false, false>, g, 128, 0, stream, q, p.pdl != 0);
        }
        else if (scaled && p.nv12.vu) launch_kernel(nv12_pair_kernel<128, 10, true, true>, g, 128, 0, stream, p, p.pdl != 0);
        else if (scaled) launch_kernel(nv12_pair_kernel<128, 10, true, false>, g, 128, 0, stream, p, p.pdl != 0);
        else if (p.nv12.vu) launch_kernel(nv12_pair_kernel<128, 10, false, true>, g, 128, 0, stream, p, p.pdl != 0);
        else launch_kernel(nv12_pair_kernel<128, 10, false, false>, g, 128, 0, stream, p, p.pdl != 0);
    }
    else if (p.nv12.src_px) launch_kernel(rgb_kernel, grid, 256, 0, stream, p, p.pdl != 0);
    else launch_kernel(nv12_kernel, grid, 256, 0, stream, p, p.pdl != 0);
    return cudaGetLastError();
}

cudaError_t launch_gather4(const LaunchParams& p, dim3 grid, cudaStream_t stream) {
    if (p.four.enabled) {
        const dim3 g2((grid.x + 1) / 2, grid.y, grid.z);  // two pixels per thread
#define FKB_RGBA(N) (p.four.src3 ? launch_kernel(rgba_kernel<N, true>, g2, 256, 0, stream, p, p.pdl != 0) : launch_kernel(rgba_kernel<N, false>, g2, 256, 0, stream, p, p.pdl != 0))
        switch (p.four.n_steps) {
        case 0: FKB_RGBA(0); break;
        case 1: FKB_RGBA(1); break;
        case 2: FKB_RGBA(2); break;
        case 3: FKB_RGBA(3); break;
        case 4: FKB_RGBA(4); break;
        case 5: FKB_RGBA(5); break;
        default: FKB_RGBA(6); break;
        }
#undef FKB_RGBA
        return cudaGetLastError();
    }
    launch_kernel(gather4_kernel, grid, 256, 0, stream, p, p.pdl != 0);
    return cudaGetLastError();
}

cudaError_t launch_gather(const LaunchParams& p, dim3 grid, int pixels_per_thread, cudaStream_t stream) {
    const bool inl = p.table == nullptr;
    if (pixels_per_thread == 1) { if (inl) launch_kernel(gather_kernel<1, true>, grid, 256, 0, stream, p, p.pdl != 0); else launch_kernel(gather_kernel<1, false>, grid, 256, 0, stream, p, p.pdl != 0); }
    else { if (inl) launch_kernel(gather_kernel<4, true>, grid, 256, 0, stream, p, p.pdl != 0); else launch_kernel(gather_kernel<4, false>, grid, 256, 0, stream, p, p.pdl != 0); }
    return cudaGetLastError();
}

cudaError_t status_word_address(int** out) { return cudaGetSymbolAddress(reinterpret_cast<void**>(out), g_status_word); }

}  // namespace fkb
