// The two sm_100a kernels behind fkb_launch_*:
//
//   staged_kernel  — persistent CTAs (two per SM).  Each CTA walks a strided list of output tiles.  For every
//                    tile it (1) stages the tile's bounded source footprint into shared memory with
//                    non-multicast bulk async copies (cp.async.bulk, one per source row, completion on an
//                    mbarrier), double-buffered so the next tile's footprint is in flight while this one is
//                    computed, (2) computes the tile from shared memory into a shared output tile and (3)
//                    writes that tile with bulk async stores (full 16-byte-aligned lines, no partial sectors).
//                    Two tile kinds: POINT (no resampling, 16 or 4 pixels per thread, 128-bit shared accesses)
//                    and RESIZE (bilinear from the staged footprint).  The chain of a plane is picked once per
//                    tile, so a divergent launch never diverges inside a warp.
//   gather_kernel  — the general path: any source format (uchar3, NV12), ops before the interpolation, planar
//                    writes, unaligned buffers, or footprints too sparse/large to stage (heavy decimation).
//                    Four pixels per thread, read-only global loads, vector stores when aligned.
//
// Replaces launchTransformDPP_Kernel / launchDivergentBatchTransformDPP_Kernel of the reference
// (core/execution_model/executor_details/executor_kernels.h:20-30).  No tensor cores: nothing here is a
// contraction; the bound is HBM bandwidth.
#include "fkb_device.cuh"
#include "fkb_launch.h"

namespace fkb {

// ---------------------------------------------------------------------------------------------------------
// shared helpers
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ const PlaneRec* plane_table(const LaunchParams& p) {
    return p.table ? p.table : p.inline_planes;
}

__device__ __forceinline__ void read_tap_global(const fkb_chain_desc& ch, const PlaneRec& pl, int cx, int cy, float (&o)[3]) {
    const size_t X = static_cast<size_t>(cx) + pl.crop_x, Y = static_cast<size_t>(cy) + pl.crop_y;
    if (ch.src_format == FKB_PIX_NV12) {
        const uint8_t* uv = pl.src_chroma + (Y >> 1) * pl.src_pitch + (X >> 1) * 2;
        o[0] = static_cast<float>(__ldg(pl.src + Y * pl.src_pitch + X));
        o[1] = static_cast<float>(__ldg(uv));
        o[2] = static_cast<float>(__ldg(uv + 1));
    } else {
        const uint8_t* q = pl.src + Y * pl.src_pitch + X * 3;
        o[0] = static_cast<float>(__ldg(q));
        o[1] = static_cast<float>(__ldg(q + 1));
        o[2] = static_cast<float>(__ldg(q + 2));
    }
}

// ---------------------------------------------------------------------------------------------------------
// gather_kernel
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gather_kernel(const __grid_constant__ LaunchParams p) {
    __shared__ PlaneRec s_pl;
    const PlaneRec* table = plane_table(p);
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (uint32_t z = blockIdx.z; z < p.n_planes; z += gridDim.z) {
        __syncthreads();
        if (threadIdx.x < sizeof(PlaneRec) / 16)
            reinterpret_cast<uint4*>(&s_pl)[threadIdx.x] = reinterpret_cast<const uint4*>(table + z)[threadIdx.x];
        __syncthreads();
        const PlaneRec& pl = s_pl;
        if (pl.kclass != KCLASS_GATHER) continue;
        const fkb_chain_desc& ch = p.chains[pl.chain];
        const uint32_t y = blockIdx.y * 8 + ty;
        const uint32_t x0 = (blockIdx.x * 32 + tx) * 4;
        if (y >= pl.dst_h || x0 >= pl.dst_w) continue;
        const uint32_t nvalid = min(4u, pl.dst_w - x0);

        float v[4][3];
        if (ch.geometry == FKB_GEOM_NONE) {
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                if (n < nvalid) read_tap_global(ch, pl, x0 + n, y, v[n]);
                else { v[n][0] = v[n][1] = v[n][2] = 0.f; }
            }
            apply_ops<4>(v, ch, pl, 0, ch.n_ops);
        } else {
            const bool par = ch.geometry == FKB_GEOM_RESIZE_PRESERVE_AR;
            const int ox = par ? pl.x1 : 0, oy = par ? pl.y1 : 0;
            const bool row_in = !par || (static_cast<int>(y) >= pl.y1 && static_cast<int>(y) <= pl.y2);
            const AxisTap ay = axis_tap(row_in ? static_cast<int>(y) - oy : 0, pl.fy, pl.crop_h);
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const int x = static_cast<int>(x0) + n;
                const bool inside = n < nvalid && row_in && (!par || (x >= pl.x1 && x <= pl.x2));
                if (inside) {
                    const AxisTap ax = axis_tap(x - ox, pl.fx, pl.crop_w);
                    float t[4][3];
                    read_tap_global(ch, pl, ax.i0, ay.i0, t[0]);
                    read_tap_global(ch, pl, ax.i1, ay.i0, t[1]);
                    read_tap_global(ch, pl, ax.i0, ay.i1, t[2]);
                    read_tap_global(ch, pl, ax.i1, ay.i1, t[3]);
                    apply_ops<4>(t, ch, pl, 0, ch.n_pre_ops);
                    const float w00 = __fmul_rn(ax.w0, ay.w0), w10 = __fmul_rn(ax.w1, ay.w0);
                    const float w01 = __fmul_rn(ax.w0, ay.w1), w11 = __fmul_rn(ax.w1, ay.w1);
#pragma unroll
                    for (int c = 0; c < 3; ++c) v[n][c] = bilerp(t[0][c], t[1][c], t[2][c], t[3][c], w00, w10, w01, w11);
                } else {
                    v[n][0] = pl.bg[0]; v[n][1] = pl.bg[1]; v[n][2] = pl.bg[2];
                }
            }
            apply_ops<4>(v, ch, pl, ch.n_pre_ops, ch.n_ops);
        }

        uint8_t* row = pl.dst + static_cast<size_t>(y) * pl.dst_pitch;
        if (ch.write_kind == FKB_WRITE_SPLIT) {
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                uint8_t* q = row + static_cast<size_t>(c) * pl.dst_cstride;
                if (ch.dst_format == FKB_PIX_F32C3) {
                    float* f = reinterpret_cast<float*>(q) + x0;
                    if (nvalid == 4 && (reinterpret_cast<uintptr_t>(f) & 15) == 0) {
                        *reinterpret_cast<float4*>(f) = make_float4(v[0][c], v[1][c], v[2][c], v[3][c]);
                    } else {
                        for (uint32_t n = 0; n < nvalid; ++n) f[n] = v[n][c];
                    }
                } else {
                    for (uint32_t n = 0; n < nvalid; ++n) q[x0 + n] = static_cast<uint8_t>(v[n][c]);
                }
            }
        } else if (ch.dst_format == FKB_PIX_F32C3) {
            float* f = reinterpret_cast<float*>(row) + static_cast<size_t>(x0) * 3;
            if (nvalid == 4 && (reinterpret_cast<uintptr_t>(f) & 15) == 0) {
                float4* f4 = reinterpret_cast<float4*>(f);
                f4[0] = make_float4(v[0][0], v[0][1], v[0][2], v[1][0]);
                f4[1] = make_float4(v[1][1], v[1][2], v[2][0], v[2][1]);
                f4[2] = make_float4(v[2][2], v[3][0], v[3][1], v[3][2]);
            } else {
                for (uint32_t n = 0; n < nvalid; ++n) { f[3 * n] = v[n][0]; f[3 * n + 1] = v[n][1]; f[3 * n + 2] = v[n][2]; }
            }
        } else {
            uint8_t* q = row + static_cast<size_t>(x0) * 3;
            if (nvalid == 4 && (reinterpret_cast<uintptr_t>(q) & 3) == 0) {
                uint32_t b[12];
#pragma unroll
                for (int n = 0; n < 4; ++n)
#pragma unroll
                    for (int c = 0; c < 3; ++c) b[3 * n + c] = static_cast<uint32_t>(v[n][c]);
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
// staged_kernel
// ---------------------------------------------------------------------------------------------------------
struct TileInfo {
    uint32_t ox, oy, ow, oh;     // tile origin / extent in output pixels
    int32_t r_lo, c_lo;          // first staged source row / column, in crop coordinates
    uint32_t n_rows, row_bytes;  // staged rows and bytes per row
    uint32_t shift;              // byte offset of column c_lo inside a staged row
    uint32_t ok;                 // 0 when the footprint did not fit (lowering bug): tile is skipped, status set
    uint32_t pad_[2];
};

struct StagedSmem {
    uint64_t bar[2];
    TileInfo info[2];
    PlaneRec plane[2];
};
constexpr uint32_t kSmemHeader = 1024;
static_assert(sizeof(StagedSmem) <= kSmemHeader, "header region");

__device__ __forceinline__ uint32_t tile_to_plane(const LaunchParams& p, uint32_t t, uint32_t& local) {
    if (p.tiles_per_plane) { const uint32_t z = t / p.tiles_per_plane; local = t - z * p.tiles_per_plane; return z; }
    const PlaneRec* table = plane_table(p);
    uint32_t lo = 0, hi = p.n_planes;  // the last plane whose first tile is <= t (planes without tiles are skipped over)
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (table[mid].tile_base <= t) lo = mid; else hi = mid;
    }
    local = t - table[lo].tile_base;
    return lo;
}

// Warp 0 stages tile `t` into buffer `s`: copies the plane record, derives the source footprint, announces the
// byte count on the mbarrier and issues one bulk copy per footprint row.
__device__ __forceinline__ void produce_tile(const LaunchParams& p, uint32_t t, uint32_t s, StagedSmem& sm,
                                             uint8_t* in_buf, uint32_t lane) {
    uint32_t local;
    const uint32_t z = tile_to_plane(p, t, local);
    const PlaneRec* g = plane_table(p) + z;
    if (lane < sizeof(PlaneRec) / 16)
        reinterpret_cast<uint4*>(&sm.plane[s])[lane] = reinterpret_cast<const uint4*>(g)[lane];
    __syncwarp();
    const PlaneRec& pl = sm.plane[s];
    const fkb_chain_desc& ch = p.chains[pl.chain];
    const uint32_t tyi = local / pl.tiles_x, txi = local - tyi * pl.tiles_x;
    TileInfo ti;
    ti.ox = txi * pl.tile_w; ti.oy = tyi * pl.tile_h;
    ti.ow = min(pl.tile_w, pl.dst_w - ti.ox); ti.oh = min(pl.tile_h, pl.dst_h - ti.oy);
    int r_lo = 0, r_hi = -1, c_lo = 0, c_hi = -1;
    if (pl.kclass == KCLASS_POINT) {
        r_lo = ti.oy; r_hi = ti.oy + ti.oh - 1; c_lo = ti.ox; c_hi = ti.ox + ti.ow - 1;
    } else {
        const bool par = ch.geometry == FKB_GEOM_RESIZE_PRESERVE_AR;
        const int X1 = par ? pl.x1 : 0, Y1 = par ? pl.y1 : 0;
        const int X2 = par ? pl.x2 : static_cast<int>(pl.dst_w) - 1, Y2 = par ? pl.y2 : static_cast<int>(pl.dst_h) - 1;
        const int xa = max(static_cast<int>(ti.ox), X1), xb = min(static_cast<int>(ti.ox + ti.ow) - 1, X2);
        const int ya = max(static_cast<int>(ti.oy), Y1), yb = min(static_cast<int>(ti.oy + ti.oh) - 1, Y2);
        if (xa <= xb && ya <= yb) {
            c_lo = axis_tap(xa - X1, pl.fx, pl.crop_w).i0; c_hi = axis_tap(xb - X1, pl.fx, pl.crop_w).i1;
            r_lo = axis_tap(ya - Y1, pl.fy, pl.crop_h).i0; r_hi = axis_tap(yb - Y1, pl.fy, pl.crop_h).i1;
        }
    }
    ti.r_lo = r_lo; ti.c_lo = c_lo;
    ti.n_rows = r_hi >= r_lo ? static_cast<uint32_t>(r_hi - r_lo + 1) : 0u;
    const uint32_t g0 = (pl.crop_x + static_cast<uint32_t>(c_lo)) * 3u;
    const uint32_t g1 = (pl.crop_x + static_cast<uint32_t>(c_hi) + 1u) * 3u;
    const uint32_t a0 = g0 & ~15u;
    ti.shift = g0 - a0;
    ti.row_bytes = ti.n_rows ? ((g1 + 15u) & ~15u) - a0 : 0u;
    ti.ok = (ti.row_bytes <= pl.in_stride && static_cast<uint64_t>(ti.n_rows) * pl.in_stride <= kInBytes) ? 1u : 0u;
    if (!ti.ok) { ti.n_rows = 0; ti.row_bytes = 0; }
    if (lane == 0) {
        sm.info[s] = ti;
        mbar_arrive_expect_tx(&sm.bar[s], ti.n_rows * ti.row_bytes);
    }
    __syncwarp();
    const uint8_t* src0 = pl.src + static_cast<size_t>(pl.crop_y + r_lo) * pl.src_pitch + a0;
    for (uint32_t r = lane; r < ti.n_rows; r += 32)
        bulk_load(in_buf + static_cast<size_t>(r) * pl.in_stride, src0 + static_cast<size_t>(r) * pl.src_pitch, ti.row_bytes, &sm.bar[s]);
}

// --- POINT tiles ------------------------------------------------------------------------------------------
// uchar3 -> uchar3: 16 pixels (48 B) per thread step, three 128-bit shared loads and stores; thread chunks are
// 48 B apart, which maps the eight lanes of a quarter-warp onto disjoint bank groups.
__device__ __forceinline__ void point_tile_u8(const fkb_chain_desc& ch, const PlaneRec& pl, const TileInfo& ti,
                                              const uint8_t* in, uint8_t* out, uint32_t out_stride) {
    const uint32_t cpr = (ti.ow + 15) / 16, total = cpr * ti.oh;
    for (uint32_t c = threadIdx.x; c < total; c += blockDim.x) {
        const uint32_t ry = c / cpr, k = c - ry * cpr;
        const uint4* src = reinterpret_cast<const uint4*>(in + static_cast<size_t>(ry) * pl.in_stride + k * 48);
        uint32_t w[12];
#pragma unroll
        for (int i = 0; i < 3; ++i) { const uint4 q = src[i]; w[4 * i] = q.x; w[4 * i + 1] = q.y; w[4 * i + 2] = q.z; w[4 * i + 3] = q.w; }
        float v[16][3];
#pragma unroll
        for (int b = 0; b < 48; ++b) v[b / 3][b % 3] = static_cast<float>((w[b >> 2] >> (8 * (b & 3))) & 0xffu);
        apply_ops<16>(v, ch, pl, 0, ch.n_ops);
#pragma unroll
        for (int i = 0; i < 12; ++i) w[i] = 0;
#pragma unroll
        for (int b = 0; b < 48; ++b) w[b >> 2] |= static_cast<uint32_t>(v[b / 3][b % 3]) << (8 * (b & 3));
        uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(ry) * out_stride + k * 48);
#pragma unroll
        for (int i = 0; i < 3; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    }
}
// uchar3 -> float3: 4 pixels per thread step: three 32-bit shared loads (12 B apart: conflict-free), three
// 128-bit shared stores (48 B apart).
__device__ __forceinline__ void point_tile_f32(const fkb_chain_desc& ch, const PlaneRec& pl, const TileInfo& ti,
                                               const uint8_t* in, uint8_t* out, uint32_t out_stride) {
    const uint32_t cpr = (ti.ow + 3) / 4, total = cpr * ti.oh;
    for (uint32_t c = threadIdx.x; c < total; c += blockDim.x) {
        const uint32_t ry = c / cpr, k = c - ry * cpr;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(in + static_cast<size_t>(ry) * pl.in_stride + k * 12);
        const uint32_t w[3] = {src[0], src[1], src[2]};
        float v[4][3];
#pragma unroll
        for (int b = 0; b < 12; ++b) v[b / 3][b % 3] = static_cast<float>((w[b >> 2] >> (8 * (b & 3))) & 0xffu);
        apply_ops<4>(v, ch, pl, 0, ch.n_ops);
        float4* dst = reinterpret_cast<float4*>(out + static_cast<size_t>(ry) * out_stride + k * 48);
        dst[0] = make_float4(v[0][0], v[0][1], v[0][2], v[1][0]);
        dst[1] = make_float4(v[1][1], v[1][2], v[2][0], v[2][1]);
        dst[2] = make_float4(v[2][2], v[3][0], v[3][1], v[3][2]);
    }
}

// --- RESIZE tiles -----------------------------------------------------------------------------------------
// One warp per output row, lanes along x, four pixels per lane per step (so the op decode is amortised).
__device__ __forceinline__ void resize_tile(const fkb_chain_desc& ch, const PlaneRec& pl, const TileInfo& ti,
                                            const uint8_t* in, uint8_t* out, uint32_t out_stride) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const bool par = ch.geometry == FKB_GEOM_RESIZE_PRESERVE_AR;
    const int X1 = par ? pl.x1 : 0, Y1 = par ? pl.y1 : 0;
    const bool f32 = ch.dst_format == FKB_PIX_F32C3;
    for (uint32_t ry = warp; ry < ti.oh; ry += nwarps) {
        const int y = static_cast<int>(ti.oy + ry);
        const bool row_in = !par || (y >= pl.y1 && y <= pl.y2);
        const AxisTap ay = axis_tap(row_in ? y - Y1 : 0, pl.fy, pl.crop_h);
        const uint8_t* row0 = in + static_cast<size_t>(row_in ? ay.i0 - ti.r_lo : 0) * pl.in_stride + ti.shift;
        const uint8_t* row1 = in + static_cast<size_t>(row_in ? ay.i1 - ti.r_lo : 0) * pl.in_stride + ti.shift;
        uint8_t* orow = out + static_cast<size_t>(ry) * out_stride;
        for (uint32_t xb = 0; xb < ti.ow; xb += 128) {
            float v[4][3];
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const uint32_t lx = xb + lane + 32 * n;
                const int x = static_cast<int>(ti.ox + lx);
                const bool inside = lx < ti.ow && row_in && (!par || (x >= pl.x1 && x <= pl.x2));
                if (inside) {
                    const AxisTap ax = axis_tap(x - X1, pl.fx, pl.crop_w);
                    const uint32_t b0 = static_cast<uint32_t>(ax.i0 - ti.c_lo) * 3u, b1 = static_cast<uint32_t>(ax.i1 - ti.c_lo) * 3u;
                    const float w00 = __fmul_rn(ax.w0, ay.w0), w10 = __fmul_rn(ax.w1, ay.w0);
                    const float w01 = __fmul_rn(ax.w0, ay.w1), w11 = __fmul_rn(ax.w1, ay.w1);
#pragma unroll
                    for (int c = 0; c < 3; ++c)
                        v[n][c] = bilerp(static_cast<float>(row0[b0 + c]), static_cast<float>(row0[b1 + c]),
                                         static_cast<float>(row1[b0 + c]), static_cast<float>(row1[b1 + c]), w00, w10, w01, w11);
                } else {
                    v[n][0] = pl.bg[0]; v[n][1] = pl.bg[1]; v[n][2] = pl.bg[2];
                }
            }
            apply_ops<4>(v, ch, pl, ch.n_pre_ops, ch.n_ops);
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const uint32_t lx = xb + lane + 32 * n;
                if (lx < ti.ow) {
                    if (f32) {
                        float* q = reinterpret_cast<float*>(orow) + lx * 3;
                        q[0] = v[n][0]; q[1] = v[n][1]; q[2] = v[n][2];
                    } else {
                        uint8_t* q = orow + lx * 3;
                        q[0] = static_cast<uint8_t>(v[n][0]); q[1] = static_cast<uint8_t>(v[n][1]); q[2] = static_cast<uint8_t>(v[n][2]);
                    }
                }
            }
        }
    }
}

__global__ void __launch_bounds__(kStagedThreads, 2) staged_kernel(const __grid_constant__ LaunchParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    StagedSmem& sm = *reinterpret_cast<StagedSmem*>(smem_raw);
    uint8_t* in_buf[2] = {smem_raw + kSmemHeader, smem_raw + kSmemHeader + kInBytes};
    uint8_t* out_buf[2] = {smem_raw + kSmemHeader + 2 * kInBytes, smem_raw + kSmemHeader + 2 * kInBytes + kOutBytes};
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        mbar_init(&sm.bar[0], 1);
        mbar_init(&sm.bar[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0 && blockIdx.x < p.n_tiles) produce_tile(p, blockIdx.x, 0, sm, in_buf[0], lane);
    __syncthreads();

    bool failed = false;
    uint32_t it = 0;
    for (uint32_t t = blockIdx.x; t < p.n_tiles; t += gridDim.x, ++it) {
        const uint32_t s = it & 1;
        const uint32_t next = t + gridDim.x;
        if (warp == 0 && next < p.n_tiles) produce_tile(p, next, s ^ 1, sm, in_buf[s ^ 1], lane);

        const TileInfo ti = sm.info[s];
        const PlaneRec& pl = sm.plane[s];
        const fkb_chain_desc& ch = p.chains[pl.chain];
        const bool f32 = ch.dst_format == FKB_PIX_F32C3;
        const uint32_t elt = f32 ? 12u : 3u;
        const uint32_t out_stride = pl.out_stride;
        // everything the store phase needs is read here: after the barrier below warp 0 may already be
        // overwriting sm.plane / sm.info of the other buffer, and one iteration later this one
        const uint32_t dst_pitch = pl.dst_pitch;
        const uint32_t row_bytes = ti.ow * elt, bulk_bytes = row_bytes & ~15u, tail = row_bytes - bulk_bytes;
        uint8_t* const gdst = pl.dst + static_cast<size_t>(ti.oy) * dst_pitch + static_cast<size_t>(ti.ox) * elt;

        if (!mbar_wait_bounded(&sm.bar[s], (it >> 1) & 1)) failed = true;
        if (!ti.ok) failed = true;
        if (!failed) {
            if (pl.kclass == KCLASS_POINT) {
                if (f32) point_tile_f32(ch, pl, ti, in_buf[s], out_buf[s], out_stride);
                else point_tile_u8(ch, pl, ti, in_buf[s], out_buf[s], out_stride);
            } else {
                resize_tile(ch, pl, ti, in_buf[s], out_buf[s], out_stride);
            }
        }
        fence_async_smem();
        // the stores issued one iteration ago (from the other output buffer) must have been read out of shared
        // memory before anybody overwrites that buffer in the next iteration
        if (warp == 0) bulk_wait_read_all();
        if (__syncthreads_or(failed ? 1 : 0)) { failed = true; break; }

        if (warp == 0) {
            if (tail == 0 && row_bytes == out_stride && row_bytes == dst_pitch) {
                if (lane == 0) bulk_store(gdst, out_buf[s], row_bytes * ti.oh);  // the whole tile is one contiguous run
            } else if (bulk_bytes) {
                for (uint32_t r = lane; r < ti.oh; r += 32)
                    bulk_store(gdst + static_cast<size_t>(r) * dst_pitch, out_buf[s] + static_cast<size_t>(r) * out_stride, bulk_bytes);
            }
            bulk_commit();
        }
        if (tail) {  // the last (row_bytes mod 16) bytes of each row go out with plain stores
            for (uint32_t i = threadIdx.x; i < tail * ti.oh; i += blockDim.x) {
                const uint32_t r = i / tail, b = bulk_bytes + (i - r * tail);
                gdst[static_cast<size_t>(r) * dst_pitch + b] = out_buf[s][static_cast<size_t>(r) * out_stride + b];
            }
        }
    }
    if (warp == 0) bulk_wait_all();
    if (failed) {
        // give copies that are still in flight into shared memory a bounded chance to land before the CTA retires
        mbar_wait_bounded(&sm.bar[(it + 1) & 1], ((it + 1) >> 1) & 1);
        if (threadIdx.x == 0) atomicExch(p.status, FKB_ERR_DEVICE_WAIT);
    }
}

// ---------------------------------------------------------------------------------------------------------
// host-callable launchers (the only symbols the host translation unit needs from this file)
// ---------------------------------------------------------------------------------------------------------
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
    staged_kernel<<<grid, kStagedThreads, kStagedSmemBytes, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_gather(const LaunchParams& p, dim3 grid, cudaStream_t stream) {
    gather_kernel<<<grid, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

__device__ int g_status_word;

cudaError_t status_word_address(int** out) { return cudaGetSymbolAddress(reinterpret_cast<void**>(out), g_status_word); }

}  // namespace fkb
