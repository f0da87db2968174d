// Device-side building blocks of the sm_100a transform kernels: the lowered plane record, bulk-async-copy
// (TMA) and mbarrier wrappers with bounded waits, and the per-pixel op interpreter.
//
// Arithmetic contract (matches the FusedKernelLibrary CPU backend built without FMA contraction): every
// multiply/add/sub/div goes through an explicit round-to-nearest intrinsic, so no FMA is ever formed,
// division is IEEE, and SaturateCast is cvt.rni.sat.u8.f32 (round half to even, clamp, NaN -> 0), which is
// what core/constexpr_libs/constexpr_saturate.h:28-150 of the reference computes.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fkb/fkb.h"

namespace fkb {

enum : uint32_t { KCLASS_GATHER = 0, KCLASS_POINT = 1, KCLASS_RESIZE = 2, KCLASS_LUT = 3, KCLASS_NV12 = 4, KCLASS_GATHER4 = 5 };

// One output plane as the kernels see it: the caller's fkb_plane_desc plus what the host lowering derived
// (which kernel path runs it, its tile shape and its first tile index).
struct __align__(16) PlaneRec {
    const uint8_t* src;
    const uint8_t* src_chroma;
    uint8_t* dst;
    uint64_t dst_cstride;       // planar writes: byte offset of channel 1 from channel 0 ...
    uint64_t dst_cstride2;      // ... and of channel 2 (twice the former for a tensor; arbitrary for three separate planes)
    uint32_t src_pitch;
    uint32_t crop_x, crop_y;
    int32_t crop_w, crop_h;
    uint32_t dst_w, dst_h, dst_pitch;
    float fx, fy;
    int32_t x1, y1, x2, y2;
    float bg[3];
    uint32_t chain;
    uint32_t kclass;
    uint32_t tile_w, tile_h;    // output pixels per tile
    uint32_t tiles_x;           // column tiles per plane
    uint32_t tile_base;         // index of this plane's first staged tile in the launch (LUT planes: first LUT unit)
    uint32_t src_w, src_h;      // frame size in pixels (what a BorderReader maps coordinates into)
    float params[FKB_MAX_PLANE_PARAMS][3];
    uint32_t lut_base;          // LUT units of all earlier planes (monotone over the table, searched by lut_kernel)
    float bg_w;                 // four-channel chains: the fourth channel of bg and of the per-plane operands
    float params_w[FKB_MAX_PLANE_PARAMS];
    uint32_t all_background;    // a plane of a resampling chain whose every pixel is `bg` put through the ops behind the
                                // interpolation (a conditional batch read's plane beyond the used ones): no source is read
    uint32_t spare_[2];
};
static_assert(sizeof(PlaneRec) == 224, "layout is mirrored by the host lowering");
// byte offset of channel c of a planar destination
__host__ __device__ __forceinline__ uint64_t channel_offset(const PlaneRec& pl, int c) {
    return c == 0 ? 0ull : c == 1 ? pl.dst_cstride : pl.dst_cstride2;
}
static_assert(sizeof(PlaneRec) % 16 == 0, "PlaneRec is copied in 16-byte words");

constexpr uint32_t kInlinePlanes = 8;  // launches of up to this many planes carry their records in the kernel parameters

// Operands of a chain's specialised post-ops [Mul][Add|Sub][Div], resolved on the host when none of them is a per-plane
// operand (slots = 0); x - s is stored as x + (-s).
struct PostImm {
    float m[3], a[3], d[3];
    uint32_t slots;  // non-zero: some operand lives in the plane record, read it there instead
};

// Everything nv12_kernel needs to know about its chain, flattened so that every read has a fixed parameter offset.
struct Nv12Consts {
    float ccm[9], sub[3];
    float m[3], a[3], d[3];  // post-op operands (Mul, Add or negated Sub, Div)
    uint32_t kind;           // post-op shape bits
    uint32_t chain;          // the one chain whose planes take nv12_kernel
    uint32_t preserve_ar, f32, split, slots;
    uint32_t src_px;      // 0: NV12 / NV21 source (nv12 kernels); 3 or 4: bytes per pixel of a packed byte source (rgb_kernel)
    uint32_t vu;          // NV21: the chroma pairs are stored V,U
    uint32_t yuv_fmt;     // with src_px == 0: the FKB_PIX_* code of the YCbCr source (nv12_kernel reads all six; the pair kernel NV12 / NV21)
    uint32_t pair;        // nv12_pair_kernel's conditions hold (two pixels per thread, reduced colour matrix)
    uint32_t wide_store;  // with `pair`: destinations, pitches and channel strides are multiples of 8 bytes
    float kmag[3];        // with `pair`: 2^23 + sub[c], exact
};

// A four-channel chain flattened for rgba_kernel.  Mul, Add and Sub are each one fused multiply-add on every channel —
// x * m is fma(x, m, -0), x + a is fma(x, 1, a), x - a is fma(x, 1, -a): the same single rounding and the same signed
// zeros as the plain operation — so a chain of them needs no per-op decoding; Div and SaturateCast are the two other step
// kinds.  Channel reorders are folded into the operands' order and one final permutation, an appended alpha channel is
// fma(x, 0, alpha) on a channel that holds a finite value.
constexpr uint32_t kFourMaxSteps = 6;
struct FourConsts {
    uint32_t enabled;     // every four-channel plane of the launch runs this chain and meets rgba_kernel's conditions
    uint32_t n_steps;
    uint32_t kinds;       // two bits per step: 0 fused multiply-add, 1 division by m, 2 SaturateCast
    uint32_t perm;        // two bits per output channel: which stored channel it takes
    uint32_t src3;        // the source is uchar3 (the fourth channel starts as 0 and gets its value from an appended alpha)
    uint32_t f32;         // float4 destination (else uchar4)
    uint32_t resize, preserve_ar;
    float m[kFourMaxSteps][4], a[kFourMaxSteps][4];
};

struct LaunchParams {
    fkb_chain_desc chains[FKB_MAX_CHAINS];
    const PlaneRec* table;    // device table, or null when `inline_planes` is used
    uint32_t n_planes;
    uint32_t n_tiles;
    uint32_t n_split;         // the last n_split items of the staged kernel are dealt as two halves each (first rows, last rows):
                              // n_tiles + n_split item numbers in all; the launch then ends behind half an item, not a whole one
    uint32_t tiles_per_plane;  // > 0 when every plane has the same shape; else PlaneRec::tile_base is searched
    int* status;
    uint32_t* work;            // staged_kernel: {next item, warps finished} for dynamic item claiming; null = items dealt round-robin
    uint32_t n_lut_units;     // work units of lut_kernel (a block of rows of one LUT plane)
    uint32_t lut_swap;        // bit c: chain c contains an odd number of channel reorders
    uint32_t gather_z0, gather_z1;    // planes [z0, z1) hold every plane of the general kernel (grid.z covers this range only)
    uint32_t gather4_z0, gather4_z1;  // the same for the four-channel kernel
    uint32_t pixel_z0, pixel_z1;      // the same for the one-pixel-per-thread kernels (nv12_kernel, nv12_pair_kernel, rgb_kernel)
    uint32_t post_kind[FKB_MAX_CHAINS];
    PostImm post_imm[FKB_MAX_CHAINS];
    Nv12Consts nv12;  // per chain: bit mask of {Mul, Add|Sub, SaturateCast} when its post-ops have that shape, else 8
    FourConsts four;
    float neg_zero;           // -0.0f, deliberately opaque to the compiler (see mul2_unfusable)
    uint32_t test_extra_tx;   // 0 in every real launch; a test sets it so that staged_kernel's loads announce bytes that never
                              // arrive and its bounded waits run out (the FKB_ERR_DEVICE_WAIT path)
    uint32_t wait_limit_ns;   // how long a device-side wait for a bulk copy may last before the kernel gives up (one second)
    uint32_t pdl;             // host side only: launch the kernels with programmatic stream serialisation allowed
    PlaneRec inline_planes[kInlinePlanes];
};

static_assert(sizeof(LaunchParams) <= 8192, "kernel parameters (CUDA 12.1+ allows up to 32 764 bytes on sm_70 and later)");

// ---------------------------------------------------------------------------------------------------------
// shared-memory / mbarrier / bulk-copy wrappers
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Waits for a phase, but not for ever: gives up after `limit_ns` nanoseconds (LaunchParams::wait_limit_ns, one second in
// every real launch) or 2^26 polls, whichever comes first.  Returns false when it gave up (a lowering bug: the expected
// byte count never arrived); the caller records it in the status word and leaves without touching the data.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t round = 0; round < (1u << 20); ++round) {
        for (uint32_t i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > limit_ns) return false;
    }
    return false;
}
// global -> shared bulk copy (the TMA engine, no tensor map, no multicast); completion is signalled on `bar`.
// Both addresses and the size must be multiples of 16.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
// shared -> global bulk copy, tracked by the per-thread bulk group.
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(gmem_dst), "r"(smem_addr(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Programmatic dependent launch.  pdl_signal() lets the next kernel of the stream (if it was launched with programmatic
// stream serialisation allowed) be set up while this grid still runs; pdl_wait() returns once the grid before this one
// has completed and its writes are visible (at once when this launch has no such dependency).  Every kernel calls
// pdl_signal() first and pdl_wait() before it reads a source, writes a destination or touches a counter; plane records,
// which only the host writes, may be read ahead of it.
__device__ __forceinline__ void pdl_signal() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// make this thread's shared-memory writes visible to the async (bulk-copy) proxy
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------------
// the self-checking build (-DFKB_DEBUG)
// ---------------------------------------------------------------------------------------------------------
// Stands in for a memory checker where none can be run: every bulk copy's addresses, sizes and alignment and every
// gathered tap's coordinates are tested against the buffer the plane record describes before the access is made.  A
// failed test records FKB_ERR_DEVICE_CHECK in the status word and the access is skipped — nothing traps, nothing faults.
#ifdef FKB_DEBUG
constexpr bool kSelfChecking = true;
#else
constexpr bool kSelfChecking = false;
#endif
__device__ __forceinline__ bool self_check(int* status, bool good) {
    if (!good) atomicCAS(status, 0, FKB_ERR_DEVICE_CHECK);
    return good;
}
// [a, a + bytes) lies in [lo, lo + size), a and bytes are multiples of 16
__device__ __forceinline__ bool bulk_range_ok(const void* a, uint32_t bytes, const void* lo, size_t size) {
    const uintptr_t p = reinterpret_cast<uintptr_t>(a), l = reinterpret_cast<uintptr_t>(lo);
    return (p & 15u) == 0 && (bytes & 15u) == 0 && p >= l && p + bytes <= l + size;
}

// ---------------------------------------------------------------------------------------------------------
// the phase-clock build (-DFKB_PHASE_CLOCKS)
// ---------------------------------------------------------------------------------------------------------
// Shows where a warp of staged_kernel spends the cycles of a resize row: lane 0 reads the SM's cycle counter between
// the phases of the row loop and adds the differences up; at the end of an item it adds them to its warp's own slot of
// a device array (no atomics: a slot belongs to one warp), which fkb_debug_phase_clocks() sums and returns.  The reads
// keep the compiler from moving instructions across them, so this build runs slower than the product; what it gives is
// the split.  In the product build all of this compiles to nothing.
enum : int {
    kPhaseWait = 0,      // shuffles + waiting for the row's source rows to land (+ the claim and look-up of the next item on two rows)
    kPhaseCompute = 1,   // taps, arithmetic, stores into the row buffer, proxy fence, warp sync
    kPhaseStore = 2,     // issuing the bulk store(s) of the row
    kPhaseCommit = 3,    // closing the bulk group
    kPhaseLoads = 4,     // arrive.expect_tx + issuing the two bulk loads of a later row
    kPhaseWaitRead = 5,  // waiting until the previous row's store has read its buffer
    kPhaseRows = 6,      // rows processed (a count, not cycles)
    kPhaseTotal = 7,     // cycles of the whole item (set-up and row loop)
    kPhaseSetup = 8,     // an item's set-up: from its start (first loads requested) to the first row
    kPhaseFirstWait = 9, // waiting for the source rows of the item's first row inside the image (part of no other phase)
    kPhaseItems = 10,    // items processed (a count)
    kPhaseCount = 12
};
#ifdef FKB_PHASE_CLOCKS
constexpr bool kPhaseClocks = true;
#else
constexpr bool kPhaseClocks = false;
#endif
struct PhaseClock {
    long long t, acc[kPhaseCount];
    __device__ __forceinline__ PhaseClock() {
        if (kPhaseClocks) {
#pragma unroll
            for (int i = 0; i < kPhaseCount; ++i) acc[i] = 0;
            t = clock64();
        }
    }
    // the cycles since the previous call go to phase i
    __device__ __forceinline__ void lap(int i) {
        if (kPhaseClocks) { const long long n = clock64(); acc[i] += n - t; acc[kPhaseTotal] += n - t; t = n; }
    }
    __device__ __forceinline__ void count(int i) { if (kPhaseClocks) acc[i] += 1; }
};

// ---------------------------------------------------------------------------------------------------------
// arithmetic
// ---------------------------------------------------------------------------------------------------------
// Integer <-> float without conversion instructions (those run at a quarter of the FP32 rate).
// kMagic + n is exactly representable for every integer 0 <= n < 2^23 and its low mantissa bits are n.
constexpr float kMagic = 8388608.0f;  // 2^23
// float whose value is 2^23 + (byte `k` of w); sel = 0x7540 | k
__device__ __forceinline__ float magic_byte(uint32_t w, uint32_t sel) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, sel));
}
// exact float value of byte k of w
#define FKB_BYTE_F32(w, k) __fsub_rn(magic_byte((w), 0x7540u | (k)), kMagic)
// the 8-bit integer held exactly by a float in [0, 255]
__device__ __forceinline__ uint32_t u8_of_exact(float v) { return __float_as_uint(__fadd_rn(v, kMagic)) & 0xffu; }

// SaturateCast<float,uchar>: NaN -> 0, round half to even, clamp to [0,255].  Clamping first and then adding 2^23
// (which rounds to nearest-even at unit granularity) gives the same integer as rounding first and clamping after,
// which is what the reference does (core/constexpr_libs/constexpr_saturate.h:28-66, 97-117).
__device__ __forceinline__ float sat_u8_as_float(float v) {
    const float t = fminf(fmaxf(v, 0.f), 255.f);  // fmaxf returns the non-NaN operand
    return __fsub_rn(__fadd_rn(t, kMagic), kMagic);
}

// Two fp32 values per instruction (sm_100 f32x2 arithmetic): each lane is rounded to nearest on its own, so the
// results are bit-identical to two scalar operations at half the issue cost.
struct f2 { float x, y; };
#define FKB_F32X2_OP(name, opcode)                                                                              \
    __device__ __forceinline__ f2 name(f2 a, f2 b) {                                                            \
        f2 r;                                                                                                   \
        asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t" opcode            \
            " rc, ra, rb;\n\tmov.b64 {%0, %1}, rc;\n\t}"                                                         \
            : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));                                    \
        return r;                                                                                               \
    }
FKB_F32X2_OP(mul2, "mul.rn.f32x2")
FKB_F32X2_OP(add2, "add.rn.f32x2")
FKB_F32X2_OP(sub2, "sub.rn.f32x2")
#undef FKB_F32X2_OP
// ptxas contracts a packed multiply whose only use is a packed add into one fused multiply-add, even with explicit
// .rn modifiers and --fmad=false, which changes the rounding.  Products that feed additions are therefore written as
// fma(a, b, -0.0): adding -0.0 leaves every product (and the sign of a zero product) unchanged, and an FMA result
// cannot be contracted any further.  The -0.0 comes from a kernel parameter so that it is not folded away.
__device__ __forceinline__ f2 mul2_unfusable(f2 a, f2 b, float neg_zero) {
    f2 r;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %6};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(neg_zero));
    return r;
}

__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) {
    f2 r;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return r;
}

// Exact fp32 value b * 2^-24 of a byte b: the byte is read as the bit pattern of a subnormal half and widened, which
// runs on the FP pipe instead of the slow integer->float conversion unit.  Multiplying by a weight that was pre-scaled
// by 2^24 (exact) gives exactly the correctly rounded product b * w.
constexpr float kByteScale = 16777216.0f;  // 2^24
__device__ __forceinline__ float byte_times_2m24(uint32_t b) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(b)));
}

// Tap bytes read as fp32 subnormals (b * 2^-149) meet weights that carry 2^127; 2^22 is what is left to multiply by.
constexpr float kTapScale = 1.7014118346046923e38f;  // 2^127
constexpr float kTapUnscale = 4194304.0f;            // 2^22 = 2^149 / 2^127

// Runs ops[first..last) of `ch` on N pixels held in registers.  The op loop is outside the pixel loop so
// the (uniform) decode cost is paid once per N pixels.
template <int N>
__device__ __forceinline__ void apply_ops(float (&v)[N][3], const fkb_chain_desc& ch, const PlaneRec& pl,
                                          uint32_t first, uint32_t last) {
    for (uint32_t i = first; i < last; ++i) {
        const uint32_t code = ch.ops[i].code;
        const int slot = ch.ops[i].plane_slot;
        float p0, p1, p2;
        if (slot >= 0) { p0 = pl.params[slot][0]; p1 = pl.params[slot][1]; p2 = pl.params[slot][2]; }
        else { p0 = ch.ops[i].v[0]; p1 = ch.ops[i].v[1]; p2 = ch.ops[i].v[2]; }
        switch (code) {
        case FKB_OP_MUL:
            if (N % 2 == 0) {
                const float pp[3] = {p0, p1, p2};
#pragma unroll
                for (int n = 0; n + 1 < N; n += 2)
#pragma unroll
                    for (int c = 0; c < 3; ++c) { const f2 r = mul2(f2{v[n][c], v[n + 1][c]}, f2{pp[c], pp[c]}); v[n][c] = r.x; v[n + 1][c] = r.y; }
            } else {
#pragma unroll
                for (int n = 0; n < N; ++n) { v[n][0] = __fmul_rn(v[n][0], p0); v[n][1] = __fmul_rn(v[n][1], p1); v[n][2] = __fmul_rn(v[n][2], p2); }
            }
            break;
        case FKB_OP_ADD:
            if (N % 2 == 0) {
                const float pp[3] = {p0, p1, p2};
#pragma unroll
                for (int n = 0; n + 1 < N; n += 2)
#pragma unroll
                    for (int c = 0; c < 3; ++c) { const f2 r = add2(f2{v[n][c], v[n + 1][c]}, f2{pp[c], pp[c]}); v[n][c] = r.x; v[n + 1][c] = r.y; }
            } else {
#pragma unroll
                for (int n = 0; n < N; ++n) { v[n][0] = __fadd_rn(v[n][0], p0); v[n][1] = __fadd_rn(v[n][1], p1); v[n][2] = __fadd_rn(v[n][2], p2); }
            }
            break;
        case FKB_OP_SUB:
            if (N % 2 == 0) {
                const float pp[3] = {p0, p1, p2};
#pragma unroll
                for (int n = 0; n + 1 < N; n += 2)
#pragma unroll
                    for (int c = 0; c < 3; ++c) { const f2 r = sub2(f2{v[n][c], v[n + 1][c]}, f2{pp[c], pp[c]}); v[n][c] = r.x; v[n + 1][c] = r.y; }
            } else {
#pragma unroll
                for (int n = 0; n < N; ++n) { v[n][0] = __fsub_rn(v[n][0], p0); v[n][1] = __fsub_rn(v[n][1], p1); v[n][2] = __fsub_rn(v[n][2], p2); }
            }
            break;
        case FKB_OP_DIV:
#pragma unroll
            for (int n = 0; n < N; ++n) { v[n][0] = __fdiv_rn(v[n][0], p0); v[n][1] = __fdiv_rn(v[n][1], p1); v[n][2] = __fdiv_rn(v[n][2], p2); }
            break;
        case FKB_OP_REORDER_ZYX:
#pragma unroll
            for (int n = 0; n < N; ++n) { const float t = v[n][0]; v[n][0] = v[n][2]; v[n][2] = t; }
            break;
        case FKB_OP_YUV2RGB:
#pragma unroll
            for (int n = 0; n < N; ++n) {
                const float a = __fsub_rn(v[n][0], ch.yuv_sub[0]), b = __fsub_rn(v[n][1], ch.yuv_sub[1]), d = __fsub_rn(v[n][2], ch.yuv_sub[2]);
#pragma unroll
                for (int c = 0; c < 3; ++c)
                    v[n][c] = __fadd_rn(__fadd_rn(__fmul_rn(a, ch.ccm[3 * c]), __fmul_rn(b, ch.ccm[3 * c + 1])), __fmul_rn(d, ch.ccm[3 * c + 2]));
            }
            break;
        case FKB_OP_RGB2YUV:
#pragma unroll
            for (int n = 0; n < N; ++n) {
                const float r = v[n][0], g = v[n][1], b = v[n][2];
#pragma unroll
                for (int c = 0; c < 3; ++c) {
                    const float y = __fadd_rn(__fadd_rn(__fmul_rn(r, ch.ccm2[3 * c]), __fmul_rn(g, ch.ccm2[3 * c + 1])), __fmul_rn(b, ch.ccm2[3 * c + 2]));
                    v[n][c] = ch.yuv_add[c] != 0.f ? __fadd_rn(y, ch.yuv_add[c]) : y;  // full-range luma gets no offset at all
                }
            }
            break;
        case FKB_OP_SATCAST_U8:
#pragma unroll
            for (int n = 0; n < N; ++n) { v[n][0] = sat_u8_as_float(v[n][0]); v[n][1] = sat_u8_as_float(v[n][1]); v[n][2] = sat_u8_as_float(v[n][2]); }
            break;
        case FKB_OP_RGB2GRAY:  // (the later ops and the write use channel 0 only; the others keep running along unused)
#pragma unroll
            for (int n = 0; n < N; ++n) {
                const float l = __fadd_rn(__fadd_rn(__fmul_rn(v[n][0], 0.299f), __fmul_rn(v[n][1], 0.587f)), __fmul_rn(v[n][2], 0.114f));
                v[n][0] = rintf(l);  // nearest integer, ties to even, whatever the output type (see FKB_OP_RGB2GRAY in fkb.h)
            }
            break;
        default: break;  // FKB_OP_CAST_F32: values are already carried as fp32
        }
    }
}

// Bilinear weights and tap indices of one axis, exactly as InterpolateComplete<INTER_LINEAR>::exec
// (algorithms/image_processing/interpolation.h:70-104): floor, unclamped x2 = x1 + 1 for the weights, the
// read index clamped to the back operation's extent.
struct AxisTap {
    int i0, i1;    // clamped read indices
    float w0, w1;  // (x2 - s), (s - x1)
};
// No conversion instructions (they run at a quarter of the FP32 rate and sit on the critical path of every tap address):
// float(t) is 2^23 + t minus 2^23, floor(s) is the mantissa of s + 2^23 rounded toward minus infinity, and float(floor(s))
// is that sum minus 2^23 — all exact for 0 <= t and 0 <= s < 2^22, which the host's validation guarantees
// (fx * dst_w and fy * dst_h below 2^22).
__device__ __forceinline__ AxisTap axis_tap(int t, float f, int extent) {
    const float tf = __fsub_rn(__uint_as_float(0x4B000000u | static_cast<uint32_t>(t)), kMagic);
    const float s = __fmul_rn(tf, f);
    const float m = __fadd_rd(s, kMagic);                       // 2^23 + floor(s)
    const int a = static_cast<int>(__float_as_uint(m) & 0x7fffffu);
    const float af = __fsub_rn(m, kMagic);                      // float(a)
    AxisTap r;
    r.w0 = __fsub_rn(__fadd_rn(af, 1.0f), s);
    r.w1 = __fsub_rn(s, af);
    r.i0 = min(a, extent - 1);
    r.i1 = min(a + 1, extent - 1);
    return r;
}
__device__ __forceinline__ float bilerp(float p00, float p10, float p01, float p11, float w00, float w10, float w01, float w11) {
    return __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(p00, w00), __fmul_rn(p10, w10)), __fmul_rn(p01, w01)), __fmul_rn(p11, w11));
}

}  // namespace fkb
