// TEST INFRASTRUCTURE — not part of the product.  This translation unit contains no arithmetic of its own:
// it includes the FusedKernelLibrary headers from where they are installed (-I<reference>/include, see
// oracle/Makefile) and runs the reference's own CPU backend (TransformDPP<ParArch::CPU>,
// core/execution_model/data_parallel_patterns.h:246-284, executors.h:163-239) on caller-provided host
// buffers.  The result, oracle/_ref/libfkl_ref.so, pins oracle/fkb_oracle.cpp, produces the fixtures under
// tests/golden/ and is the timed CPU baseline.  Build flags: -O2 -ffp-contract=off, no -march=native.
//
// BATCH is a template parameter in the reference; a batch of n planes is run as independent calls of
// 32/16/8/4/2/1 planes (planes never interact), optionally spread over std::threads — the reference CPU
// backend itself is single-threaded.
#include <fused_kernel/algorithms/basic_ops/arithmetic.h>
#include <fused_kernel/algorithms/basic_ops/cast.h>
#include <fused_kernel/algorithms/basic_ops/memory_operations.h>
#include <fused_kernel/algorithms/image_processing/color_conversion.h>
#include <fused_kernel/algorithms/image_processing/border_reader.h>
#include <fused_kernel/algorithms/image_processing/crop.h>
#include <fused_kernel/algorithms/image_processing/image.h>
#include <fused_kernel/algorithms/image_processing/resize.h>
#include <fused_kernel/algorithms/image_processing/saturate.h>
#include <fused_kernel/fused_kernel.h>
#include <fused_kernel/core/data/circular_tensor.h>

#include <array>
#include <cstdint>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

using namespace fk;

namespace {

using CpuStream = Stream_<ParArch::CPU>;
using CpuDPP = TransformDPP<ParArch::CPU>;

struct Chunk { int first; int size; };

std::vector<Chunk> chunks_of(int n) {
    std::vector<Chunk> out;
    int at = 0;
    for (int s : {32, 16, 8, 4, 2, 1})
        while (n - at >= s) { out.push_back({at, s}); at += s; }
    return out;
}

void run_parallel(const std::vector<std::function<void()>>& jobs, int n_threads) {
    if (n_threads <= 1 || jobs.size() <= 1) { for (auto& j : jobs) j(); return; }
    const int T = std::min<int>(n_threads, static_cast<int>(jobs.size()));
    std::vector<std::thread> pool;
    for (int t = 0; t < T; ++t)
        pool.emplace_back([&, t] { for (size_t i = t; i < jobs.size(); i += T) jobs[i](); });
    for (auto& th : pool) th.join();
}

inline Ptr2D<uchar3> wrap_frame(const uint8_t* p, int w, int h, int pitch) {
    return Ptr2D<uchar3>(reinterpret_cast<uchar3*>(const_cast<uint8_t*>(p)), w, h, pitch, MemType::Host, 0);
}

struct BatchArgs {
    const uint8_t* const* frames; int w, h, pitch; const int32_t* rects; int dw, dh;
    float3 bg, mul, sub; uint8_t* out;
};

// Read -> Crop -> Resize(PRESERVE_AR, bg) -> Mul -> Sub -> SaturateCast -> TensorWrite<uchar3>
template <size_t B>
void crop_resize_u8(const BatchArgs& a, int first) {
    CpuStream stream;
    std::array<Ptr2D<uchar3>, B> ptrs; std::array<Rect, B> rects;
    for (size_t i = 0; i < B; ++i) {
        ptrs[i] = wrap_frame(a.frames[first + i], a.w, a.h, a.pitch);
        const int32_t* r = a.rects + 4 * (first + i);
        rects[i] = Rect(r[0], r[1], r[2], r[3]);
    }
    Tensor<uchar3> out(reinterpret_cast<uchar3*>(a.out) + static_cast<size_t>(first) * a.dw * a.dh, a.dw, a.dh, B, 1, MemType::Host, 0);
    executeOperations<CpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(ptrs), Crop<>::build(rects),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(Size(a.dw, a.dh), a.bg),
        Mul<float3>::build(a.mul), Sub<float3>::build(a.sub), SaturateCast<float3, uchar3>::build(),
        TensorWrite<uchar3>::build(out));
}

// Read -> Crop -> Resize(PRESERVE_AR, bg) -> Mul -> TensorWrite<float3>
template <size_t B>
void crop_resize_f32(const BatchArgs& a, int first) {
    CpuStream stream;
    std::array<Ptr2D<uchar3>, B> ptrs; std::array<Rect, B> rects;
    for (size_t i = 0; i < B; ++i) {
        ptrs[i] = wrap_frame(a.frames[first + i], a.w, a.h, a.pitch);
        const int32_t* r = a.rects + 4 * (first + i);
        rects[i] = Rect(r[0], r[1], r[2], r[3]);
    }
    Tensor<float3> out(reinterpret_cast<float3*>(a.out) + static_cast<size_t>(first) * a.dw * a.dh, a.dw, a.dh, B, 1, MemType::Host, 0);
    executeOperations<CpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(ptrs), Crop<>::build(rects),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(Size(a.dw, a.dh), a.bg),
        Mul<float3>::build(a.mul), TensorWrite<float3>::build(out));
}

// Read -> Crop -> ColorConversion<BGR2RGB> on uchar3 -> TensorWrite<uchar3>   (integer only; all rects cw x ch)
template <size_t B>
void crop_reorder_u8(const BatchArgs& a, int first) {
    CpuStream stream;
    std::array<Ptr2D<uchar3>, B> ptrs; std::array<Rect, B> rects;
    for (size_t i = 0; i < B; ++i) {
        ptrs[i] = wrap_frame(a.frames[first + i], a.w, a.h, a.pitch);
        const int32_t* r = a.rects + 4 * (first + i);
        rects[i] = Rect(r[0], r[1], r[2], r[3]);
    }
    Tensor<uchar3> out(reinterpret_cast<uchar3*>(a.out) + static_cast<size_t>(first) * a.dw * a.dh, a.dw, a.dh, B, 1, MemType::Host, 0);
    // a chain whose last ReadBack is followed by compute ops only is fused by hand with .then(), as the
    // reference's own crop tests do (tests/algorithm/test_crop.h:33-37)
    executeOperations<CpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(ptrs).then(Crop<>::build(rects)),
        ColorConversion<ColorConversionCodes::COLOR_BGR2RGB, uchar3, uchar3>::build(), TensorWrite<uchar3>::build(out));
}

#define FKLREF_DISPATCH(fn)                                                               \
    [](const BatchArgs& a, int n, int n_threads) {                                        \
        std::vector<std::function<void()>> jobs;                                          \
        for (const Chunk c : chunks_of(n)) {                                              \
            switch (c.size) {                                                             \
            case 32: jobs.push_back([&a, c] { fn<32>(a, c.first); }); break;              \
            case 16: jobs.push_back([&a, c] { fn<16>(a, c.first); }); break;              \
            case 8: jobs.push_back([&a, c] { fn<8>(a, c.first); }); break;                \
            case 4: jobs.push_back([&a, c] { fn<4>(a, c.first); }); break;                \
            case 2: jobs.push_back([&a, c] { fn<2>(a, c.first); }); break;                \
            default: jobs.push_back([&a, c] { fn<1>(a, c.first); }); break;               \
            }                                                                             \
        }                                                                                 \
        run_parallel(jobs, n_threads);                                                    \
    }

template <uint N> struct SelN { FK_HOST_DEVICE_FUSE uint at(const uint& z) { return z < N ? 0u : 1u; } };

// Divergent horizontal fusion over 2N planes of one size: planes [0,N) Resize(IGNORE_AR) -> SaturateCast ->
// TensorWrite<uchar3>; planes [N,2N) Cast -> Mul(scale_i) -> Sub(off_i) fused into each plane's Read ->
// TensorWrite<float3> into a 2N-plane tensor addressed by the global plane index.
template <uint N>
void divergent(const uint8_t* const* frames, int w, int h, int pitch, int dw, int dh, const float* scales,
               const float* offs, uint8_t* outA, float* outB) {
    CpuStream stream;
    std::array<Ptr2D<uchar3>, N> firstN;
    for (uint i = 0; i < N; ++i) firstN[i] = wrap_frame(frames[i], w, h, pitch);
    Tensor<uchar3> tA(reinterpret_cast<uchar3*>(outA), dw, dh, N, 1, MemType::Host, 0);
    const auto seq0 = buildOperationSequence(PerThreadRead<ND::_2D, uchar3>::build(firstN),
        Resize<InterpolationType::INTER_LINEAR>::build(Size(dw, dh)), SaturateCast<float3, uchar3>::build(),
        TensorWrite<uchar3>::build(tA));
    const Ptr2D<uchar3> f0 = wrap_frame(frames[N], w, h, pitch);
    using FusedRead = decltype(PerThreadRead<ND::_2D, uchar3>::build(f0).then(Cast<uchar3, float3>::build())
        .then(Mul<float3>::build(make_set<float3>(1.f))).then(Sub<float3>::build(make_set<float3>(0.f))));
    std::array<FusedRead, 2 * N> reads;
    for (uint i = 0; i < 2 * N; ++i) {
        const uint k = i < N ? 0 : i - N;
        reads[i] = PerThreadRead<ND::_2D, uchar3>::build(wrap_frame(frames[N + k], w, h, pitch))
            .then(Cast<uchar3, float3>::build()).then(Mul<float3>::build(make_set<float3>(scales[k])))
            .then(Sub<float3>::build(make_set<float3>(offs[k])));
    }
    auto batchRead = BatchRead<PlanePolicy::PROCESS_ALL>::build(reads);
    batchRead.params.activeThreads.z = N;  // this sequence owns N planes; indices stay global
    Tensor<float3> tB(reinterpret_cast<float3*>(outB), w, h, 2 * N, 1, MemType::Host, 0);
    const auto seq1 = buildOperationSequence(batchRead, TensorWrite<float3>::build(tB));
    Executor<DivergentBatchTransformDPP<ParArch::CPU, SelN<N>>>::executeOperations(stream, seq0, seq1);
}

}  // namespace

template <AspectRatio AR, typename Read>
static void letterbox_params(const Read& read, int dw, int dh, float* f2, int32_t* r4) {
    const auto r = Resize<InterpolationType::INTER_LINEAR, AR, float3>::build(read, Size(dw, dh), make_<float3>(0.f, 0.f, 0.f));
    f2[0] = r.params.src_conv_factors.x; f2[1] = r.params.src_conv_factors.y;
    r4[0] = r.params.x1; r4[1] = r.params.y1; r4[2] = r.params.x2; r4[3] = r.params.y2;
}

// Four uchar4 frames -> Crop -> Resize(IGNORE_AR) on float4 -> ColorConversion<BGRA2BGR | BGRA2RGB, float4, float3> ->
// Mul<float3> -> TensorWrite<float3>: the alpha channel is discarded after the interpolation.
template <ColorConversionCodes CODE>
static int bgra_crop_resize(const uint8_t* const* frames, int w, int h, int pitch, const int32_t* rects, int dw, int dh, const float* mul, float* out) {
    CpuStream stream;
    std::array<Ptr2D<uchar4>, 4> ptrs; std::array<Rect, 4> rs;
    for (size_t i = 0; i < 4; ++i) {
        ptrs[i] = Ptr2D<uchar4>(reinterpret_cast<uchar4*>(const_cast<uint8_t*>(frames[i])), w, h, pitch, MemType::Host, 0);
        rs[i] = Rect(rects[4 * i], rects[4 * i + 1], rects[4 * i + 2], rects[4 * i + 3]);
    }
    Tensor<float3> t(reinterpret_cast<float3*>(out), dw, dh, 4, 1, MemType::Host, 0);
    executeOperations<CpuDPP>(stream, PerThreadRead<ND::_2D, uchar4>::build(ptrs), Crop<>::build(rs),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(dw, dh)), ColorConversion<CODE, float4, float3>::build(),
        Mul<float3>::build(make_<float3>(mul[0], mul[1], mul[2])), TensorWrite<float3>::build(t));
    return 0;
}

// CircularTensor<float, 3, 4, ORDER, MODE>::update (core/data/circular_tensor.h:111-161), n_updates times: frame k ->
// Resize(IGNORE_AR) -> Mul -> write into the circular tensor.  kind: 0 TensorWrite<float3> (Standard, packed float3 planes),
// 1 TensorSplit<float3> (Standard, planar), 2 TensorTSplit<float3> (Transposed).  The tensor's bytes after the last update
// are copied to `out`.
template <CircularTensorOrder ORDER>
static int circular_updates(const uint8_t* const* frames, int n_updates, int w, int h, int pitch, int dw, int dh, const float* mul, int kind, void* out) {
    CpuStream stream;
    const auto resize = Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(dw, dh));
    const auto m = Mul<float3>::build(make_<float3>(mul[0], mul[1], mul[2]));
    if (kind == 0) {
        CircularTensor<float3, 1, 4, ORDER, ColorPlanes::Standard> ct(dw, dh, MemType::Host, 0);
        std::memset(ct.ptr().data, 0, ct.sizeInBytes());
        for (int k = 0; k < n_updates; ++k)
            ct.update(stream, PerThreadRead<ND::_2D, uchar3>::build(wrap_frame(frames[k], w, h, pitch)), resize, m, TensorWrite<float3>::build(ct.ptr()));
        std::memcpy(out, ct.ptr().data, ct.sizeInBytes());
    } else if (kind == 1) {
        CircularTensor<float, 3, 4, ORDER, ColorPlanes::Standard> ct(dw, dh, MemType::Host, 0);
        std::memset(ct.ptr().data, 0, ct.sizeInBytes());
        for (int k = 0; k < n_updates; ++k)
            ct.update(stream, PerThreadRead<ND::_2D, uchar3>::build(wrap_frame(frames[k], w, h, pitch)), resize, m, TensorSplit<float3>::build(ct.ptr()));
        std::memcpy(out, ct.ptr().data, ct.sizeInBytes());
    } else {
        CircularTensor<float, 3, 4, ORDER, ColorPlanes::Transposed> ct(dw, dh, MemType::Host, 0);
        std::memset(ct.ptr().data, 0, ct.sizeInBytes());
        for (int k = 0; k < n_updates; ++k)
            ct.update(stream, PerThreadRead<ND::_2D, uchar3>::build(wrap_frame(frames[k], w, h, pitch)), resize, m, TensorTSplit<float3>::build(ct.ptr()));
        std::memcpy(out, ct.ptr().data, ct.sizeInBytes());
    }
    return 0;
}
extern "C" int fklref_circular_updates(const uint8_t* const* frames, int n_updates, int w, int h, int pitch, int dw, int dh, const float* mul,
                                       int kind, int oldest_first, void* out) {
    return oldest_first ? circular_updates<CircularTensorOrder::OldestFirst>(frames, n_updates, w, h, pitch, dw, dh, mul, kind, out)
                        : circular_updates<CircularTensorOrder::NewestFirst>(frames, n_updates, w, h, pitch, dw, dh, mul, kind, out);
}

extern "C" {

int fklref_crop_resize_u8(const uint8_t* const* frames, int w, int h, int pitch, const int32_t* rects, int n,
                          int dw, int dh, const float* bg, const float* mul, const float* sub, uint8_t* out,
                          int n_threads) {
    const BatchArgs a{frames, w, h, pitch, rects, dw, dh, make_<float3>(bg[0], bg[1], bg[2]),
                      make_<float3>(mul[0], mul[1], mul[2]), make_<float3>(sub[0], sub[1], sub[2]), out};
    FKLREF_DISPATCH(crop_resize_u8)(a, n, n_threads);
    return 0;
}

int fklref_crop_resize_f32(const uint8_t* const* frames, int w, int h, int pitch, const int32_t* rects, int n,
                           int dw, int dh, const float* bg, const float* mul, float* out, int n_threads) {
    const BatchArgs a{frames, w, h, pitch, rects, dw, dh, make_<float3>(bg[0], bg[1], bg[2]),
                      make_<float3>(mul[0], mul[1], mul[2]), make_<float3>(0.f, 0.f, 0.f),
                      reinterpret_cast<uint8_t*>(out)};
    FKLREF_DISPATCH(crop_resize_f32)(a, n, n_threads);
    return 0;
}

int fklref_crop_reorder_u8(const uint8_t* const* frames, int w, int h, int pitch, const int32_t* rects, int n,
                           uint8_t* out, int n_threads) {
    const BatchArgs a{frames, w, h, pitch, rects, rects[2], rects[3], make_<float3>(0.f, 0.f, 0.f),
                      make_<float3>(0.f, 0.f, 0.f), make_<float3>(0.f, 0.f, 0.f), out};
    FKLREF_DISPATCH(crop_reorder_u8)(a, n, n_threads);
    return 0;
}

// BatchRead<CONDITIONAL_WITH_DEFAULT> (batch_operations.h:221-281): eight planes of which the first `used` are read;
// the others yield `dflt`.  Two chains: with a Resize (the default value passes through the fused ReadBack as its
// float3 cast, then Mul), and without (Cast -> Mul -> SaturateCast on the uchar3 default).
int fklref_conditional_resize_f32(const uint8_t* const* frames, int w, int h, int pitch, int used, const uint8_t* dflt,
                                  int dw, int dh, const float* mul, float* out) {
    CpuStream stream;
    std::array<Ptr2D<uchar3>, 8> ptrs;
    for (size_t i = 0; i < 8; ++i) ptrs[i] = wrap_frame(frames[i], w, h, pitch);
    Tensor<float3> t(reinterpret_cast<float3*>(out), dw, dh, 8, 1, MemType::Host, 0);
    executeOperations<CpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(used, make_<uchar3>(dflt[0], dflt[1], dflt[2]), ptrs),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(dw, dh)),
        Mul<float3>::build(make_<float3>(mul[0], mul[1], mul[2])), TensorWrite<float3>::build(t));
    return 0;
}
int fklref_conditional_pointwise_u8(const uint8_t* const* frames, int w, int h, int pitch, int used, const uint8_t* dflt,
                                    const float* mul, uint8_t* out) {
    CpuStream stream;
    std::array<Ptr2D<uchar3>, 8> ptrs;
    for (size_t i = 0; i < 8; ++i) ptrs[i] = wrap_frame(frames[i], w, h, pitch);
    Tensor<uchar3> t(reinterpret_cast<uchar3*>(out), w, h, 8, 1, MemType::Host, 0);
    executeOperations<CpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(used, make_<uchar3>(dflt[0], dflt[1], dflt[2]), ptrs),
        Cast<uchar3, float3>::build(), Mul<float3>::build(make_<float3>(mul[0], mul[1], mul[2])),
        SaturateCast<float3, uchar3>::build(), TensorWrite<uchar3>::build(t));
    return 0;
}

// One frame -> Resize(IGNORE_AR) -> Mul [-> SaturateCast] -> SplitWrite<_2D, float3|uchar3> into three separate planes
int fklref_resize_split_planes(const uint8_t* frame, int w, int h, int pitch, int dw, int dh, const float* mul, int f32, void* px, void* py,
                               void* pz, int dpitch) {
    CpuStream stream;
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(wrap_frame(frame, w, h, pitch));
    const auto resize = Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(dw, dh));
    const auto m = Mul<float3>::build(make_<float3>(mul[0], mul[1], mul[2]));
    if (f32) {
        const std::vector<Ptr2D<float>> out{Ptr2D<float>(static_cast<float*>(px), dw, dh, dpitch, MemType::Host, 0),
                                            Ptr2D<float>(static_cast<float*>(py), dw, dh, dpitch, MemType::Host, 0),
                                            Ptr2D<float>(static_cast<float*>(pz), dw, dh, dpitch, MemType::Host, 0)};
        executeOperations<CpuDPP>(stream, read, resize, m, SplitWrite<ND::_2D, float3>::build(out));
    } else {
        const std::vector<Ptr2D<uchar>> out{Ptr2D<uchar>(static_cast<uchar*>(px), dw, dh, dpitch, MemType::Host, 0),
                                            Ptr2D<uchar>(static_cast<uchar*>(py), dw, dh, dpitch, MemType::Host, 0),
                                            Ptr2D<uchar>(static_cast<uchar*>(pz), dw, dh, dpitch, MemType::Host, 0)};
        executeOperations<CpuDPP>(stream, read, resize, m, SaturateCast<float3, uchar3>::build(), SplitWrite<ND::_2D, uchar3>::build(out));
    }
    return 0;
}

int fklref_bgra_crop_resize_f32(const uint8_t* const* frames, int w, int h, int pitch, const int32_t* rects, int dw, int dh, const float* mul,
                                int swap, float* out) {
    return swap ? bgra_crop_resize<ColorConversionCodes::COLOR_BGRA2RGB>(frames, w, h, pitch, rects, dw, dh, mul, out)
                : bgra_crop_resize<ColorConversionCodes::COLOR_BGRA2BGR>(frames, w, h, pitch, rects, dw, dh, mul, out);
}

// The four-channel pipeline of tests/examples/compiler_explorer_example.h:23-46 on one uchar4 frame and five crops:
// Crop -> Resize -> Mul x2 -> Add -> Mul -> [BGRA2RGBA] -> SaturateCast -> TensorWrite<uchar4>, or without the SaturateCast into
// a float4 tensor.
int fklref_rgba_crops(const uint8_t* frame, int w, int h, int pitch, const int32_t* rects, int dw, int dh, const float* m1, const float* a1,
                      int reorder, int f32, void* out) {
    CpuStream stream;
    const Ptr2D<uchar4> input(reinterpret_cast<uchar4*>(const_cast<uint8_t*>(frame)), w, h, pitch, MemType::Host, 0);
    std::array<Rect, 5> rs;
    for (size_t i = 0; i < 5; ++i) rs[i] = Rect(rects[4 * i], rects[4 * i + 1], rects[4 * i + 2], rects[4 * i + 3]);
    const auto read = PerThreadRead<ND::_2D, uchar4>::build(input);
    const auto crop = Crop<>::build(rs);
    const auto resize = Resize<InterpolationType::INTER_LINEAR>::build(Size(dw, dh));
    const auto mul = Mul<float4>::build(make_<float4>(m1[0], m1[1], m1[2], m1[3]));
    const auto add = Add<float4>::build(make_<float4>(a1[0], a1[1], a1[2], a1[3]));
    const auto mul255 = Mul<float4>::build(make_set<float4>(255.f));
    if (f32) {
        Tensor<float4> t(static_cast<float4*>(out), dw, dh, 5, 1, MemType::Host, 0);
        if (reorder) executeOperations<CpuDPP>(stream, read, crop, resize, mul, add, ColorConversion<ColorConversionCodes::COLOR_BGRA2RGBA, float4, float4>::build(), TensorWrite<float4>::build(t));
        else executeOperations<CpuDPP>(stream, read, crop, resize, mul, add, TensorWrite<float4>::build(t));
    } else {
        Tensor<uchar4> t(static_cast<uchar4*>(out), dw, dh, 5, 1, MemType::Host, 0);
        if (reorder) executeOperations<CpuDPP>(stream, read, crop, resize, mul, add, mul255, ColorConversion<ColorConversionCodes::COLOR_BGRA2RGBA, float4, float4>::build(),
                                               SaturateCast<float4, uchar4>::build(), TensorWrite<uchar4>::build(t));
        else executeOperations<CpuDPP>(stream, read, crop, resize, mul, add, mul255, SaturateCast<float4, uchar4>::build(), TensorWrite<uchar4>::build(t));
    }
    return 0;
}

// Conversions that append an opaque alpha channel.  One uchar3 frame, five crops -> Crop -> Resize -> Mul<float3> ->
// ColorConversion<COLOR_BGR2BGRA | COLOR_BGR2RGBA, float3, float4> (alpha = 255) -> Mul<float4> ->
// [SaturateCast<float4,uchar4> -> TensorWrite<uchar4> | TensorWrite<float4>].
int fklref_add_alpha_crops(const uint8_t* frame, int w, int h, int pitch, const int32_t* rects, int dw, int dh, const float* m3, const float* m4,
                           int swap, int f32, void* out) {
    CpuStream stream;
    std::array<Rect, 5> rs;
    for (size_t i = 0; i < 5; ++i) rs[i] = Rect(rects[4 * i], rects[4 * i + 1], rects[4 * i + 2], rects[4 * i + 3]);
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(wrap_frame(frame, w, h, pitch));
    const auto crop = Crop<>::build(rs);
    const auto resize = Resize<InterpolationType::INTER_LINEAR>::build(Size(dw, dh));
    const auto mul3 = Mul<float3>::build(make_<float3>(m3[0], m3[1], m3[2]));
    const auto mul4 = Mul<float4>::build(make_<float4>(m4[0], m4[1], m4[2], m4[3]));
    const auto keep = ColorConversion<ColorConversionCodes::COLOR_BGR2BGRA, float3, float4>::build();
    const auto flip = ColorConversion<ColorConversionCodes::COLOR_BGR2RGBA, float3, float4>::build();
    if (f32) {
        Tensor<float4> t(static_cast<float4*>(out), dw, dh, 5, 1, MemType::Host, 0);
        if (swap) executeOperations<CpuDPP>(stream, read, crop, resize, mul3, flip, mul4, TensorWrite<float4>::build(t));
        else executeOperations<CpuDPP>(stream, read, crop, resize, mul3, keep, mul4, TensorWrite<float4>::build(t));
    } else {
        Tensor<uchar4> t(static_cast<uchar4*>(out), dw, dh, 5, 1, MemType::Host, 0);
        if (swap) executeOperations<CpuDPP>(stream, read, crop, resize, mul3, flip, mul4, SaturateCast<float4, uchar4>::build(), TensorWrite<uchar4>::build(t));
        else executeOperations<CpuDPP>(stream, read, crop, resize, mul3, keep, mul4, SaturateCast<float4, uchar4>::build(), TensorWrite<uchar4>::build(t));
    }
    return 0;
}
// PerThreadRead<uchar3> -> ColorConversion<COLOR_BGR2BGRA | COLOR_BGR2RGBA, uchar3, uchar4> -> PerThreadWrite<uchar4>
int fklref_add_alpha_image(const uint8_t* frame, int w, int h, int pitch, int swap, uint8_t* out, int opitch) {
    CpuStream stream;
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(wrap_frame(frame, w, h, pitch));
    const Ptr2D<uchar4> o(reinterpret_cast<uchar4*>(out), w, h, opitch, MemType::Host, 0);
    if (swap) executeOperations<CpuDPP>(stream, read, ColorConversion<ColorConversionCodes::COLOR_BGR2RGBA, uchar3, uchar4>::build(), PerThreadWrite<ND::_2D, uchar4>::build(o));
    else executeOperations<CpuDPP>(stream, read, ColorConversion<ColorConversionCodes::COLOR_BGR2BGRA, uchar3, uchar4>::build(), PerThreadWrite<ND::_2D, uchar4>::build(o));
    return 0;
}

}  // extern "C"
// PerThreadRead<uchar3 | uchar4> -> ColorConversion<COLOR_{RGB,BGR,RGBA,BGRA}2GRAY, I, uchar> -> PerThreadWrite<uchar>
template <ColorConversionCodes CODE, typename I>
static int gray_image(const uint8_t* frame, int w, int h, int pitch, uint8_t* out, int opitch) {
    CpuStream stream;
    const Ptr2D<I> in(reinterpret_cast<I*>(const_cast<uint8_t*>(frame)), w, h, pitch, MemType::Host, 0);
    const Ptr2D<uchar> o(reinterpret_cast<uchar*>(out), w, h, opitch, MemType::Host, 0);
    executeOperations<CpuDPP>(stream, PerThreadRead<ND::_2D, I>::build(in), ColorConversion<CODE, I, uchar>::build(), PerThreadWrite<ND::_2D, uchar>::build(o));
    return 0;
}
extern "C" int fklref_gray_image(const uint8_t* frame, int w, int h, int pitch, int bgr, int src4, uint8_t* out, int opitch) {
    if (src4) return bgr ? gray_image<ColorConversionCodes::COLOR_BGRA2GRAY, uchar4>(frame, w, h, pitch, out, opitch)
                         : gray_image<ColorConversionCodes::COLOR_RGBA2GRAY, uchar4>(frame, w, h, pitch, out, opitch);
    return bgr ? gray_image<ColorConversionCodes::COLOR_BGR2GRAY, uchar3>(frame, w, h, pitch, out, opitch)
               : gray_image<ColorConversionCodes::COLOR_RGB2GRAY, uchar3>(frame, w, h, pitch, out, opitch);
}
// Five crops of one frame -> Resize(IGNORE_AR) -> ColorConversion<COLOR_RGB2GRAY | COLOR_BGR2GRAY, float3, float> -> Mul<float>
// -> [SaturateCast<float, uchar> -> TensorWrite<uchar> | TensorWrite<float>]
template <ColorConversionCodes CODE>
static int gray_crops(const uint8_t* frame, int w, int h, int pitch, const int32_t* rects, int dw, int dh, float mul, int f32, void* out) {
    CpuStream stream;
    constexpr size_t B = 5;
    std::array<Rect, B> crops;
    for (size_t i = 0; i < B; ++i) crops[i] = Rect(rects[4 * i], rects[4 * i + 1], rects[4 * i + 2], rects[4 * i + 3]);
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(wrap_frame(frame, w, h, pitch));
    const auto crop = Crop<>::build(crops);
    const auto resize = Resize<InterpolationType::INTER_LINEAR>::build(Size(dw, dh));
    const auto gray = ColorConversion<CODE, float3, float>::build();
    const auto scale = Mul<float>::build(mul);
    if (f32) {
        const Tensor<float> t(static_cast<float*>(out), dw, dh, B, 1, MemType::Host, 0);
        executeOperations<CpuDPP>(stream, read, crop, resize, gray, scale, TensorWrite<float>::build(t));
    } else {
        const Tensor<uchar> t(static_cast<uchar*>(out), dw, dh, B, 1, MemType::Host, 0);
        executeOperations<CpuDPP>(stream, read, crop, resize, gray, scale, SaturateCast<float, uchar>::build(), TensorWrite<uchar>::build(t));
    }
    return 0;
}
extern "C" int fklref_gray_crops(const uint8_t* frame, int w, int h, int pitch, const int32_t* rects, int dw, int dh, float mul, int bgr, int f32, void* out) {
    return bgr ? gray_crops<ColorConversionCodes::COLOR_BGR2GRAY>(frame, w, h, pitch, rects, dw, dh, mul, f32, out)
               : gray_crops<ColorConversionCodes::COLOR_RGB2GRAY>(frame, w, h, pitch, rects, dw, dh, mul, f32, out);
}
extern "C" {

// Four frames -> Resize(IGNORE_AR) -> Mul -> TensorTSplit<float3> into a colour-plane-transposed tensor
// (memory_operations.h:214-241): all R planes, then all G planes, then all B planes.
int fklref_resize_tsplit_f32(const uint8_t* const* frames, int w, int h, int pitch, int dw, int dh, const float* mul, float* out) {
    CpuStream stream;
    std::array<Ptr2D<uchar3>, 4> ptrs;
    for (size_t i = 0; i < 4; ++i) ptrs[i] = wrap_frame(frames[i], w, h, pitch);
    // (the reference's TensorT constructor that wraps caller memory leaves the three pitches at zero; they are set here
    // the way its allocating constructor sets them, ptr_nd.h:119-125)
    PtrDims<ND::T3D> dims(dw, dh, 4, 3);
    dims.pitch = sizeof(float) * dw; dims.plane_pitch = dims.pitch * dh; dims.color_planes_pitch = dims.plane_pitch * 4;
    const RawPtr<ND::T3D, float> t{out, dims};
    executeOperations<CpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(ptrs),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(dw, dh)),
        Mul<float3>::build(make_<float3>(mul[0], mul[1], mul[2])), TensorTSplit<float3>::build(t));
    return 0;
}

// Read -> Cast -> Mul -> Add -> Div -> ColorConversion<BGR2RGB> -> SaturateCast -> PerThreadWrite
int fklref_pointwise_u8(const uint8_t* src, int w, int h, int spitch, const float* mul, const float* add,
                        const float* div, uint8_t* dst, int dpitch) {
    CpuStream stream;
    const Ptr2D<uchar3> in = wrap_frame(src, w, h, spitch);
    const Ptr2D<uchar3> out = wrap_frame(dst, w, h, dpitch);
    executeOperations<CpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(in), Cast<uchar3, float3>::build(),
        Mul<float3>::build(make_<float3>(mul[0], mul[1], mul[2])),
        Add<float3>::build(make_<float3>(add[0], add[1], add[2])),
        Div<float3>::build(make_<float3>(div[0], div[1], div[2])),
        ColorConversion<ColorConversionCodes::COLOR_BGR2RGB, float3, float3>::build(),
        SaturateCast<float3, uchar3>::build(), PerThreadWrite<ND::_2D, uchar3>::build(out));
    return 0;
}

// ReadYUV<NV12> -> ConvertYUVToRGB<p8bit,Full,bt709> -> Resize(IGNORE_AR) -> Sub -> Div -> TensorSplit<float3>
int fklref_nv12_resize_split(const uint8_t* nv12, int w, int h, int pitch, int dw, int dh, const float* sub,
                             const float* div, float* out) {
    CpuStream stream;
    const Ptr<ND::_2D, uchar> data(const_cast<uint8_t*>(nv12), PtrDims<ND::_2D>(w, h + h / 2, pitch), MemType::Host, 0);
    const Image<PixelFormat::NV12> img(data, w, h);
    Tensor<float> t(out, dw, dh, 1, 3, MemType::Host, 0);
    executeOperations<CpuDPP>(stream, ReadYUV<PixelFormat::NV12>::build(img),
        ConvertYUVToRGB<ColorDepth::p8bit, ColorRange::Full, ColorPrimitives::bt709>::build(),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(dw, dh)),
        Sub<float3>::build(make_<float3>(sub[0], sub[1], sub[2])),
        Div<float3>::build(make_<float3>(div[0], div[1], div[2])), TensorSplit<float3>::build(t));
    return 0;
}

// frames: 2*n_per_seq pointers.  outA: n_per_seq planes of dw x dh uchar3.  outB: 2*n_per_seq planes of w x h float3.
int fklref_divergent(const uint8_t* const* frames, int w, int h, int pitch, int dw, int dh, const float* scales,
                     const float* offs, uint8_t* outA, float* outB, int n_per_seq) {
    switch (n_per_seq) {
    case 1: divergent<1>(frames, w, h, pitch, dw, dh, scales, offs, outA, outB); return 0;
    case 2: divergent<2>(frames, w, h, pitch, dw, dh, scales, offs, outA, outB); return 0;
    case 4: divergent<4>(frames, w, h, pitch, dw, dh, scales, offs, outA, outB); return 0;
    default: return -1;
    }
}

// The constexpr bt709 / Full / 8-bit YCbCr->RGB matrix the reference evaluates (itu_color.h:185-258), row-major.
void fklref_bt709_full_matrix(float* m9) {
    constexpr M3x3Float m = ccMatrix<ColorRange::Full, ColorPrimitives::bt709, ColorConversionDir::YCbCr2RGB, ColorDepth::p8bit>;
    m9[0] = m.x.x; m9[1] = m.x.y; m9[2] = m.x.z; m9[3] = m.y.x; m9[4] = m.y.y; m9[5] = m.y.z;
    m9[6] = m.z.x; m9[7] = m.z.y; m9[8] = m.z.z;
}

}  // extern "C"

// ccMatrix<range, primitives, YCbCr2RGB, p8bit> for range 0 Limited / 1 Full, primitives 0 bt601 / 1 bt709 / 2 bt2020
template <ColorRange CR, ColorPrimitives CP>
static void matrix_of(float* m9) {
    constexpr M3x3Float m = ccMatrix<CR, CP, ColorConversionDir::YCbCr2RGB, ColorDepth::p8bit>;
    m9[0] = m.x.x; m9[1] = m.x.y; m9[2] = m.x.z; m9[3] = m.y.x; m9[4] = m.y.y; m9[5] = m.y.z;
    m9[6] = m.z.x; m9[7] = m.z.y; m9[8] = m.z.z;
}
extern "C" int fklref_ycbcr_matrix(int range, int primitives, float* m9) {
    switch (range * 3 + primitives) {
    case 0: matrix_of<ColorRange::Limited, ColorPrimitives::bt601>(m9); return 0;
    case 1: matrix_of<ColorRange::Limited, ColorPrimitives::bt709>(m9); return 0;
    case 2: matrix_of<ColorRange::Limited, ColorPrimitives::bt2020>(m9); return 0;
    case 3: matrix_of<ColorRange::Full, ColorPrimitives::bt601>(m9); return 0;
    case 4: matrix_of<ColorRange::Full, ColorPrimitives::bt709>(m9); return 0;
    case 5: matrix_of<ColorRange::Full, ColorPrimitives::bt2020>(m9); return 0;
    default: return -1;
    }
}

// Four frames -> BorderReader<BT> -> Crop (rectangles that may leave the frame) -> Resize(PRESERVE_AR, bg) -> Mul ->
// TensorWrite<float3>.  mode: the reference's BorderType value (0 CONSTANT .. 4 REFLECT_101).
template <BorderType BT>
static int border_crop_resize(const uint8_t* const* frames, int w, int h, int pitch, const int32_t* rects, const float* value, int dw, int dh,
                              const float* bg, const float* mul, float* out) {
    CpuStream stream;
    std::array<Ptr2D<uchar3>, 4> ptrs; std::array<Rect, 4> rs;
    for (size_t i = 0; i < 4; ++i) {
        ptrs[i] = wrap_frame(frames[i], w, h, pitch);
        rs[i] = Rect(rects[4 * i], rects[4 * i + 1], rects[4 * i + 2], rects[4 * i + 3]);
    }
    Tensor<float3> t(reinterpret_cast<float3*>(out), dw, dh, 4, 1, MemType::Host, 0);
    const auto resize = Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(Size(dw, dh), make_<float3>(bg[0], bg[1], bg[2]));
    const auto m = Mul<float3>::build(make_<float3>(mul[0], mul[1], mul[2]));
    if constexpr (BT == BorderType::CONSTANT) {
        // the incomplete form BorderReader<CONSTANT>::build(value) does not compile as a link of a chain in the reference;
        // its complete form build(readIOp, value) does (tests/algorithm/test_border_reader.h:26): one plane per call
        const uchar3 v = make_<uchar3>(static_cast<uchar>(value[0]), static_cast<uchar>(value[1]), static_cast<uchar>(value[2]));
        for (size_t i = 0; i < 4; ++i) {
            Tensor<float3> ti(reinterpret_cast<float3*>(out) + i * static_cast<size_t>(dw) * dh, dw, dh, 1, 1, MemType::Host, 0);
            const auto bordered = BorderReader<BT>::build(PerThreadRead<ND::_2D, uchar3>::build(ptrs[i]), v);
            executeOperations<CpuDPP>(stream, bordered, Crop<>::build(rs[i]), resize, m, TensorWrite<float3>::build(ti));
        }
    } else {
        executeOperations<CpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(ptrs), BorderReader<BT>::build(), Crop<>::build(rs), resize, m,
                                  TensorWrite<float3>::build(t));
    }
    return 0;
}
extern "C" int fklref_border_crop_resize(int mode, const uint8_t* const* frames, int w, int h, int pitch, const int32_t* rects, const float* value,
                                         int dw, int dh, const float* bg, const float* mul, float* out) {
    switch (mode) {
    case 0: return border_crop_resize<BorderType::CONSTANT>(frames, w, h, pitch, rects, value, dw, dh, bg, mul, out);
    case 1: return border_crop_resize<BorderType::REPLICATE>(frames, w, h, pitch, rects, value, dw, dh, bg, mul, out);
    case 2: return border_crop_resize<BorderType::REFLECT>(frames, w, h, pitch, rects, value, dw, dh, bg, mul, out);
    case 3: return border_crop_resize<BorderType::WRAP>(frames, w, h, pitch, rects, value, dw, dh, bg, mul, out);
    case 4: return border_crop_resize<BorderType::REFLECT_101>(frames, w, h, pitch, rects, value, dw, dh, bg, mul, out);
    default: return -1;
    }
}
// ReadYUV<NV12> -> ConvertYUVToRGB<p8bit, Full, bt709> -> BorderReader<CONSTANT>(float3) -> Crop -> Resize(IGNORE_AR) -> TensorSplit:
// the constant replaces the converted colour, not the YCbCr triple.
extern "C" int fklref_nv12_border_constant(const uint8_t* nv12, int w, int h, int pitch, const int32_t* rect, const float* value, int dw, int dh,
                                           float* out) {
    CpuStream stream;
    const Ptr<ND::_2D, uchar> data(const_cast<uint8_t*>(nv12), PtrDims<ND::_2D>(w, h + h / 2, pitch), MemType::Host, 0);
    const Image<PixelFormat::NV12> img(data, w, h);
    Tensor<float> t(out, dw, dh, 1, 3, MemType::Host, 0);
    const auto rgb = ReadYUV<PixelFormat::NV12>::build(img).then(ConvertYUVToRGB<ColorDepth::p8bit, ColorRange::Full, ColorPrimitives::bt709>::build());
    const auto bordered = BorderReader<BorderType::CONSTANT>::build(rgb, make_<float3>(value[0], value[1], value[2]));
    executeOperations<CpuDPP>(stream, bordered, Crop<>::build(Rect(rect[0], rect[1], rect[2], rect[3])),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(dw, dh)), TensorSplit<float3>::build(t));
    return 0;
}

// PerThreadRead<uchar3> (R,G,B) -> ConvertRGBToYUV<p8bit, CR, CP> -> SaturateCast -> WriteYUV<PF>
template <PixelFormat PF, ColorRange CR, ColorPrimitives CP>
static int rgb_to_yuv_image(const uint8_t* rgb, int w, int h, int pitch, uint8_t* out, int opitch) {
    CpuStream stream;
    constexpr bool packed = PF == PixelFormat::UYVY;
    const Ptr<ND::_2D, uchar> buf(out, packed ? PtrDims<ND::_2D>(w * 2, h, opitch) : PtrDims<ND::_2D>(w, h + h / 2, opitch), MemType::Host, 0);
    const Image<PF> img(buf, w, h);
    executeOperations<CpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(wrap_frame(rgb, w, h, pitch)),
        ConvertRGBToYUV<ColorDepth::p8bit, CR, CP>::build(), SaturateCast<float3, uchar3>::build(), WriteYUV<PF>::build(img));
    return 0;
}
extern "C" int fklref_rgb_to_yuv_image(int format, int range, int primitives, const uint8_t* rgb, int w, int h, int pitch, uint8_t* out, int opitch) {
    switch (format * 100 + range * 10 + primitives) {
    case 311: return rgb_to_yuv_image<PixelFormat::NV12, ColorRange::Full, ColorPrimitives::bt709>(rgb, w, h, pitch, out, opitch);
    case 300: return rgb_to_yuv_image<PixelFormat::NV12, ColorRange::Limited, ColorPrimitives::bt601>(rgb, w, h, pitch, out, opitch);
    case 402: return rgb_to_yuv_image<PixelFormat::NV21, ColorRange::Limited, ColorPrimitives::bt2020>(rgb, w, h, pitch, out, opitch);
    case 410: return rgb_to_yuv_image<PixelFormat::NV21, ColorRange::Full, ColorPrimitives::bt601>(rgb, w, h, pitch, out, opitch);
    case 501: return rgb_to_yuv_image<PixelFormat::UYVY, ColorRange::Limited, ColorPrimitives::bt709>(rgb, w, h, pitch, out, opitch);
    case 512: return rgb_to_yuv_image<PixelFormat::UYVY, ColorRange::Full, ColorPrimitives::bt2020>(rgb, w, h, pitch, out, opitch);
    default: return -1;
    }
}
template <ColorRange CR, ColorPrimitives CP>
static void inverse_matrix_of(float* m9) {
    constexpr M3x3Float m = ccMatrix<CR, CP, ColorConversionDir::RGB2YCbCr, ColorDepth::p8bit>;
    m9[0] = m.x.x; m9[1] = m.x.y; m9[2] = m.x.z; m9[3] = m.y.x; m9[4] = m.y.y; m9[5] = m.y.z;
    m9[6] = m.z.x; m9[7] = m.z.y; m9[8] = m.z.z;
}
extern "C" int fklref_rgb_to_ycbcr_matrix(int range, int primitives, float* m9) {
    switch (range * 3 + primitives) {
    case 0: inverse_matrix_of<ColorRange::Limited, ColorPrimitives::bt601>(m9); return 0;
    case 1: inverse_matrix_of<ColorRange::Limited, ColorPrimitives::bt709>(m9); return 0;
    case 2: inverse_matrix_of<ColorRange::Limited, ColorPrimitives::bt2020>(m9); return 0;
    case 3: inverse_matrix_of<ColorRange::Full, ColorPrimitives::bt601>(m9); return 0;
    case 4: inverse_matrix_of<ColorRange::Full, ColorPrimitives::bt709>(m9); return 0;
    case 5: inverse_matrix_of<ColorRange::Full, ColorPrimitives::bt2020>(m9); return 0;
    default: return -1;
    }
}

// ReadYUV<PF> -> ConvertYUVToRGB<p8bit, CR, CP> -> Resize(IGNORE_AR) -> Sub -> Div -> TensorSplit<float3>
template <PixelFormat PF, ColorRange CR, ColorPrimitives CP>
static int yuv_resize_split(const uint8_t* data, int w, int h, int pitch, int dw, int dh, const float* sub, const float* div, float* out) {
    CpuStream stream;
    constexpr bool packed = PF == PixelFormat::UYVY;
    const Ptr<ND::_2D, uchar> buf(const_cast<uint8_t*>(data), packed ? PtrDims<ND::_2D>(w * 2, h, pitch) : PtrDims<ND::_2D>(w, h + h / 2, pitch),
                                  MemType::Host, 0);
    const Image<PF> img(buf, w, h);
    Tensor<float> t(out, dw, dh, 1, 3, MemType::Host, 0);
    executeOperations<CpuDPP>(stream, ReadYUV<PF>::build(img), ConvertYUVToRGB<ColorDepth::p8bit, CR, CP>::build(),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(dw, dh)),
        Sub<float3>::build(make_<float3>(sub[0], sub[1], sub[2])), Div<float3>::build(make_<float3>(div[0], div[1], div[2])),
        TensorSplit<float3>::build(t));
    return 0;
}
// format: 3 NV12, 4 NV21, 5 UYVY (this library's source-format codes); a spread of range / primitives per format
extern "C" int fklref_yuv_resize_split(int format, int range, int primitives, const uint8_t* data, int w, int h, int pitch, int dw,
                                       int dh, const float* sub, const float* div, float* out) {
    const int key = format * 100 + range * 10 + primitives;
    switch (key) {
    case 311: return yuv_resize_split<PixelFormat::NV12, ColorRange::Full, ColorPrimitives::bt709>(data, w, h, pitch, dw, dh, sub, div, out);
    case 300: return yuv_resize_split<PixelFormat::NV12, ColorRange::Limited, ColorPrimitives::bt601>(data, w, h, pitch, dw, dh, sub, div, out);
    case 302: return yuv_resize_split<PixelFormat::NV12, ColorRange::Limited, ColorPrimitives::bt2020>(data, w, h, pitch, dw, dh, sub, div, out);
    case 410: return yuv_resize_split<PixelFormat::NV21, ColorRange::Full, ColorPrimitives::bt601>(data, w, h, pitch, dw, dh, sub, div, out);
    case 401: return yuv_resize_split<PixelFormat::NV21, ColorRange::Limited, ColorPrimitives::bt709>(data, w, h, pitch, dw, dh, sub, div, out);
    case 512: return yuv_resize_split<PixelFormat::UYVY, ColorRange::Full, ColorPrimitives::bt2020>(data, w, h, pitch, dw, dh, sub, div, out);
    case 500: return yuv_resize_split<PixelFormat::UYVY, ColorRange::Limited, ColorPrimitives::bt601>(data, w, h, pitch, dw, dh, sub, div, out);
    default: return -1;
    }
}

// ccMatrix<range, primitives, YCbCr2RGB, p10bit> and subCoefficients<p10bit> (luma, chroma)
template <ColorRange CR, ColorPrimitives CP>
static void matrix10_of(float* m9, float* sub2) {
    constexpr M3x3Float m = ccMatrix<CR, CP, ColorConversionDir::YCbCr2RGB, ColorDepth::p10bit>;
    m9[0] = m.x.x; m9[1] = m.x.y; m9[2] = m.x.z; m9[3] = m.y.x; m9[4] = m.y.y; m9[5] = m.y.z;
    m9[6] = m.z.x; m9[7] = m.z.y; m9[8] = m.z.z;
    sub2[0] = subCoefficients<ColorDepth::p10bit>.luma; sub2[1] = subCoefficients<ColorDepth::p10bit>.chroma;
}
extern "C" int fklref_ycbcr_matrix10(int range, int primitives, float* m9, float* sub2) {
    switch (range * 3 + primitives) {
    case 0: matrix10_of<ColorRange::Limited, ColorPrimitives::bt601>(m9, sub2); return 0;
    case 1: matrix10_of<ColorRange::Limited, ColorPrimitives::bt709>(m9, sub2); return 0;
    case 2: matrix10_of<ColorRange::Limited, ColorPrimitives::bt2020>(m9, sub2); return 0;
    case 3: matrix10_of<ColorRange::Full, ColorPrimitives::bt601>(m9, sub2); return 0;
    case 4: matrix10_of<ColorRange::Full, ColorPrimitives::bt709>(m9, sub2); return 0;
    case 5: matrix10_of<ColorRange::Full, ColorPrimitives::bt2020>(m9, sub2); return 0;
    default: return -1;
    }
}

// ReadYUV<PF> (ushort samples) -> ConvertYUVToRGB<p10bit, CR, CP> -> Resize(IGNORE_AR) -> Sub -> Div -> TensorSplit<float3>.
// The buffer is PixelFormatTraits<PF>::rf times the picture, in ushort elements; pitch is in bytes.
template <PixelFormat PF, ColorRange CR, ColorPrimitives CP>
static int yuv10_resize_split(const uint16_t* data, int w, int h, int pitch, int dw, int dh, const float* sub, const float* div, float* out) {
    CpuStream stream;
    const uint bw = static_cast<uint>(w * PixelFormatTraits<PF>::rf.width_f), bh = static_cast<uint>(h * PixelFormatTraits<PF>::rf.height_f);
    const Ptr<ND::_2D, ushort> buf(const_cast<uint16_t*>(data), PtrDims<ND::_2D>(bw, bh, pitch), MemType::Host, 0);
    const Image<PF> img(buf, w, h);
    Tensor<float> t(out, dw, dh, 1, 3, MemType::Host, 0);
    executeOperations<CpuDPP>(stream, ReadYUV<PF>::build(img), ConvertYUVToRGB<ColorDepth::p10bit, CR, CP>::build(),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(dw, dh)),
        Sub<float3>::build(make_<float3>(sub[0], sub[1], sub[2])), Div<float3>::build(make_<float3>(div[0], div[1], div[2])),
        TensorSplit<float3>::build(t));
    return 0;
}
// format: 9 P010, 10 P210, 11 Y210 (this library's source-format codes)
extern "C" int fklref_yuv10_resize_split(int format, int range, int primitives, const uint16_t* data, int w, int h, int pitch, int dw,
                                         int dh, const float* sub, const float* div, float* out) {
    const int key = format * 100 + range * 10 + primitives;
    switch (key) {
    case 902: return yuv10_resize_split<PixelFormat::P010, ColorRange::Limited, ColorPrimitives::bt2020>(data, w, h, pitch, dw, dh, sub, div, out);
    case 911: return yuv10_resize_split<PixelFormat::P010, ColorRange::Full, ColorPrimitives::bt709>(data, w, h, pitch, dw, dh, sub, div, out);
    case 1001: return yuv10_resize_split<PixelFormat::P210, ColorRange::Limited, ColorPrimitives::bt709>(data, w, h, pitch, dw, dh, sub, div, out);
    case 1012: return yuv10_resize_split<PixelFormat::P210, ColorRange::Full, ColorPrimitives::bt2020>(data, w, h, pitch, dw, dh, sub, div, out);
    case 1102: return yuv10_resize_split<PixelFormat::Y210, ColorRange::Limited, ColorPrimitives::bt2020>(data, w, h, pitch, dw, dh, sub, div, out);
    case 1110: return yuv10_resize_split<PixelFormat::Y210, ColorRange::Full, ColorPrimitives::bt601>(data, w, h, pitch, dw, dh, sub, div, out);
    default: return -1;
    }
}

extern "C" {
uint8_t fklref_saturate_u8(float v) { return cxp::saturate_cast<uchar>::f(v); }

// Resize<INTER_LINEAR,AR>::build on a w x h source: returns fx, fy, x1, y1, x2, y2.  `ar` is the reference's own
// AspectRatio value: 0 PRESERVE_AR, 1 IGNORE_AR, 2 PRESERVE_AR_RN_EVEN, 3 PRESERVE_AR_LEFT.
void fklref_resize_params(int sw, int sh, int dw, int dh, int ar, float* f2, int32_t* r4) {
    static uchar3 dummy;
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(RawPtr<ND::_2D, uchar3>{&dummy, {static_cast<uint>(sw), static_cast<uint>(sh), static_cast<uint>(sw * 3)}});
    if (ar == 1) {
        const auto r = Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(read, Size(dw, dh));
        f2[0] = r.params.src_conv_factors.x; f2[1] = r.params.src_conv_factors.y;
        r4[0] = 0; r4[1] = 0; r4[2] = dw - 1; r4[3] = dh - 1;
    } else if (ar == 2) {
        letterbox_params<AspectRatio::PRESERVE_AR_RN_EVEN>(read, dw, dh, f2, r4);
    } else if (ar == 3) {
        letterbox_params<AspectRatio::PRESERVE_AR_LEFT>(read, dw, dh, f2, r4);
    } else {
        letterbox_params<AspectRatio::PRESERVE_AR>(read, dw, dh, f2, r4);
    }
}

}  // extern "C"
