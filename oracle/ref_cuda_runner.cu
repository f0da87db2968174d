// TEST / BENCHMARK INFRASTRUCTURE — not part of the product.  Like ref_runner.cpp this file has no arithmetic of its
// own: it includes the FusedKernelLibrary headers from where they are installed and runs the reference's own CUDA
// backend (TransformDPP<ParArch::GPU_NVIDIA>: core/execution_model/executors.h:311-358, the generic templated kernel
// of executor_details/executor_kernels.h:26-30) on caller-provided DEVICE buffers and stream, so that the benchmark can
// time the reference's GPU path beside this library's kernels on the same B200.  Built by oracle/Makefile into
// oracle/_ref/libfkl_ref_cuda.so with the reference's default arithmetic flags (FMA contraction on, as its CMake does).
//
// The reference passes every IOp by value as a kernel parameter (96 bytes per plane of a crop+resize batch), so a batch
// is limited by the 32 KB parameter space: the 2048-plane workload runs as 8 launches of 256 planes here.
#include <fused_kernel/algorithms/basic_ops/arithmetic.h>
#include <fused_kernel/algorithms/basic_ops/cast.h>
#include <fused_kernel/algorithms/basic_ops/memory_operations.h>
#include <fused_kernel/algorithms/image_processing/color_conversion.h>
#include <fused_kernel/algorithms/image_processing/crop.h>
#include <fused_kernel/algorithms/image_processing/image.h>
#include <fused_kernel/algorithms/image_processing/resize.h>
#include <fused_kernel/algorithms/image_processing/saturate.h>
#include <fused_kernel/fused_kernel.h>

#include <array>
#include <cstdint>

using namespace fk;

namespace {
using GpuStream = Stream_<ParArch::GPU_NVIDIA>;
using GpuDPP = TransformDPP<ParArch::GPU_NVIDIA>;

inline Ptr2D<uchar3> wrap(const uint8_t* p, int w, int h, int pitch) {
    return Ptr2D<uchar3>(reinterpret_cast<uchar3*>(const_cast<uint8_t*>(p)), w, h, pitch, MemType::Device, 0);
}

template <size_t B>
void crop_resize_f32(GpuStream& stream, const uint8_t* const* frames, int w, int h, int pitch, const int32_t* rects, int first,
                     int dw, int dh, float3 bg, float3 mul, float* out) {
    std::array<Ptr2D<uchar3>, B> ptrs;
    std::array<Rect, B> rs;
    for (size_t i = 0; i < B; ++i) {
        ptrs[i] = wrap(frames[first + i], w, h, pitch);
        const int32_t* r = rects + 4 * (first + i);
        rs[i] = Rect(r[0], r[1], r[2], r[3]);
    }
    Tensor<float3> t(reinterpret_cast<float3*>(out) + static_cast<size_t>(first) * dw * dh, dw, dh, B, 1, MemType::Device, 0);
    executeOperations<GpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(ptrs), Crop<>::build(rs),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(Size(dw, dh), bg), Mul<float3>::build(mul),
        TensorWrite<float3>::build(t));
}
// README pipeline: five crops of one frame -> Resize(PRESERVE_AR, bg) -> Mul -> Sub -> SaturateCast -> TensorWrite<uchar3>
void readme_crops(GpuStream& stream, const uint8_t* frame, int w, int h, int pitch, const int32_t* rects, int dw, int dh, float3 bg, float3 mul,
                  float3 sub, uint8_t* out) {
    std::array<Ptr2D<uchar3>, 5> ptrs;
    std::array<Rect, 5> rs;
    for (size_t i = 0; i < 5; ++i) { ptrs[i] = wrap(frame, w, h, pitch); rs[i] = Rect(rects[4 * i], rects[4 * i + 1], rects[4 * i + 2], rects[4 * i + 3]); }
    Tensor<uchar3> t(reinterpret_cast<uchar3*>(out), dw, dh, 5, 1, MemType::Device, 0);
    executeOperations<GpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(ptrs), Crop<>::build(rs),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(Size(dw, dh), bg), Mul<float3>::build(mul), Sub<float3>::build(sub),
        SaturateCast<float3, uchar3>::build(), TensorWrite<uchar3>::build(t));
}

// Divergent batch of 2N planes: planes [0,N) Resize -> SaturateCast -> TensorWrite<uchar3>; planes [N,2N) Cast -> Mul -> Sub fused
// into each plane's Read -> TensorWrite<float3> by global plane index (executors.h:360-411).
template <uint N>
struct SelN { FK_HOST_DEVICE_FUSE uint at(const uint& z) { return z < N ? 0u : 1u; } };
template <uint N>
void divergent(GpuStream& stream, const uint8_t* const* frames, int w, int h, int pitch, int dw, int dh, const float* scales, const float* offs,
               uint8_t* outA, float* outB) {
    std::array<Ptr2D<uchar3>, N> firstN;
    for (uint i = 0; i < N; ++i) firstN[i] = wrap(frames[i], w, h, pitch);
    Tensor<uchar3> tA(reinterpret_cast<uchar3*>(outA), dw, dh, N, 1, MemType::Device, 0);
    const auto seq0 = buildOperationSequence(PerThreadRead<ND::_2D, uchar3>::build(firstN), Resize<InterpolationType::INTER_LINEAR>::build(Size(dw, dh)),
                                             SaturateCast<float3, uchar3>::build(), TensorWrite<uchar3>::build(tA));
    const Ptr2D<uchar3> f0 = wrap(frames[N], w, h, pitch);
    using FusedRead = decltype(PerThreadRead<ND::_2D, uchar3>::build(f0).then(Cast<uchar3, float3>::build())
        .then(Mul<float3>::build(make_set<float3>(1.f))).then(Sub<float3>::build(make_set<float3>(0.f))));
    std::array<FusedRead, 2 * N> reads;
    for (uint i = 0; i < 2 * N; ++i) {
        const uint k = i < N ? 0 : i - N;
        reads[i] = PerThreadRead<ND::_2D, uchar3>::build(wrap(frames[N + k], w, h, pitch)).then(Cast<uchar3, float3>::build())
            .then(Mul<float3>::build(make_set<float3>(scales[k]))).then(Sub<float3>::build(make_set<float3>(offs[k])));
    }
    auto batchRead = BatchRead<PlanePolicy::PROCESS_ALL>::build(reads);
    batchRead.params.activeThreads.z = N;
    Tensor<float3> tB(reinterpret_cast<float3*>(outB), w, h, 2 * N, 1, MemType::Device, 0);
    const auto seq1 = buildOperationSequence(batchRead, TensorWrite<float3>::build(tB));
    Executor<DivergentBatchTransformDPP<ParArch::GPU_NVIDIA, SelN<N>>>::executeOperations(stream, seq0, seq1);
}
}  // namespace

extern "C" {

int fklrefcuda_readme_crops(const uint8_t* frame, int w, int h, int pitch, const int32_t* rects, int dw, int dh, const float* bg, const float* mul,
                            const float* sub, uint8_t* out, void* cuda_stream) {
    GpuStream stream(static_cast<cudaStream_t>(cuda_stream));
    readme_crops(stream, frame, w, h, pitch, rects, dw, dh, make_<float3>(bg[0], bg[1], bg[2]), make_<float3>(mul[0], mul[1], mul[2]),
                 make_<float3>(sub[0], sub[1], sub[2]), out);
    return 1;
}

// frames: 2*4 host-array of device pointers; outA: 4 planes of dw x dh uchar3; outB: 8 planes of w x h float3
int fklrefcuda_divergent4(const uint8_t* const* frames, int w, int h, int pitch, int dw, int dh, const float* scales, const float* offs,
                          uint8_t* outA, float* outB, void* cuda_stream) {
    GpuStream stream(static_cast<cudaStream_t>(cuda_stream));
    divergent<4>(stream, frames, w, h, pitch, dw, dh, scales, offs, outA, outB);
    return 1;
}

// frames/rects are HOST arrays (of device pointers / of ints); out is a device pointer.  n must be a multiple of 32.
// Returns the number of kernel launches, or -1.
int fklrefcuda_crop_resize_f32(const uint8_t* const* frames, int w, int h, int pitch, const int32_t* rects, int n, int dw, int dh,
                               const float* bg, const float* mul, float* out, void* cuda_stream) {
    if (n % 32) return -1;
    GpuStream stream(static_cast<cudaStream_t>(cuda_stream));
    const float3 b = make_<float3>(bg[0], bg[1], bg[2]), m = make_<float3>(mul[0], mul[1], mul[2]);
    int at = 0, launches = 0;
    for (; n - at >= 256; at += 256, ++launches) crop_resize_f32<256>(stream, frames, w, h, pitch, rects, at, dw, dh, b, m, out);
    for (; n - at >= 32; at += 32, ++launches) crop_resize_f32<32>(stream, frames, w, h, pitch, rects, at, dw, dh, b, m, out);
    return launches;
}

// Read -> Cast -> Mul -> Add -> Div -> ColorConversion<BGR2RGB> -> SaturateCast -> PerThreadWrite (device pointers)
int fklrefcuda_pointwise_u8(const uint8_t* src, int w, int h, int spitch, const float* mul, const float* add, const float* div,
                            uint8_t* dst, int dpitch, void* cuda_stream) {
    GpuStream stream(static_cast<cudaStream_t>(cuda_stream));
    executeOperations<GpuDPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(wrap(src, w, h, spitch)), Cast<uchar3, float3>::build(),
        Mul<float3>::build(make_<float3>(mul[0], mul[1], mul[2])), Add<float3>::build(make_<float3>(add[0], add[1], add[2])),
        Div<float3>::build(make_<float3>(div[0], div[1], div[2])), ColorConversion<ColorConversionCodes::COLOR_BGR2RGB, float3, float3>::build(),
        SaturateCast<float3, uchar3>::build(), PerThreadWrite<ND::_2D, uchar3>::build(wrap(dst, w, h, dpitch)));
    return 1;
}

// ReadYUV<NV12> -> ConvertYUVToRGB<p8bit,Full,bt709> -> Resize(IGNORE_AR) -> Sub -> Div -> TensorSplit<float3>
int fklrefcuda_nv12_resize_split(const uint8_t* nv12, int w, int h, int pitch, int dw, int dh, const float* sub, const float* div,
                                 float* out, void* cuda_stream) {
    GpuStream stream(static_cast<cudaStream_t>(cuda_stream));
    const Ptr<ND::_2D, uchar> data(const_cast<uint8_t*>(nv12), PtrDims<ND::_2D>(w, h + h / 2, pitch), MemType::Device, 0);
    const Image<PixelFormat::NV12> img(data, w, h);
    Tensor<float> t(out, dw, dh, 1, 3, MemType::Device, 0);
    executeOperations<GpuDPP>(stream, ReadYUV<PixelFormat::NV12>::build(img),
        ConvertYUVToRGB<ColorDepth::p8bit, ColorRange::Full, ColorPrimitives::bt709>::build(),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(dw, dh)),
        Sub<float3>::build(make_<float3>(sub[0], sub[1], sub[2])), Div<float3>::build(make_<float3>(div[0], div[1], div[2])),
        TensorSplit<float3>::build(t));
    return 1;
}

}  // extern "C"
