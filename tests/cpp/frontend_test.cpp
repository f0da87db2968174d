// GPU test of the fk:: front end: the benchmark pipelines written exactly as a FusedKernelLibrary user writes them
// (compare the reference's tests/examples/readme_test_code.h:26-106, utests/core/execution_model/utest_executors.h:91-134,
// tests/data_parallel_patterns/test_divergent_batch.h:28-92), executed through the front end -> C ABI -> sm_100a
// kernels, and compared bit for bit with the CPU oracle run on the same host data (descriptors built by hand here, so
// the front end's lowering is checked too).  Prints one line per case; exit code 0 = all passed.
#include <fused_kernel/algorithms/basic_ops/arithmetic.h>
#include <fused_kernel/algorithms/basic_ops/cast.h>
#include <fused_kernel/algorithms/basic_ops/memory_operations.h>
#include <fused_kernel/algorithms/image_processing/color_conversion.h>
#include <fused_kernel/algorithms/image_processing/crop.h>
#include <fused_kernel/algorithms/image_processing/image.h>
#include <fused_kernel/algorithms/image_processing/resize.h>
#include <fused_kernel/algorithms/image_processing/saturate.h>
#include <fused_kernel/fused_kernel.h>

#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

using namespace fk;

extern "C" int fkb_oracle_resize_params(uint32_t geometry, fkb_plane_desc* pl);
extern "C" int fkb_oracle_run(const fkb_chain_desc* chains, uint32_t n_chains, const fkb_plane_desc* planes, uint32_t n_planes, uint32_t n_threads);

static int g_failed = 0;
static void report(const char* name, bool ok) {
    std::printf("%-38s %s\n", name, ok ? "PASS" : "FAIL");
    if (!ok) ++g_failed;
}
template <typename P>
static void fill_random(P& p, uint32_t seed, int lo = 0, int hi = 255) {
    std::mt19937 rng(seed);
    uint8_t* b = reinterpret_cast<uint8_t*>(p.ptrPinned().data);
    for (size_t i = 0; i < p.sizeInBytes(); ++i) b[i] = static_cast<uint8_t>(lo + rng() % (hi - lo + 1));
}
static fkb_op op(uint16_t code, float a = 0, float b = 0, float c = 0, int slot = -1) {
    fkb_op o{}; o.code = code; o.plane_slot = static_cast<int16_t>(slot); o.v[0] = a; o.v[1] = b; o.v[2] = c; return o;
}
static fkb_plane_desc host_plane(const Ptr2D<uchar3>& src, Rect crop, uint32_t dw, uint32_t dh, void* dst, uint32_t dpitch, uint32_t geometry) {
    fkb_plane_desc d{};
    const auto r = src.ptrPinned();
    d.src = r.data; d.src_pitch = r.dims.pitch; d.src_w = r.dims.width; d.src_h = r.dims.height;
    d.crop_x = crop.x; d.crop_y = crop.y; d.crop_w = crop.width; d.crop_h = crop.height;
    d.dst = dst; d.dst_w = dw; d.dst_h = dh; d.dst_pitch = dpitch;
    if (geometry != FKB_GEOM_NONE) fkb_oracle_resize_params(geometry, &d);
    return d;
}

// ---- README pipeline: 5 crops of a 1080p frame -> 128x64 uchar3 tensor ------------------------------------------
static void test_readme() {
    Stream stream;
    constexpr int BATCH = 5;
    Ptr2D<uchar3> inputImage(1920, 1080);  // cudaMallocPitch: the pitch may be padded
    fill_random(inputImage, 1);
    inputImage.upload(stream);
    constexpr std::array<Rect, BATCH> crops{Rect(300, 125, 60, 40), Rect(400, 125, 60, 40), Rect(530, 270, 130, 140), Rect(560, 115, 100, 35), Rect(572, 196, 40, 15)};
    constexpr Size outputSize(128, 64);
    Tensor<uchar3> output(outputSize.width, outputSize.height, BATCH);
    executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(inputImage), Crop<>::build(crops),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(outputSize, make_<float3>(0.f, 0.f, 0.f)),
        Mul<float3>::build(make_<float3>(2.f, 2.f, 2.f)), Sub<float3>::build(make_set<float3>(128.f)),
        SaturateCast<float3, uchar3>::build(), TensorWrite<uchar3>::build(output));
    output.download(stream);
    // the same chain in .then() form must give the same result (utest_executors.h:91-134)
    Tensor<uchar3> output2(outputSize.width, outputSize.height, BATCH);
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(inputImage).then(Crop<>::build(crops))
        .then(Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(outputSize, make_<float3>(0.f, 0.f, 0.f)))
        .then(Mul<float3>::build(make_<float3>(2.f, 2.f, 2.f))).then(Sub<float3>::build(make_set<float3>(128.f)))
        .then(SaturateCast<float3, uchar3>::build());
    executeOperations<TransformDPP<>>(stream, sender, TensorWrite<uchar3>::build(output2));
    output2.download(stream);
    stream.sync();

    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C3; ch.geometry = FKB_GEOM_RESIZE_PRESERVE_AR; ch.dst_format = FKB_PIX_U8C3; ch.write_kind = FKB_WRITE_PACKED;
    ch.n_ops = 3; ch.ops[0] = op(FKB_OP_MUL, 2, 2, 2); ch.ops[1] = op(FKB_OP_SUB, 128, 128, 128); ch.ops[2] = op(FKB_OP_SATCAST_U8);
    std::vector<uint8_t> want(128 * 64 * 3 * BATCH);
    std::vector<fkb_plane_desc> planes;
    for (int i = 0; i < BATCH; ++i) planes.push_back(host_plane(inputImage, crops[i], 128, 64, want.data() + i * 128 * 64 * 3, 128 * 3, ch.geometry));
    fkb_oracle_run(&ch, 1, planes.data(), BATCH, 1);
    report("readme crop pipeline (variadic)", std::memcmp(want.data(), output.ptrPinned().data, want.size()) == 0);
    report("readme crop pipeline (.then form)", std::memcmp(want.data(), output2.ptrPinned().data, want.size()) == 0);
    report("activeThreads of the fused read", sender.getActiveThreads().x == 128 && sender.getActiveThreads().y == 64 && sender.getActiveThreads().z == 5);
}

// ---- thread fusion: TransformDPP<PA, TF::ENABLED> is the same launch ----------------------------------------------
// The reference's TF::ENABLED makes a thread process several elements of narrow types (core/execution_model/
// thread_fusion.h:82-160, data_parallel_patterns.h:143-171); its three- and four-channel types get one element per thread
// either way (thread_fusion.h:54), and a ReadBack switches it off.  Here every path is vectorised by construction, so the
// flag must compile and change no byte.
static void test_thread_fusion() {
    Stream stream;
    const uint W = 1000, H = 75;
    Ptr2D<uchar3> in(W, H), out0(W, H), out1(W, H);
    fill_random(in, 7);
    in.upload(stream);
    auto run = [&](auto dpp, Ptr2D<uchar3>& out) {
        using DPP = decltype(dpp);
        executeOperations<DPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(in), Cast<uchar3, float3>::build(),
            Mul<float3>::build(make_<float3>(0.5f, 1.5f, 2.0f)), Add<float3>::build(make_<float3>(10.f, -20.f, 5.f)),
            SaturateCast<float3, uchar3>::build(), PerThreadWrite<ND::_2D, uchar3>::build(out));
        out.download(stream);
    };
    run(TransformDPP<ParArch::GPU_NVIDIA, TF::DISABLED>{}, out0);
    run(TransformDPP<ParArch::GPU_NVIDIA, TF::ENABLED>{}, out1);
    // and a chain with a ReadBack (crop + resize) under both flags
    constexpr std::array<Rect, 2> crops{Rect(30, 5, 60, 40), Rect(400, 12, 130, 60)};
    Tensor<float3> t0(64, 48, 2), t1(64, 48, 2);
    auto run_resize = [&](auto dpp, Tensor<float3>& out) {
        using DPP = decltype(dpp);
        executeOperations<DPP>(stream, PerThreadRead<ND::_2D, uchar3>::build(in), Crop<>::build(crops),
            Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(Size(64, 48), make_<float3>(1.f, 2.f, 3.f)),
            Mul<float3>::build(make_set<float3>(1.f / 255.f)), TensorWrite<float3>::build(out));
        out.download(stream);
    };
    run_resize(TransformDPP<ParArch::GPU_NVIDIA, TF::DISABLED>{}, t0);
    run_resize(TransformDPP<ParArch::GPU_NVIDIA, TF::ENABLED>{}, t1);
    stream.sync();
    bool ok = true;
    const uint pitch = out0.dims().pitch;
    for (uint y = 0; y < H && ok; ++y)
        ok = std::memcmp(reinterpret_cast<uint8_t*>(out0.ptrPinned().data) + static_cast<size_t>(y) * pitch,
                         reinterpret_cast<uint8_t*>(out1.ptrPinned().data) + static_cast<size_t>(y) * pitch, W * 3) == 0;
    report("TF::ENABLED == TF::DISABLED (pointwise chain)", ok);
    report("TF::ENABLED == TF::DISABLED (crop + resize chain)", std::memcmp(t0.ptrPinned().data, t1.ptrPinned().data, 64 * 48 * 2 * 12) == 0);
}

// ---- gray conversions: one-channel outputs -------------------------------------------------------------------------
static void test_gray() {
    Stream stream;
    // (1) a whole uchar4 image: ColorConversion<COLOR_BGRA2GRAY, uchar4, uchar> -> PerThreadWrite<_2D, uchar>
    const uint W = 322, H = 45;
    Ptr2D<uchar4> in4(W, H);
    Ptr2D<uchar> g(W, H);
    fill_random(in4, 31);
    in4.upload(stream);
    executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar4>::build(in4),
        ColorConversion<ColorConversionCodes::COLOR_BGRA2GRAY, uchar4, uchar>::build(), PerThreadWrite<ND::_2D, uchar>::build(g));
    g.download(stream);
    // (2) crops of a uchar3 image: Resize -> RGB2GRAY on float3 -> Mul<float> -> SaturateCast<float, uchar> -> TensorWrite<uchar>
    Ptr2D<uchar3> in3(640, 360);
    fill_random(in3, 32);
    in3.upload(stream);
    constexpr std::array<Rect, 3> crops{Rect(30, 20, 200, 120), Rect(300, 60, 64, 200), Rect(0, 0, 640, 360)};
    Tensor<uchar> t(96, 64, 3);
    executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(in3), Crop<>::build(crops),
        Resize<InterpolationType::INTER_LINEAR>::build(Size(96, 64)), ColorConversion<ColorConversionCodes::COLOR_RGB2GRAY, float3, float>::build(),
        Mul<float>::build(1.25f), SaturateCast<float, uchar>::build(), TensorWrite<uchar>::build(t));
    t.download(stream);
    stream.sync();

    fkb_chain_desc c1{};
    c1.src_format = FKB_PIX_U8C4; c1.geometry = FKB_GEOM_NONE; c1.dst_format = FKB_PIX_U8C1; c1.write_kind = FKB_WRITE_PACKED;
    c1.n_ops = 2; c1.ops[0] = op(FKB_OP_REORDER_ZYX); c1.ops[1] = op(FKB_OP_RGB2GRAY, 1.f);
    const uint gp = g.dims().pitch;
    std::vector<uint8_t> want1(static_cast<size_t>(gp) * H, 0);
    fkb_plane_desc d1{};
    const auto r4 = in4.ptrPinned();
    d1.src = r4.data; d1.src_pitch = r4.dims.pitch; d1.src_w = W; d1.src_h = H; d1.crop_w = W; d1.crop_h = H;
    d1.dst = want1.data(); d1.dst_w = W; d1.dst_h = H; d1.dst_pitch = gp;
    fkb_oracle_run(&c1, 1, &d1, 1, 1);
    bool ok = true;
    for (uint y = 0; y < H && ok; ++y) ok = std::memcmp(want1.data() + static_cast<size_t>(y) * gp, reinterpret_cast<uint8_t*>(g.ptrPinned().data) + static_cast<size_t>(y) * gp, W) == 0;
    report("COLOR_BGRA2GRAY uchar4 -> uchar image", ok);

    fkb_chain_desc c2{};
    c2.src_format = FKB_PIX_U8C3; c2.geometry = FKB_GEOM_RESIZE_IGNORE_AR; c2.dst_format = FKB_PIX_U8C1; c2.write_kind = FKB_WRITE_PACKED;
    c2.n_ops = 3; c2.ops[0] = op(FKB_OP_RGB2GRAY); c2.ops[1] = op(FKB_OP_MUL, 1.25f, 1.25f, 1.25f); c2.ops[2] = op(FKB_OP_SATCAST_U8);
    std::vector<uint8_t> want2(96 * 64 * 3);
    std::vector<fkb_plane_desc> planes;
    for (int i = 0; i < 3; ++i) planes.push_back(host_plane(in3, crops[i], 96, 64, want2.data() + i * 96 * 64, 96, c2.geometry));
    fkb_oracle_run(&c2, 1, planes.data(), 3, 1);
    report("crops -> Resize -> COLOR_RGB2GRAY -> Mul<float> -> uchar tensor", std::memcmp(want2.data(), t.ptrPinned().data, want2.size()) == 0);
}

// ---- vertical fusion: Cast, Mul, Add, Div, BGR2RGB, SaturateCast on every pixel ----------------------------------
static void test_vertical_fusion() {
    Stream stream;
    const uint W = 1000, H = 75;
    Ptr2D<uchar3> in(W, H), out(W, H);
    fill_random(in, 2);
    in.upload(stream);
    executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(in), Cast<uchar3, float3>::build(),
        Mul<float3>::build(make_<float3>(0.5f, 1.5f, 2.0f)), Add<float3>::build(make_<float3>(10.f, -20.f, 5.f)),
        Div<float3>::build(make_set<float3>(1.7f)), ColorConversion<ColorConversionCodes::COLOR_BGR2RGB, float3, float3>::build(),
        SaturateCast<float3, uchar3>::build(), PerThreadWrite<ND::_2D, uchar3>::build(out));
    out.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C3; ch.geometry = FKB_GEOM_NONE; ch.dst_format = FKB_PIX_U8C3; ch.write_kind = FKB_WRITE_PACKED;
    ch.n_ops = 6; ch.ops[0] = op(FKB_OP_CAST_F32); ch.ops[1] = op(FKB_OP_MUL, 0.5f, 1.5f, 2.0f); ch.ops[2] = op(FKB_OP_ADD, 10.f, -20.f, 5.f);
    ch.ops[3] = op(FKB_OP_DIV, 1.7f, 1.7f, 1.7f); ch.ops[4] = op(FKB_OP_REORDER_ZYX); ch.ops[5] = op(FKB_OP_SATCAST_U8);
    const uint pitch = out.dims().pitch;
    std::vector<uint8_t> want(static_cast<size_t>(pitch) * H, 0);
    fkb_plane_desc d = host_plane(in, Rect(0, 0, W, H), W, H, want.data(), pitch, FKB_GEOM_NONE);
    fkb_oracle_run(&ch, 1, &d, 1, 1);
    bool ok = true;
    for (uint y = 0; y < H && ok; ++y) ok = std::memcmp(want.data() + static_cast<size_t>(y) * pitch, reinterpret_cast<uint8_t*>(out.ptrPinned().data) + static_cast<size_t>(y) * pitch, W * 3) == 0;
    report("vertical fusion uchar3 -> uchar3", ok);
}

// ---- NV12 -> RGB -> resize -> normalise -> planar CHW ---------------------------------------------------------------
static void test_nv12() {
    Stream stream;
    const uint W = 640, H = 360, DW = 160, DH = 96;
    Image<PixelFormat::NV12> img(W, H);
    auto data = img.getData();
    fill_random(data, 3, 16, 235);
    img.upload(stream);
    Tensor<float> out(DW, DH, 1, 3);
    executeOperations<TransformDPP<>>(stream, ReadYUV<PixelFormat::NV12>::build(img),
        ConvertYUVToRGB<ColorDepth::p8bit, ColorRange::Full, ColorPrimitives::bt709>::build(),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(DW, DH)),
        Sub<float3>::build(make_<float3>(123.675f, 116.28f, 103.53f)), Div<float3>::build(make_<float3>(58.395f, 57.12f, 57.375f)),
        TensorSplit<float3>::build(out));
    out.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_NV12; ch.geometry = FKB_GEOM_RESIZE_IGNORE_AR; ch.dst_format = FKB_PIX_F32C3; ch.write_kind = FKB_WRITE_SPLIT;
    ch.n_ops = 3; ch.n_pre_ops = 1; ch.ops[0] = op(FKB_OP_YUV2RGB); ch.ops[1] = op(FKB_OP_SUB, 123.675f, 116.28f, 103.53f); ch.ops[2] = op(FKB_OP_DIV, 58.395f, 57.12f, 57.375f);
    const float m[9] = {1.f, 0.f, 1.57480001f, 1.f, -0.187324256f, -0.46812427f, 1.f, 1.8556f, 0.f};
    std::memcpy(ch.ccm, m, sizeof(m)); ch.yuv_sub[1] = 128.f; ch.yuv_sub[2] = 128.f;
    std::vector<float> want(DW * DH * 3);
    fkb_plane_desc d{};
    const auto r = data.ptrPinned();
    d.src = r.data; d.src_chroma = reinterpret_cast<uint8_t*>(r.data) + static_cast<size_t>(r.dims.pitch) * H; d.src_pitch = r.dims.pitch; d.src_w = W; d.src_h = H;
    d.crop_w = W; d.crop_h = H; d.dst = want.data(); d.dst_w = DW; d.dst_h = DH; d.dst_pitch = DW * 4; d.dst_channel_stride = DW * DH * 4;
    fkb_oracle_resize_params(ch.geometry, &d);
    fkb_oracle_run(&ch, 1, &d, 1, 1);
    report("NV12 -> planar float CHW", std::memcmp(want.data(), out.ptrPinned().data, want.size() * 4) == 0);
}

// ---- the other 8-bit sources and colour descriptions: NV21 / UYVY, limited range, bt601 / bt2020 -------------------
extern "C" int fkb_oracle_ycbcr_to_rgb_bits(uint32_t bits, uint32_t range, uint32_t primitives, float* ccm, float* yuv_sub);
template <PixelFormat PF, ColorRange CR, ColorPrimitives CP>
static void test_yuv(const char* what, uint32_t fmt, uint32_t range, uint32_t prim) {
    Stream stream;
    const uint W = 320, H = 180, DW = 111, DH = 70;
    Image<PF> img(W, H);
    auto data = img.getData();
    constexpr bool wide = PixelFormatTraits<PF>::wide;  // ushort samples holding ten bits
    if constexpr (wide) {
        std::mt19937 rng(5);
        uint16_t* b = reinterpret_cast<uint16_t*>(data.ptrPinned().data);
        for (size_t i = 0; i < data.sizeInBytes() / 2; ++i) b[i] = static_cast<uint16_t>(40 + rng() % 960);
    } else {
        fill_random(data, 5, 16, 235);
    }
    img.upload(stream);
    Tensor<float> out(DW, DH, 1, 3);
    executeOperations<TransformDPP<>>(stream, ReadYUV<PF>::build(img), ConvertYUVToRGB<PixelFormatTraits<PF>::depth, CR, CP>::build(),
        Resize<InterpolationType::INTER_LINEAR, AspectRatio::IGNORE_AR>::build(Size(DW, DH)),
        Sub<float3>::build(make_<float3>(123.675f, 116.28f, 103.53f)), TensorSplit<float3>::build(out));
    out.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = fmt; ch.geometry = FKB_GEOM_RESIZE_IGNORE_AR; ch.dst_format = FKB_PIX_F32C3; ch.write_kind = FKB_WRITE_SPLIT;
    ch.n_ops = 2; ch.n_pre_ops = 1; ch.ops[0] = op(FKB_OP_YUV2RGB); ch.ops[1] = op(FKB_OP_SUB, 123.675f, 116.28f, 103.53f);
    fkb_oracle_ycbcr_to_rgb_bits(wide ? 10 : 8, range, prim, ch.ccm, ch.yuv_sub);
    std::vector<float> want(DW * DH * 3);
    fkb_plane_desc d{};
    const auto r = data.ptrPinned();
    d.src = r.data; d.src_pitch = r.dims.pitch; d.src_w = W; d.src_h = H;
    if (fmt != FKB_PIX_UYVY && fmt != FKB_PIX_Y210) d.src_chroma = reinterpret_cast<uint8_t*>(r.data) + static_cast<size_t>(r.dims.pitch) * H;
    d.crop_w = W; d.crop_h = H; d.dst = want.data(); d.dst_w = DW; d.dst_h = DH; d.dst_pitch = DW * 4; d.dst_channel_stride = DW * DH * 4;
    fkb_oracle_resize_params(ch.geometry, &d);
    fkb_oracle_run(&ch, 1, &d, 1, 1);
    report(what, std::memcmp(want.data(), out.ptrPinned().data, want.size() * 4) == 0);
}

// ---- RGB -> YCbCr image: ConvertRGBToYUV, SaturateCast, WriteYUV -----------------------------------------------------
extern "C" int fkb_oracle_rgb_to_ycbcr(uint32_t range, uint32_t primitives, float* ccm2, float* yuv_add);
static void test_write_yuv() {
    Stream stream;
    const uint W = 322, H = 180;
    Ptr2D<uchar3> rgb(W, H);
    fill_random(rgb, 700);
    rgb.upload(stream);
    Image<PixelFormat::NV12> img(W, H);
    executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(rgb),
        ConvertRGBToYUV<ColorDepth::p8bit, ColorRange::Limited, ColorPrimitives::bt601>::build(), SaturateCast<float3, uchar3>::build(),
        WriteYUV<PixelFormat::NV12>::build(img));
    img.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C3; ch.geometry = FKB_GEOM_NONE; ch.dst_format = FKB_PIX_U8C3; ch.write_kind = FKB_WRITE_NV12;
    ch.n_ops = 2; ch.ops[0] = op(FKB_OP_RGB2YUV); ch.ops[1] = op(FKB_OP_SATCAST_U8);
    fkb_oracle_rgb_to_ycbcr(FKB_RANGE_LIMITED, FKB_PRIMITIVES_BT601, ch.ccm2, ch.yuv_add);
    const auto out = img.getData().ptrPinned();
    std::vector<uint8_t> want(static_cast<size_t>(out.dims.pitch) * (H + H / 2), 0);
    fkb_plane_desc d = host_plane(rgb, Rect(0, 0, W, H), W, H, want.data(), out.dims.pitch, ch.geometry);
    d.dst_y = want.data() + static_cast<size_t>(out.dims.pitch) * H;
    fkb_oracle_run(&ch, 1, &d, 1, 1);
    bool same = true;
    for (uint y = 0; y < H + H / 2; ++y)
        same = same && std::memcmp(want.data() + y * out.dims.pitch, reinterpret_cast<const uint8_t*>(out.data) + y * out.dims.pitch, W) == 0;
    report("RGB -> NV12 image (ConvertRGBToYUV, WriteYUV)", same);
}

// ---- batched crop-resize-normalise over several frames --------------------------------------------------------------
template <AspectRatio AR>
static void test_batched(const char* what, uint32_t geometry) {
    Stream stream;
    constexpr size_t FRAMES = 3, PER = 4, BATCH = FRAMES * PER;
    std::vector<Ptr2D<uchar3>> frames;
    for (size_t f = 0; f < FRAMES; ++f) { frames.emplace_back(640, 360); fill_random(frames[f], 100 + f); frames[f].upload(stream); }
    std::array<Ptr2D<uchar3>, BATCH> ptrs;
    std::array<Rect, BATCH> rects;
    std::mt19937 rng(42);
    for (size_t i = 0; i < BATCH; ++i) {
        ptrs[i] = frames[i / PER];
        int x = rng() % 640, y = rng() % 360, w = 8 + rng() % 300, h = 8 + rng() % 300;
        if (x + w > 640) w = 640 - x;
        if (y + h > 360) h = 360 - y;
        rects[i] = Rect(x, y, w, h);
    }
    Tensor<float3> out(96, 80, BATCH);
    executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(ptrs), Crop<>::build(rects),
        Resize<InterpolationType::INTER_LINEAR, AR>::build(Size(96, 80), make_<float3>(114.f, 114.f, 114.f)),
        Mul<float3>::build(make_set<float3>(1.f / 255.f)), TensorWrite<float3>::build(out));
    out.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C3; ch.geometry = geometry; ch.dst_format = FKB_PIX_F32C3; ch.write_kind = FKB_WRITE_PACKED;
    ch.n_ops = 1; ch.ops[0] = op(FKB_OP_MUL, 1.f / 255.f, 1.f / 255.f, 1.f / 255.f);
    std::vector<float> want(96 * 80 * 3 * BATCH);
    std::vector<fkb_plane_desc> planes;
    for (size_t i = 0; i < BATCH; ++i) {
        fkb_plane_desc d = host_plane(ptrs[i], rects[i], 96, 80, want.data() + i * 96 * 80 * 3, 96 * 12, ch.geometry);
        d.bg[0] = d.bg[1] = d.bg[2] = 114.f;
        planes.push_back(d);
    }
    fkb_oracle_run(&ch, 1, planes.data(), BATCH, 1);
    report(what, std::memcmp(want.data(), out.ptrPinned().data, want.size() * 4) == 0);
}

// ---- conditional batch read: planes beyond activeBatch come out as the operations applied to the default value -----
static void test_conditional_batch() {
    Stream stream;
    constexpr size_t BATCH = 6;
    const int used = 4;
    std::array<Ptr2D<uchar3>, BATCH> ptrs;
    for (size_t i = 0; i < BATCH; ++i) { ptrs[i] = Ptr2D<uchar3>(200, 120); fill_random(ptrs[i], 300 + i); ptrs[i].upload(stream); }
    Tensor<float3> out(64, 48, BATCH);
    const uchar3 dflt = make_<uchar3>(9, 250, 77);
    executeOperations<TransformDPP<>>(ptrs, used, dflt, out, stream, Resize<InterpolationType::INTER_LINEAR>::build(Size(64, 48)),
                                      Mul<float3>::build(make_<float3>(0.5f, 2.f, 1.f / 3.f)));
    out.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C3; ch.geometry = FKB_GEOM_RESIZE_IGNORE_AR; ch.dst_format = FKB_PIX_F32C3; ch.write_kind = FKB_WRITE_PACKED;
    ch.n_ops = 1; ch.ops[0] = op(FKB_OP_MUL, 0.5f, 2.f, 1.f / 3.f);
    std::vector<float> want(64 * 48 * 3 * BATCH);
    std::vector<fkb_plane_desc> planes;
    for (size_t i = 0; i < BATCH; ++i) {
        fkb_plane_desc d = host_plane(ptrs[i], Rect(0, 0, 200, 120), 64, 48, want.data() + i * 64 * 48 * 3, 64 * 12, ch.geometry);
        if (static_cast<int>(i) >= used) { d.chain |= FKB_PLANE_DEFAULT; d.bg[0] = 9.f; d.bg[1] = 250.f; d.bg[2] = 77.f; }
        planes.push_back(d);
    }
    fkb_oracle_run(&ch, 1, planes.data(), BATCH, 1);
    report("conditional batch read (activeBatch, defaultValue)", std::memcmp(want.data(), out.ptrPinned().data, want.size() * 4) == 0);
}

// ---- BorderReader: crops that leave the frame -----------------------------------------------------------------------------
template <BorderType BT>
static void test_border(const char* what) {
    Stream stream;
    constexpr size_t BATCH = 3;
    std::array<Ptr2D<uchar3>, BATCH> ptrs;
    for (size_t i = 0; i < BATCH; ++i) { ptrs[i] = Ptr2D<uchar3>(150, 100); fill_random(ptrs[i], 500 + i); ptrs[i].upload(stream); }
    const std::array<Rect, BATCH> rects{Rect(-20, -10, 90, 70), Rect(100, 60, 120, 80), Rect(10, 10, 50, 40)};
    Tensor<float3> out(64, 64, BATCH);
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(ptrs);
    const auto resize = Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(Size(64, 64), make_<float3>(1.f, 2.f, 3.f));
    fkb_chain_desc ch{};
    if constexpr (BT == BorderType::CONSTANT) {
        executeOperations<TransformDPP<>>(stream, BorderReader<BT>::build(read, make_<uchar3>(200, 100, 50)) & Crop<>::build(rects) & resize,
                                          TensorWrite<float3>::build(out));
        ch.border_value[0] = 200.f; ch.border_value[1] = 100.f; ch.border_value[2] = 50.f;
    } else {
        executeOperations<TransformDPP<>>(stream, read, BorderReader<BT>::build(), Crop<>::build(rects), resize, TensorWrite<float3>::build(out));
    }
    out.download(stream);
    stream.sync();
    ch.src_format = FKB_PIX_U8C3; ch.geometry = FKB_GEOM_RESIZE_PRESERVE_AR; ch.dst_format = FKB_PIX_F32C3; ch.write_kind = FKB_WRITE_PACKED;
    ch.border = static_cast<uint32_t>(BT) + 1u;
    std::vector<float> want(64 * 64 * 3 * BATCH);
    std::vector<fkb_plane_desc> planes;
    for (size_t i = 0; i < BATCH; ++i) {
        fkb_plane_desc d = host_plane(ptrs[i], rects[i], 64, 64, want.data() + i * 64 * 64 * 3, 64 * 12, ch.geometry);
        d.bg[0] = 1.f; d.bg[1] = 2.f; d.bg[2] = 3.f;
        planes.push_back(d);
    }
    fkb_oracle_run(&ch, 1, planes.data(), BATCH, 1);
    report(what, std::memcmp(want.data(), out.ptrPinned().data, want.size() * 4) == 0);
}

// ---- a uchar4 (BGRA) frame: crops, resize on float4, alpha discarded with BGRA2RGB, normalise ---------------------------------
static void test_bgra_source() {
    Stream stream;
    Ptr2D<uchar4> input(320, 200);
    {
        const auto h = input.ptrPinned();
        std::mt19937 rng(800);
        for (uint y = 0; y < 200; ++y) for (uint x = 0; x < 320 * 4; ++x) reinterpret_cast<uint8_t*>(h.data)[y * h.dims.pitch + x] = rng() & 255;
    }
    input.upload(stream);
    constexpr size_t BATCH = 3;
    const std::array<Rect, BATCH> crops{Rect(0, 0, 120, 40), Rect(100, 100, 60, 40), Rect(290, 170, 30, 30)};
    Tensor<float3> out(64, 64, BATCH);
    executeOperations<TransformDPP<>>(input, stream, Crop<>::build(crops), Resize<InterpolationType::INTER_LINEAR>::build(Size(64, 64)),
                                      Mul<float4>::build(make_set<float4>(1.f / 255.f)),
                                      ColorConversion<ColorConversionCodes::COLOR_BGRA2RGB, float4, float3>::build(),
                                      Add<float3>::build(make_<float3>(0.5f, 0.25f, 0.125f)), TensorWrite<float3>::build(out));
    out.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C4; ch.geometry = FKB_GEOM_RESIZE_IGNORE_AR; ch.dst_format = FKB_PIX_F32C3; ch.write_kind = FKB_WRITE_PACKED;
    ch.n_ops = 3; ch.ops[0] = op(FKB_OP_MUL, 1.f / 255.f, 1.f / 255.f, 1.f / 255.f); ch.ops[1] = op(FKB_OP_REORDER_ZYX); ch.ops[2] = op(FKB_OP_ADD, 0.5f, 0.25f, 0.125f);
    std::vector<float> want(64 * 64 * 3 * BATCH);
    std::vector<fkb_plane_desc> planes;
    const auto r = input.ptrPinned();
    for (size_t i = 0; i < BATCH; ++i) {
        fkb_plane_desc d{};
        d.src = r.data; d.src_pitch = r.dims.pitch; d.src_w = 320; d.src_h = 200;
        d.crop_x = crops[i].x; d.crop_y = crops[i].y; d.crop_w = crops[i].width; d.crop_h = crops[i].height;
        d.dst = want.data() + i * 64 * 64 * 3; d.dst_w = 64; d.dst_h = 64; d.dst_pitch = 64 * 12;
        fkb_oracle_resize_params(ch.geometry, &d);
        planes.push_back(d);
    }
    fkb_oracle_run(&ch, 1, planes.data(), BATCH, 1);
    report("uchar4 source, alpha discarded (BGRA2RGB)", std::memcmp(want.data(), out.ptrPinned().data, want.size() * 4) == 0);
}

// ---- four channels to the end: the pipeline of the reference's compiler-explorer example ----------------------------------
static void test_four_channels() {
    Stream stream;
    Ptr2D<uchar4> input(1920, 1080);
    {
        const auto h = input.ptrPinned();
        std::mt19937 rng(900);
        for (uint y = 0; y < 1080; ++y) for (uint x = 0; x < 1920 * 4; ++x) reinterpret_cast<uint8_t*>(h.data)[y * h.dims.pitch + x] = rng() & 255;
    }
    input.upload(stream);
    const std::array<Rect, 5> crops{Rect(0, 0, 120, 40), Rect(100, 200, 60, 40), Rect(400, 20, 30, 50), Rect(1000, 800, 30, 30), Rect(40, 40, 40, 40)};
    Tensor<uchar4> output(64, 64, 5);
    executeOperations<TransformDPP<>>(input, stream, Crop<>::build(crops), Resize<InterpolationType::INTER_LINEAR>::build(Size(64, 64)),
                                      Mul<float4>::build(make_set<float4>(1.f / 255.f)), Mul<float4>::build(make_set<float4>(0.33f)),
                                      Add<float4>::build(make_<float4>(0.5f, 0.25f, 0.125f, 0.f)), Mul<float4>::build(make_set<float4>(255.f)),
                                      ColorConversion<ColorConversionCodes::COLOR_BGRA2RGBA, float4, float4>::build(),
                                      SaturateCast<float4, uchar4>::build(), TensorWrite<uchar4>::build(output));
    output.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C4; ch.geometry = FKB_GEOM_RESIZE_IGNORE_AR; ch.dst_format = FKB_PIX_U8C4; ch.write_kind = FKB_WRITE_PACKED;
    ch.n_ops = 6;
    ch.ops[0] = op(FKB_OP_MUL, 1.f / 255.f, 1.f / 255.f, 1.f / 255.f); ch.op_w[0] = 1.f / 255.f;
    ch.ops[1] = op(FKB_OP_MUL, 0.33f, 0.33f, 0.33f); ch.op_w[1] = 0.33f;
    ch.ops[2] = op(FKB_OP_ADD, 0.5f, 0.25f, 0.125f); ch.op_w[2] = 0.f;
    ch.ops[3] = op(FKB_OP_MUL, 255.f, 255.f, 255.f); ch.op_w[3] = 255.f;
    ch.ops[4] = op(FKB_OP_REORDER_ZYX); ch.ops[5] = op(FKB_OP_SATCAST_U8);
    std::vector<uint8_t> want(64 * 64 * 4 * 5);
    std::vector<fkb_plane_desc> planes;
    const auto r = input.ptrPinned();
    for (size_t i = 0; i < 5; ++i) {
        fkb_plane_desc d{};
        d.src = r.data; d.src_pitch = r.dims.pitch; d.src_w = 1920; d.src_h = 1080;
        d.crop_x = crops[i].x; d.crop_y = crops[i].y; d.crop_w = crops[i].width; d.crop_h = crops[i].height;
        d.dst = want.data() + i * 64 * 64 * 4; d.dst_w = 64; d.dst_h = 64; d.dst_pitch = 64 * 4;
        fkb_oracle_resize_params(ch.geometry, &d);
        planes.push_back(d);
    }
    fkb_oracle_run(&ch, 1, planes.data(), 5, 1);
    report("four channels to the Write (uchar4 -> uchar4 tensor)", std::memcmp(want.data(), output.ptrPinned().data, want.size()) == 0);
}

// ---- conversions that append an opaque alpha channel: uchar3 source, uchar4 tensor ---------------------------------------------------
static void test_add_alpha() {
    Stream stream;
    Ptr2D<uchar3> input(640, 360);
    fill_random(input, 901);
    input.upload(stream);
    const std::array<Rect, 3> crops{Rect(0, 0, 120, 40), Rect(100, 200, 60, 40), Rect(400, 20, 30, 50)};
    Tensor<uchar4> output(48, 40, 3);
    executeOperations<TransformDPP<>>(input, stream, Crop<>::build(crops), Resize<InterpolationType::INTER_LINEAR>::build(Size(48, 40)),
                                      Mul<float3>::build(make_<float3>(0.5f, 1.f, 1.5f)),
                                      ColorConversion<ColorConversionCodes::COLOR_BGR2RGBA, float3, float4>::build(),
                                      Mul<float4>::build(make_<float4>(1.f, 0.5f, 0.75f, 0.5f)), SaturateCast<float4, uchar4>::build(),
                                      TensorWrite<uchar4>::build(output));
    output.download(stream);
    Ptr2D<uchar4> image(640, 360);  // and the conversion alone, on byte pixels
    executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(input),
                                      ColorConversion<ColorConversionCodes::COLOR_RGB2RGBA, uchar3, uchar4>::build(),
                                      PerThreadWrite<ND::_2D, uchar4>::build(image));
    image.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C3; ch.geometry = FKB_GEOM_RESIZE_IGNORE_AR; ch.dst_format = FKB_PIX_U8C4; ch.write_kind = FKB_WRITE_PACKED;
    ch.n_ops = 5;
    ch.ops[0] = op(FKB_OP_MUL, 0.5f, 1.f, 1.5f); ch.ops[1] = op(FKB_OP_REORDER_ZYX); ch.ops[2] = op(FKB_OP_ADD_ALPHA, 255.f);
    ch.ops[3] = op(FKB_OP_MUL, 1.f, 0.5f, 0.75f); ch.op_w[3] = 0.5f; ch.ops[4] = op(FKB_OP_SATCAST_U8);
    std::vector<uint8_t> want(48 * 40 * 4 * 3);
    std::vector<fkb_plane_desc> planes;
    for (size_t i = 0; i < 3; ++i) planes.push_back(host_plane(input, crops[i], 48, 40, want.data() + i * 48 * 40 * 4, 48 * 4, ch.geometry));
    fkb_oracle_run(&ch, 1, planes.data(), 3, 1);
    report("BGR2RGBA in a resize chain (uchar3 -> uchar4 tensor)", std::memcmp(want.data(), output.ptrPinned().data, want.size()) == 0);
    fkb_chain_desc pc{};
    pc.src_format = FKB_PIX_U8C3; pc.geometry = FKB_GEOM_NONE; pc.dst_format = FKB_PIX_U8C4; pc.write_kind = FKB_WRITE_PACKED;
    pc.n_ops = 1; pc.ops[0] = op(FKB_OP_ADD_ALPHA, 255.f);
    const auto o = image.ptrPinned();
    std::vector<uint8_t> want2(static_cast<size_t>(o.dims.pitch) * 360, 0);
    fkb_plane_desc d = host_plane(input, Rect(0, 0, 640, 360), 640, 360, want2.data(), o.dims.pitch, pc.geometry);
    fkb_oracle_run(&pc, 1, &d, 1, 1);
    bool same = true;
    for (uint y = 0; y < 360; ++y)
        same = same && std::memcmp(want2.data() + y * o.dims.pitch, reinterpret_cast<const uint8_t*>(o.data) + y * o.dims.pitch, 640 * 4) == 0;
    report("RGB2RGBA on byte pixels (uchar3 -> uchar4 image)", same);
}

// ---- CircularTensor: after n updates plane z holds the chain's result for the z-th newest (or oldest) frame --------------------
template <CircularTensorOrder ORDER, ColorPlanes MODE>
static void test_circular(const char* what) {
    Stream stream;
    constexpr int BATCH = 4, N = 7;
    const uint W = 200, H = 120, DW = 80, DH = 48;
    std::vector<Ptr2D<uchar3>> frames;
    for (int k = 0; k < N; ++k) { frames.emplace_back(W, H); fill_random(frames[k], 1000 + k); frames[k].upload(stream); }
    CircularTensor<float, 3, BATCH, ORDER, MODE> ct(DW, DH);
    const auto resize = Resize<InterpolationType::INTER_LINEAR>::build(Size(DW, DH));
    const auto mul = Mul<float3>::build(make_<float3>(0.5f, 1.f, 2.f));
    for (int k = 0; k < N; ++k) {
        if constexpr (MODE == ColorPlanes::Standard) ct.update(stream, PerThreadRead<ND::_2D, uchar3>::build(frames[k]), resize, mul, TensorSplit<float3>::build(ct.ptr()));
        else ct.update(stream, PerThreadRead<ND::_2D, uchar3>::build(frames[k]), resize, mul, TensorTSplit<float3>::build(ct.ptr()));
    }
    ct.download(stream);
    stream.sync();
    // expected: plane z = the chain on frame N-1-z (newest first) or N-BATCH+z (oldest first), computed one plane at a time
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C3; ch.geometry = FKB_GEOM_RESIZE_IGNORE_AR; ch.dst_format = FKB_PIX_F32C3; ch.write_kind = FKB_WRITE_SPLIT;
    ch.n_ops = 1; ch.ops[0] = op(FKB_OP_MUL, 0.5f, 1.f, 2.f);
    const size_t px = static_cast<size_t>(DW) * DH;
    bool same = true;
    for (int z = 0; z < BATCH; ++z) {
        const int k = ORDER == CircularTensorOrder::NewestFirst ? N - 1 - z : N - BATCH + z;
        std::vector<float> want(px * 3);
        fkb_plane_desc d = host_plane(frames[k], Rect(0, 0, W, H), DW, DH, want.data(), DW * 4, ch.geometry);
        d.dst_channel_stride = px * 4;
        fkb_oracle_run(&ch, 1, &d, 1, 1);
        const float* got = ct.ptrPinned().data;
        for (int c = 0; c < 3; ++c) {
            const float* g = MODE == ColorPlanes::Standard ? got + (static_cast<size_t>(z) * 3 + c) * px : got + (static_cast<size_t>(c) * BATCH + z) * px;
            same = same && std::memcmp(want.data() + c * px, g, px * 4) == 0;
        }
    }
    report(what, same);
}
static void test_circular_packed() {
    Stream stream;
    constexpr int BATCH = 3, N = 5;
    const uint W = 160, H = 90, DW = 64, DH = 40;
    std::vector<Ptr2D<uchar3>> frames;
    for (int k = 0; k < N; ++k) { frames.emplace_back(W, H); fill_random(frames[k], 1100 + k); frames[k].upload(stream); }
    CircularTensor<float3, 1, BATCH, CircularTensorOrder::NewestFirst, ColorPlanes::Standard> ct(DW, DH);
    for (int k = 0; k < N; ++k)
        ct.update(stream, PerThreadRead<ND::_2D, uchar3>::build(frames[k]), Resize<InterpolationType::INTER_LINEAR>::build(Size(DW, DH)),
                  Mul<float3>::build(make_<float3>(2.f, 1.f, 0.5f)), TensorWrite<float3>::build(ct.ptr()));
    ct.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C3; ch.geometry = FKB_GEOM_RESIZE_IGNORE_AR; ch.dst_format = FKB_PIX_F32C3; ch.write_kind = FKB_WRITE_PACKED;
    ch.n_ops = 1; ch.ops[0] = op(FKB_OP_MUL, 2.f, 1.f, 0.5f);
    const size_t px = static_cast<size_t>(DW) * DH;
    bool same = true;
    for (int z = 0; z < BATCH; ++z) {
        std::vector<float> want(px * 3);
        fkb_plane_desc d = host_plane(frames[N - 1 - z], Rect(0, 0, W, H), DW, DH, want.data(), DW * 12, ch.geometry);
        fkb_oracle_run(&ch, 1, &d, 1, 1);
        same = same && std::memcmp(want.data(), reinterpret_cast<const float*>(ct.ptrPinned().data) + z * px * 3, px * 12) == 0;
    }
    report("CircularTensor<float3, 1, 3, NewestFirst> (packed)", same);
}

// ---- transposed planar tensor: TensorTSplit<float3> ---------------------------------------------------------------------
static void test_tensor_t_split() {
    Stream stream;
    constexpr size_t BATCH = 3;
    std::array<Ptr2D<uchar3>, BATCH> ptrs;
    for (size_t i = 0; i < BATCH; ++i) { ptrs[i] = Ptr2D<uchar3>(160, 90); fill_random(ptrs[i], 400 + i); ptrs[i].upload(stream); }
    TensorT<float> out(80, 40, BATCH, 3);
    executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(ptrs), Resize<InterpolationType::INTER_LINEAR>::build(Size(80, 40)),
                                      Mul<float3>::build(make_<float3>(2.f, 0.5f, 1.f)), TensorTSplit<float3>::build(out));
    out.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C3; ch.geometry = FKB_GEOM_RESIZE_IGNORE_AR; ch.dst_format = FKB_PIX_F32C3; ch.write_kind = FKB_WRITE_SPLIT;
    ch.n_ops = 1; ch.ops[0] = op(FKB_OP_MUL, 2.f, 0.5f, 1.f);
    const size_t plane = 80 * 40;
    std::vector<float> want(plane * 3 * BATCH);
    std::vector<fkb_plane_desc> planes;
    for (size_t i = 0; i < BATCH; ++i) {
        fkb_plane_desc d = host_plane(ptrs[i], Rect(0, 0, 160, 90), 80, 40, want.data() + i * plane, 80 * 4, ch.geometry);
        d.dst_channel_stride = plane * BATCH * 4;  // all first channels, then all second ones, ...
        planes.push_back(d);
    }
    fkb_oracle_run(&ch, 1, planes.data(), BATCH, 1);
    report("TensorTSplit<float3> (transposed planar tensor)", std::memcmp(want.data(), out.ptrPinned().data, want.size() * 4) == 0);
}

// ---- SplitWrite: three separate planes ------------------------------------------------------------------------------------
static void test_split_write() {
    Stream stream;
    Ptr2D<uchar3> in(200, 120);
    fill_random(in, 600);
    in.upload(stream);
    std::vector<Ptr2D<float>> out{Ptr2D<float>(90, 50), Ptr2D<float>(90, 50), Ptr2D<float>(90, 50)};
    executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(in), Resize<InterpolationType::INTER_LINEAR>::build(Size(90, 50)),
                                      Mul<float3>::build(make_<float3>(1.f, 2.f, 3.f)), SplitWrite<ND::_2D, float3>::build(out));
    for (auto& p : out) p.download(stream);
    stream.sync();
    fkb_chain_desc ch{};
    ch.src_format = FKB_PIX_U8C3; ch.geometry = FKB_GEOM_RESIZE_IGNORE_AR; ch.dst_format = FKB_PIX_F32C3; ch.write_kind = FKB_WRITE_SPLIT_PLANES;
    ch.n_ops = 1; ch.ops[0] = op(FKB_OP_MUL, 1.f, 2.f, 3.f);
    const uint32_t pitch = out[0].dims().pitch;
    std::vector<uint8_t> wx(pitch * 50), wy(pitch * 50), wz(pitch * 50);
    fkb_plane_desc d = host_plane(in, Rect(0, 0, 200, 120), 90, 50, wx.data(), pitch, ch.geometry);
    d.dst_y = wy.data(); d.dst_z = wz.data();
    fkb_oracle_run(&ch, 1, &d, 1, 1);
    bool same = true;
    const std::vector<uint8_t>* want[3] = {&wx, &wy, &wz};
    for (int c = 0; c < 3; ++c)
        for (int y = 0; y < 50; ++y)
            same = same && std::memcmp(want[c]->data() + y * pitch, reinterpret_cast<const uint8_t*>(out[c].ptrPinned().data) + y * pitch, 90 * 4) == 0;
    report("SplitWrite<ND::_2D, float3> (three planes)", same);
}

// ---- divergent horizontal fusion: two sequences in one launch, global plane indices ------------------------------------
struct Sel { static uint at(const uint& z) { return z < 2 ? 0u : 1u; } };
static void test_divergent() {
    Stream stream;
    const uint W = 320, H = 180;
    std::array<Ptr2D<uchar3>, 4> frames;
    for (int f = 0; f < 4; ++f) { frames[f] = Ptr2D<uchar3>(W, H); fill_random(frames[f], 7 + f); frames[f].upload(stream); }
    std::array<Ptr2D<uchar3>, 2> first2{frames[0], frames[1]};
    Tensor<uchar3> outA(W / 2, H / 2, 2);
    const auto seq0 = buildOperationSequence(PerThreadRead<ND::_2D, uchar3>::build(first2),
        Resize<InterpolationType::INTER_LINEAR>::build(Size(W / 2, H / 2)), SaturateCast<float3, uchar3>::build(), TensorWrite<uchar3>::build(outA));
    using FusedRead = decltype(PerThreadRead<ND::_2D, uchar3>::build(frames[0]).then(Cast<uchar3, float3>::build())
        .then(Mul<float3>::build(make_set<float3>(1.f))).then(Sub<float3>::build(make_set<float3>(0.f))));
    std::array<FusedRead, 4> reads;
    const float scales[4] = {0.f, 0.f, 0.75f, 1.9f}, offs[4] = {0.f, 0.f, 13.5f, 60.f};
    for (int i = 0; i < 4; ++i)
        reads[i] = PerThreadRead<ND::_2D, uchar3>::build(frames[i < 2 ? 2 : i]).then(Cast<uchar3, float3>::build())
            .then(Mul<float3>::build(make_set<float3>(scales[i]))).then(Sub<float3>::build(make_set<float3>(offs[i])));
    auto batchRead = BatchRead<PlanePolicy::PROCESS_ALL>::build(reads);
    batchRead.params.activeThreads.z = 2;  // this sequence owns planes 2 and 3; indices stay global
    Tensor<float3> outB(W, H, 4);
    std::memset(outB.ptrPinned().data, 0, outB.sizeInBytes());
    outB.upload(stream);
    const auto seq1 = buildOperationSequence(batchRead, TensorWrite<float3>::build(outB));
    Executor<DivergentBatchTransformDPP<ParArch::GPU_NVIDIA, Sel>>::executeOperations(stream, seq0, seq1);
    outA.download(stream); outB.download(stream);
    stream.sync();
    bool ok = true;
    for (uint z = 0; z < 2; ++z)  // scale exactly 2: the even-pixel subsample
        for (uint y = 0; y < H / 2; ++y) for (uint x = 0; x < W / 2; ++x) {
            const uchar3 a = outA.at(x, y, z), b = frames[z].at(2 * x, 2 * y);
            ok = ok && a.x == b.x && a.y == b.y && a.z == b.z;
        }
    for (uint z = 2; z < 4; ++z)
        for (uint y = 0; y < H; ++y) for (uint x = 0; x < W; ++x) {
            const float3 a = outB.at(x, y, z); const uchar3 b = frames[z].at(x, y);
            ok = ok && a.x == b.x * scales[z] - offs[z] && a.y == b.y * scales[z] - offs[z] && a.z == b.z * scales[z] - offs[z];
        }
    const float3 untouched = outB.at(5, 5, 0);
    report("divergent batch (two sequences)", ok && untouched.x == 0.f);
}

// ---- error behaviour: a bad launch throws std::runtime_error, like the reference's gpuErrchk -------------------------
static void test_errors() {
    Stream stream;
    Ptr2D<uchar3> in(64, 48);
    Tensor<uchar3> out(32, 32, 1);
    bool threw = false;
    try {
        executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(in), Crop<>::build(Rect(60, 40, 32, 32)),
            Resize<InterpolationType::INTER_LINEAR>::build(Size(32, 32)), SaturateCast<float3, uchar3>::build(), TensorWrite<uchar3>::build(out));
    } catch (const std::runtime_error&) { threw = true; }
    report("rectangle outside the frame throws", threw);
    threw = false;
    try { Ptr2D<uchar3> bad(0, 10); } catch (const std::runtime_error&) { threw = true; }
    report("zero-sized Ptr2D throws", threw);
}

int main() {
    test_readme();
    test_vertical_fusion();
    test_thread_fusion();
    test_gray();
    test_nv12();
    test_yuv<PixelFormat::NV21, ColorRange::Limited, ColorPrimitives::bt601>("NV21, limited range bt601", FKB_PIX_NV21, FKB_RANGE_LIMITED, FKB_PRIMITIVES_BT601);
    test_yuv<PixelFormat::UYVY, ColorRange::Full, ColorPrimitives::bt2020>("UYVY, full range bt2020", FKB_PIX_UYVY, FKB_RANGE_FULL, FKB_PRIMITIVES_BT2020);
    test_yuv<PixelFormat::NV12, ColorRange::Limited, ColorPrimitives::bt709>("NV12, limited range bt709", FKB_PIX_NV12, FKB_RANGE_LIMITED, FKB_PRIMITIVES_BT709);
    test_yuv<PixelFormat::P010, ColorRange::Limited, ColorPrimitives::bt2020>("P010, limited range bt2020", FKB_PIX_P010, FKB_RANGE_LIMITED, FKB_PRIMITIVES_BT2020);
    test_yuv<PixelFormat::P210, ColorRange::Full, ColorPrimitives::bt709>("P210, full range bt709", FKB_PIX_P210, FKB_RANGE_FULL, FKB_PRIMITIVES_BT709);
    test_yuv<PixelFormat::Y210, ColorRange::Limited, ColorPrimitives::bt601>("Y210, limited range bt601", FKB_PIX_Y210, FKB_RANGE_LIMITED, FKB_PRIMITIVES_BT601);
    test_batched<AspectRatio::PRESERVE_AR>("batched crop-resize-normalise", FKB_GEOM_RESIZE_PRESERVE_AR);
    test_batched<AspectRatio::PRESERVE_AR_RN_EVEN>("batched crop-resize-normalise, PRESERVE_AR_RN_EVEN", FKB_GEOM_RESIZE_PRESERVE_AR_RN_EVEN);
    test_batched<AspectRatio::PRESERVE_AR_LEFT>("batched crop-resize-normalise, PRESERVE_AR_LEFT", FKB_GEOM_RESIZE_PRESERVE_AR_LEFT);
    test_conditional_batch();
    test_tensor_t_split();
    test_circular<CircularTensorOrder::NewestFirst, ColorPlanes::Standard>("CircularTensor<float, 3, 4, NewestFirst, Standard>");
    test_circular<CircularTensorOrder::OldestFirst, ColorPlanes::Standard>("CircularTensor<float, 3, 4, OldestFirst, Standard>");
    test_circular<CircularTensorOrder::NewestFirst, ColorPlanes::Transposed>("CircularTensor<float, 3, 4, NewestFirst, Transposed>");
    test_circular<CircularTensorOrder::OldestFirst, ColorPlanes::Transposed>("CircularTensor<float, 3, 4, OldestFirst, Transposed>");
    test_circular_packed();
    test_bgra_source();
    test_four_channels();
    test_add_alpha();
    test_write_yuv();
    test_split_write();
    test_border<BorderType::CONSTANT>("BorderReader<CONSTANT> (complete form, operator&)");
    test_border<BorderType::REPLICATE>("BorderReader<REPLICATE>");
    test_border<BorderType::REFLECT_101>("BorderReader<REFLECT_101>");
    test_border<BorderType::WRAP>("BorderReader<WRAP>");
    test_divergent();
    test_errors();
    std::printf("%s\n", g_failed ? "FAILED" : "ALL PASSED");
    return g_failed ? 1 : 0;
}
