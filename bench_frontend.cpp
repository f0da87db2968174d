// Host cost of one launch through the fk:: front end, for bench.py.
//
// Builds the batched crop -> resize -> normalise launch of the benchmark (64 frames of 1920x1080 uchar3, 32 crops each,
// 224x224 float3 tensor of 2048 planes) with the front end's own API, exactly as a user of the reference would write it,
// and times the synchronous part of fk::executeOperations<TransformDPP<>> — building the IOps, folding them, lowering
// them to plane descriptors, fkb_launch_transform's own lowering and the copy of the plane table — with the GPU idle
// before every call.  Prints one JSON object.  The reference's documentation quotes 19-70 us per call for its generated
// bindings in steady state (.github/skills/fkl-language-bindings/SKILL.md:90).
#include <array>
#include <chrono>
#include <cstdio>
#include <memory>
#include <random>
#include <vector>

#include <fused_kernel/algorithms/basic_ops/arithmetic.h>
#include <fused_kernel/algorithms/basic_ops/memory_operations.h>
#include <fused_kernel/algorithms/image_processing/crop.h>
#include <fused_kernel/algorithms/image_processing/resize.h>
#include <fused_kernel/fused_kernel.h>

using namespace fk;

int main(int argc, char** argv) {
    constexpr size_t FRAMES = 64, PER = 32, BATCH = FRAMES * PER;
    const int calls = argc > 1 ? std::atoi(argv[1]) : 30;
    try {
        Stream stream;
        std::vector<Ptr2D<uchar3>> frames;
        for (size_t f = 0; f < FRAMES; ++f) frames.emplace_back(1920u, 1080u, 0u, MemType::Device);
        auto ptrs = std::make_unique<std::array<Ptr2D<uchar3>, BATCH>>();
        auto rects = std::make_unique<std::array<Rect, BATCH>>();
        std::mt19937 rng(4);
        for (size_t i = 0; i < BATCH; ++i) {
            (*ptrs)[i] = frames[i / PER];
            int x = rng() % 1920, y = rng() % 1080, w = 16 + rng() % 497, h = 16 + rng() % 497;
            if (x + w > 1920) w = 1920 - x;
            if (y + h > 1080) h = 1080 - y;
            (*rects)[i] = Rect(x, y, w, h);
        }
        Tensor<float3> out(224, 224, BATCH, 1, MemType::Device);
        auto call = [&]() {
            executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(*ptrs), Crop<>::build(*rects),
                Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(Size(224, 224), make_<float3>(114.f, 114.f, 114.f)),
                Mul<float3>::build(make_set<float3>(1.f / 255.f)), TensorWrite<float3>::build(out));
        };
        for (int i = 0; i < 3; ++i) { call(); stream.sync(); }
        std::vector<double> us;
        for (int i = 0; i < calls; ++i) {
            const auto t0 = std::chrono::steady_clock::now();
            call();
            const auto t1 = std::chrono::steady_clock::now();
            stream.sync();
            us.push_back(std::chrono::duration<double, std::micro>(t1 - t0).count());
        }
        std::sort(us.begin(), us.end());
        std::printf("{\"planes\": %zu, \"calls\": %d, \"median_us\": %.2f, \"min_us\": %.2f, \"max_us\": %.2f}\n", BATCH, calls,
                    us[us.size() / 2], us.front(), us.back());
    } catch (const std::exception& e) {
        std::printf("{\"error\": \"%s\"}\n", e.what());
        return 1;
    }
    return 0;
}
