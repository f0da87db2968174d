// Front end of the B200 kernels, part 1: plain data types with the spellings of FusedKernelLibrary's user API.
//
// This is not the reference's template machinery: the reference turns a list of IOps into one variadic-template
// kernel; here an IOp is a small value that knows how to append itself to a run-time chain descriptor
// (include/fkb/fkb.h).  The names, argument meanings and error behaviour of the user-facing pieces follow the
// reference so that a program written against its API for the supported chains compiles unchanged.
//   ND, PtrDims, RawPtr ........ core/data/rawptr.h:22-141
//   Point / Size / Rect ........ core/data/point.h:36-43, core/data/size.h, core/data/rect.h:23-32
//   MemType .................... core/data/ptr_nd.h:29-34
//   ParArch, defaultParArch .... core/execution_model/parallel_architectures.h:23-54
//   make_<T>, make_set<T> ...... core/utils/vector_utils.h:186-298
//   gpuErrchk .................. core/utils/utils.h:100-114 (throws std::runtime_error)
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <type_traits>

namespace fk {

using uchar = unsigned char;
using ushort = unsigned short;
using uint = unsigned int;

inline void gpuAssert(cudaError_t code, const char* file, int line) {
    if (code != cudaSuccess)
        throw std::runtime_error(std::string("GPU Error: ") + cudaGetErrorString(code) + " File: " + file + " Line: " + std::to_string(line));
}
#define gpuErrchk(ans) ::fk::gpuAssert((ans), __FILE__, __LINE__)

enum class ND { _1D = 1, _2D = 2, _3D = 3, T3D = 4 };  // core/data/ptr_nd.h: T3D is the colour-plane-transposed tensor
enum class MemType { Device, Host, HostPinned, DeviceAndPinned };
constexpr MemType defaultMemType = MemType::DeviceAndPinned;
// Only the NVIDIA GPU architecture is executable here; the other enumerators exist so that user code naming them still
// compiles up to the point where it asks for execution (a static_assert names the restriction).
enum class ParArch { CPU, GPU_NVIDIA, GPU_NVIDIA_JIT, GPU_AMD, CPU_OMP, CPU_OMPSS, MULTI_GPU_NVIDIA, CLUSTER_GPU_NVIDIA };
constexpr ParArch defaultParArch = ParArch::GPU_NVIDIA;
enum class TF { DISABLED = 0, ENABLED = 1 };

struct Point {
    int x{0}, y{0}, z{0};
    constexpr Point() = default;
    constexpr Point(int x_, int y_ = 0, int z_ = 0) : x(x_), y(y_), z(z_) {}
};
struct Size {
    int width{0}, height{0};
    constexpr Size() = default;
    constexpr Size(int w, int h) : width(w), height(h) {}
};
struct Rect {
    uint x{0}, y{0};
    int width{0}, height{0};
    constexpr Rect() = default;
    constexpr Rect(uint x_, uint y_, int w, int h) : x(x_), y(y_), width(w), height(h) {}
};
struct ActiveThreads {
    uint x{1}, y{1}, z{1};
};

// channel count and base type of the CUDA vector types this front end handles
template <typename T> struct VectorTraits { using base = T; static constexpr int cn = 1; };
template <> struct VectorTraits<uchar3> { using base = uchar; static constexpr int cn = 3; };
template <> struct VectorTraits<ushort3> { using base = ushort; static constexpr int cn = 3; };
template <> struct VectorTraits<float3> { using base = float; static constexpr int cn = 3; };
template <> struct VectorTraits<uchar2> { using base = uchar; static constexpr int cn = 2; };
template <> struct VectorTraits<uchar4> { using base = uchar; static constexpr int cn = 4; };
template <> struct VectorTraits<float4> { using base = float; static constexpr int cn = 4; };
template <typename T> using VBase = typename VectorTraits<T>::base;
template <typename T> constexpr int cn = VectorTraits<T>::cn;

template <typename T, typename... A>
constexpr T make_(A... a) { return T{static_cast<VBase<T>>(a)...}; }
template <typename T>
constexpr T make_set(VBase<T> v) {
    if constexpr (cn<T> == 4) return T{v, v, v, v};
    else if constexpr (cn<T> == 3) return T{v, v, v};
    else if constexpr (cn<T> == 2) return T{v, v};
    else return T{v};
}

template <ND D> struct PtrDims;
template <> struct PtrDims<ND::_2D> {
    uint width{0}, height{0}, pitch{0};
    constexpr PtrDims() = default;
    constexpr PtrDims(uint w, uint h, uint p = 0) : width(w), height(h), pitch(p) {}
};
template <> struct PtrDims<ND::_3D> {
    uint width{0}, height{0}, planes{0}, color_planes{0}, pitch{0}, plane_pitch{0};
    constexpr PtrDims() = default;
    constexpr PtrDims(uint w, uint h, uint planes_, uint color_planes_ = 1, uint p = 0)
        : width(w), height(h), planes(planes_), color_planes(color_planes_), pitch(p), plane_pitch(p * h) {}
};
// Colour-plane-transposed batch (core/data/rawptr.h:76-104): all first channels of all images, then all second ones, ...
template <> struct PtrDims<ND::T3D> {
    uint width{0}, height{0}, planes{0}, color_planes{0}, pitch{0}, plane_pitch{0}, color_planes_pitch{0};
    constexpr PtrDims() = default;
    constexpr PtrDims(uint w, uint h, uint planes_, uint color_planes_ = 1)
        : width(w), height(h), planes(planes_), color_planes(color_planes_) {}
};
template <ND D, typename T>
struct RawPtr {
    T* data{nullptr};
    PtrDims<D> dims;
    using type = T;
    static constexpr ND ND_VALUE = D;
};

}  // namespace fk
