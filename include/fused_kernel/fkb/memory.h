// Front end, part 2: streams and owning buffers.
//   Stream_<PA> ............. core/execution_model/stream.h:51-126 (owning / non-owning; the destructor of an owning
//                             stream synchronises)
//   Ptr / Ptr2D / Tensor .... core/data/ptr_nd.h:134-694: reference-counted; 2-D device buffers come from
//                             cudaMallocPitch (the pitch may be padded), tensors are dense (pitch = width*sizeof(T));
//                             the default MemType keeps a pinned host mirror of the same geometry; upload()/download()
//                             are asynchronous copies on the given stream; at() addresses the host side
//   Image<PixelFormat> ...... algorithms/image_processing/image.h:24-95 (NV12: one buffer of w x 1.5h bytes)
//   RawImage ................ algorithms/image_processing/raw_image.h:23-29
// Layout contract (core/data/rawptr.h:203-226): element (x,y) of a 2-D buffer is at data + y*pitch + x*sizeof(T);
// element (x,y,z) of a tensor at data + z*plane_pitch*color_planes + y*pitch + x*sizeof(T), pitches in bytes.
#pragma once
#include <cstdlib>
#include <memory>

#include "types.h"
#include "fkb/fkb.h"

namespace fk {

template <ParArch PA> class Stream_;

template <>
class Stream_<ParArch::GPU_NVIDIA> {
    struct Owned {
        cudaStream_t s{};
        ~Owned() {
            if (s) { cudaStreamSynchronize(s); cudaStreamDestroy(s); }
        }
    };
    cudaStream_t m_stream{};
    std::shared_ptr<Owned> m_owned;  // copies of an owning stream share it; the last one syncs and destroys

public:
    Stream_() : m_owned(std::make_shared<Owned>()) {
        gpuErrchk(cudaStreamCreate(&m_owned->s));
        m_stream = m_owned->s;
    }
    explicit Stream_(const cudaStream_t& stream) : m_stream(stream) {}
    Stream_(const Stream_&) = default;
    Stream_& operator=(const Stream_&) = default;
    cudaStream_t operator()() const { return m_stream; }
    operator cudaStream_t() const { return m_stream; }
    cudaStream_t getCUDAStream() const { return m_stream; }
    void sync() { gpuErrchk(cudaStreamSynchronize(m_stream)); }
    constexpr ParArch getParArch() const { return ParArch::GPU_NVIDIA; }
    static constexpr ParArch parArch() { return ParArch::GPU_NVIDIA; }
};
// Declaring a CPU stream compiles (programs written for both back ends do), executing on it does not: the executors
// accept ParArch::GPU_NVIDIA only.
template <>
class Stream_<ParArch::CPU> {
public:
    void sync() {}
    constexpr ParArch getParArch() const { return ParArch::CPU; }
    static constexpr ParArch parArch() { return ParArch::CPU; }
};
using Stream = Stream_<defaultParArch>;

namespace detail {
struct Allocation {
    void* device{nullptr};
    void* host{nullptr};
    MemType type{MemType::Host};
    bool owns{false};
    int deviceID{0};
    ~Allocation() {
        if (!owns) return;
        if (device && type != MemType::Host && type != MemType::HostPinned) cudaFree(device);
        if (host) {
            if (type == MemType::Host) std::free(host); else cudaFreeHost(host);
        }
    }
};
}  // namespace detail

template <ND D, typename T>
class Ptr {
protected:
    std::shared_ptr<detail::Allocation> m_alloc;
    RawPtr<D, T> ptr_a;       // the pointer kernels use (device memory, or host memory for the Host types)
    RawPtr<D, T> ptr_pinned;  // the host side
    MemType type{defaultMemType};
    int deviceID{0};

    size_t bytes() const {
        if constexpr (D == ND::_2D) return static_cast<size_t>(ptr_a.dims.pitch) * ptr_a.dims.height;
        else if constexpr (D == ND::T3D) return static_cast<size_t>(ptr_a.dims.color_planes_pitch) * ptr_a.dims.color_planes;
        else return static_cast<size_t>(ptr_a.dims.plane_pitch) * ptr_a.dims.planes * ptr_a.dims.color_planes;
    }

public:
    using Type = T;
    static constexpr ND nd = D;
    Ptr() = default;
    Ptr(const PtrDims<D>& dims, const MemType& type_ = defaultMemType, const int& deviceID_ = 0) { allocPtr(dims, type_, deviceID_); }
    // wraps memory owned by the caller (non-owning, as in the reference)
    Ptr(T* data_, const PtrDims<D>& dims, const MemType& type_, const int& deviceID_) {
        if (type_ == MemType::DeviceAndPinned)
            throw std::runtime_error("DeviceAndPinned type requires an additional argument for the pinned pointer.");
        ptr_a.data = data_; ptr_a.dims = dims; ptr_pinned = ptr_a; type = type_; deviceID = deviceID_;
    }

    void allocPtr(const PtrDims<D>& dims_, const MemType& type_ = defaultMemType, const int& deviceID_ = 0) {
        if (dims_.width == 0 || dims_.height == 0) throw std::runtime_error("Width and Height can't be 0");
        m_alloc = std::make_shared<detail::Allocation>();
        m_alloc->type = type_; m_alloc->owns = true; m_alloc->deviceID = deviceID_;
        type = type_; deviceID = deviceID_;
        PtrDims<D> dims = dims_;
        const bool on_device = type_ == MemType::Device || type_ == MemType::DeviceAndPinned;
        if (on_device) gpuErrchk(cudaSetDevice(deviceID_));
        if constexpr (D == ND::_2D) {
            if (on_device && dims.pitch == 0) {
                size_t pitch = 0;
                gpuErrchk(cudaMallocPitch(&m_alloc->device, &pitch, sizeof(T) * dims.width, dims.height));
                dims.pitch = static_cast<uint>(pitch);
            } else {
                if (dims.pitch == 0) dims.pitch = sizeof(T) * dims.width;
                if (on_device) gpuErrchk(cudaMalloc(&m_alloc->device, static_cast<size_t>(dims.pitch) * dims.height));
            }
        } else {
            if (dims.pitch == 0) dims.pitch = sizeof(T) * dims.width;
            dims.plane_pitch = dims.pitch * dims.height;
            if constexpr (D == ND::T3D) dims.color_planes_pitch = dims.plane_pitch * dims.planes;  // ptr_nd.h:119-125
            if (on_device) gpuErrchk(cudaMalloc(&m_alloc->device, static_cast<size_t>(dims.plane_pitch) * dims.planes * dims.color_planes));
        }
        ptr_a.dims = dims;
        const size_t n = bytes();
        if (type_ == MemType::Host) { m_alloc->host = std::malloc(n); if (!m_alloc->host) throw std::bad_alloc(); }
        else if (type_ != MemType::Device) gpuErrchk(cudaMallocHost(&m_alloc->host, n));
        ptr_a.data = static_cast<T*>(on_device ? m_alloc->device : m_alloc->host);
        ptr_pinned.data = static_cast<T*>(m_alloc->host);
        ptr_pinned.dims = dims;
    }

    RawPtr<D, T> ptr() const { return ptr_a; }
    RawPtr<D, T> ptrPinned() const { return ptr_pinned; }
    operator RawPtr<D, T>() const { return ptr_a; }
    PtrDims<D> dims() const { return ptr_a.dims; }
    MemType getMemType() const { return type; }
    int getDeviceID() const { return deviceID; }
    size_t sizeInBytes() const { return bytes(); }

    // host-side element access (the pinned mirror, or the buffer itself for the host types)
    T& at(uint x, uint y = 0, uint z = 0) const {
        if (!ptr_pinned.data) throw std::runtime_error("This Ptr has no host side to index");
        char* base = reinterpret_cast<char*>(ptr_pinned.data);
        if constexpr (D == ND::_3D) base += static_cast<size_t>(z) * ptr_pinned.dims.plane_pitch * ptr_pinned.dims.color_planes;
        if constexpr (D == ND::T3D) base += static_cast<size_t>(z) * ptr_pinned.dims.plane_pitch;  // colour plane 0
        return *(reinterpret_cast<T*>(base + static_cast<size_t>(y) * ptr_pinned.dims.pitch) + x);
    }
    T& at(const Point& p) const { return at(p.x, p.y, p.z); }

    void upload(Stream_<ParArch::GPU_NVIDIA>& stream) {
        if (type == MemType::DeviceAndPinned)
            gpuErrchk(cudaMemcpyAsync(ptr_a.data, ptr_pinned.data, bytes(), cudaMemcpyHostToDevice, stream.getCUDAStream()));
    }
    void download(Stream_<ParArch::GPU_NVIDIA>& stream) {
        if (type == MemType::DeviceAndPinned)
            gpuErrchk(cudaMemcpyAsync(ptr_pinned.data, ptr_a.data, bytes(), cudaMemcpyDeviceToHost, stream.getCUDAStream()));
    }
};

template <typename T>
class Ptr2D : public Ptr<ND::_2D, T> {
public:
    Ptr2D() = default;
    Ptr2D(const Size& size, const uint& pitch_ = 0, const MemType& type_ = defaultMemType, const int& deviceID_ = 0)
        : Ptr<ND::_2D, T>(PtrDims<ND::_2D>(size.width, size.height, pitch_), type_, deviceID_) {}
    Ptr2D(const uint& width_, const uint& height_, const uint& pitch_ = 0, const MemType& type_ = defaultMemType, const int& deviceID_ = 0)
        : Ptr<ND::_2D, T>(PtrDims<ND::_2D>(width_, height_, pitch_), type_, deviceID_) {}
    Ptr2D(const Ptr<ND::_2D, T>& other) : Ptr<ND::_2D, T>(other) {}
    Ptr2D(T* data_, const uint& width_, const uint& height_, const uint& pitch_, const MemType& type_ = defaultMemType, const int& deviceID_ = 0)
        : Ptr<ND::_2D, T>(data_, PtrDims<ND::_2D>(width_, height_, pitch_), type_, deviceID_) {}
};

template <typename T>
class Tensor : public Ptr<ND::_3D, T> {
public:
    Tensor() = default;
    Tensor(const uint& width_, const uint& height_, const uint& planes_, const uint& color_planes_ = 1,
           const MemType& type_ = defaultMemType, const int& deviceID_ = 0)
        : Ptr<ND::_3D, T>(PtrDims<ND::_3D>(width_, height_, planes_, color_planes_, sizeof(T) * width_), type_, deviceID_) {}
    Tensor(T* data, const uint& width_, const uint& height_, const uint& planes_, const uint& color_planes_ = 1,
           const MemType& type_ = defaultMemType, const int& deviceID_ = 0)
        : Ptr<ND::_3D, T>(data, PtrDims<ND::_3D>(width_, height_, planes_, color_planes_, sizeof(T) * width_), type_, deviceID_) {}
};

// A colour-plane-transposed tensor (core/data/ptr_nd.h:696-714)
template <typename T>
class TensorT : public Ptr<ND::T3D, T> {
    static PtrDims<ND::T3D> wrapped(uint w, uint h, uint planes, uint color_planes) {
        PtrDims<ND::T3D> d(w, h, planes, color_planes);
        d.pitch = sizeof(T) * w; d.plane_pitch = d.pitch * h; d.color_planes_pitch = d.plane_pitch * planes;
        return d;
    }
public:
    TensorT() = default;
    TensorT(const uint& width_, const uint& height_, const uint& planes_, const uint& color_planes_ = 1,
            const MemType& type_ = defaultMemType, const int& deviceID_ = 0)
        : Ptr<ND::T3D, T>(PtrDims<ND::T3D>(width_, height_, planes_, color_planes_), type_, deviceID_) {}
    TensorT(T* data, const uint& width_, const uint& height_, const uint& planes_, const uint& color_planes_ = 1,
            const MemType& type_ = defaultMemType, const int& deviceID_ = 0)
        : Ptr<ND::T3D, T>(data, wrapped(width_, height_, planes_, color_planes_), type_, deviceID_) {}
};

// The reference's enumerators (itu_color.h:30, 53).  These kernels read the 8-bit formats NV12, NV21 and UYVY and the
// 10-bit formats P010, P210 and Y210 (ushort samples holding 0..1023).
enum class PixelFormat { NV12, NV21, YV12, P010, P016, P216, P210, Y216, Y210, Y416, UYVY };
enum class ColorDepth { p8bit, p10bit, p12bit, fn8bit, fn10bit, fn12bit };
enum class ColorRange { Limited, Full };
enum class ColorPrimitives { bt601, bt709, bt2020 };

// Depth, sample type and buffer shape of a format (PixelFormatTraits, itu_color.h:57-102): `wf` samples per pixel along
// a row; the one buffer holds `h`, `h + h/2` (4:2:0 semi-planar) or `2h` (4:2:2 semi-planar) rows.
template <PixelFormat PF>
struct PixelFormatTraits {
    static constexpr bool supported = PF == PixelFormat::NV12 || PF == PixelFormat::NV21 || PF == PixelFormat::UYVY ||
                                      PF == PixelFormat::P010 || PF == PixelFormat::P210 || PF == PixelFormat::Y210;
    static constexpr bool wide = PF == PixelFormat::P010 || PF == PixelFormat::P210 || PF == PixelFormat::Y210;
    static constexpr ColorDepth depth = wide ? ColorDepth::p10bit : ColorDepth::p8bit;
    static constexpr uint wf = (PF == PixelFormat::UYVY || PF == PixelFormat::Y210) ? 2u : 1u;
    static constexpr uint rows(uint h) { return wf == 2u ? h : PF == PixelFormat::P210 ? 2u * h : h + h / 2u; }
    static constexpr uint32_t code = PF == PixelFormat::NV12 ? FKB_PIX_NV12 : PF == PixelFormat::NV21 ? FKB_PIX_NV21
                                   : PF == PixelFormat::UYVY ? FKB_PIX_UYVY : PF == PixelFormat::P010 ? FKB_PIX_P010
                                   : PF == PixelFormat::P210 ? FKB_PIX_P210 : FKB_PIX_Y210;
};
template <ColorDepth CD> using ColorDepthPixelBaseType = std::conditional_t<CD == ColorDepth::p8bit, uchar, ushort>;
template <ColorDepth CD> using ColorDepthPixelType = std::conditional_t<CD == ColorDepth::p8bit, uchar3, ushort3>;

template <PixelFormat PF>
struct RawImage {
    RawPtr<ND::_2D, ColorDepthPixelBaseType<PixelFormatTraits<PF>::depth>> data;
    uint width, height;
};

template <PixelFormat PF>
class Image {
    static_assert(PixelFormatTraits<PF>::supported, "NV12, NV21, UYVY, P010, P210 and Y210 are the image formats the B200 kernels read");
public:
    using BaseType = ColorDepthPixelBaseType<PixelFormatTraits<PF>::depth>;
    static constexpr PixelFormat pixelFormat = PF;
private:
    Ptr<ND::_2D, BaseType> data;
    uint width{0}, height{0};

public:
    Image(const Ptr<ND::_2D, BaseType>& data_, const uint& width_, const uint& height_) : data(data_), width(width_), height(height_) {}
    Image(const uint width_, const uint height_, const MemType memType = defaultMemType, const uint deviceID = 0)
        : width(width_), height(height_) {
        data = Ptr<ND::_2D, BaseType>(PtrDims<ND::_2D>(width_ * PixelFormatTraits<PF>::wf, PixelFormatTraits<PF>::rows(height_), 0),
                                      memType, static_cast<int>(deviceID));
    }
    uint imageWidth() const { return width; }
    uint imageHeight() const { return height; }
    RawImage<PF> ptr() const { return RawImage<PF>{data.ptr(), width, height}; }
    RawImage<PF> operator()() const { return ptr(); }
    Ptr<ND::_2D, BaseType> getData() const { return data; }
    void upload(Stream_<ParArch::GPU_NVIDIA>& stream) { data.upload(stream); }
    void download(Stream_<ParArch::GPU_NVIDIA>& stream) { data.download(stream); }
};

}  // namespace fk
