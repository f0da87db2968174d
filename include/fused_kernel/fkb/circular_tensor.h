// CircularTensor: a tensor of the last BATCH results of a chain, kept in temporal order
// (FusedKernelLibrary: core/data/circular_tensor.h:80-175).
//
// update(stream, read, ops..., write) runs the chain on one new image and, in the same launch, moves the BATCH - 1 images
// that stay from a second, ring-ordered tensor into their new places: one divergent launch of two sequences, as in the
// reference (circular_tensor.h:111-161).  The reference stores the new image in the ring with a mid-chain write
// (CircularTensorWrite, memory_operations.h:554-583); here the update sequence simply runs on two planes — the ring's and
// the output's.  The copy sequence reads float planes (packed float3: TensorRead; planar: TensorPack / TensorTPack).
#pragma once
#include "execute.h"

namespace fk {

enum class CircularTensorOrder { NewestFirst, OldestFirst };
enum class ColorPlanes { Standard, Transposed };

template <typename T, int COLOR_PLANES, int BATCH, CircularTensorOrder CT_ORDER, ColorPlanes CP_MODE>
class CircularTensor : public std::conditional_t<CP_MODE == ColorPlanes::Standard, Tensor<T>, TensorT<T>> {
    using ParentType = std::conditional_t<CP_MODE == ColorPlanes::Standard, Tensor<T>, TensorT<T>>;
    static_assert((std::is_same_v<T, float3> && COLOR_PLANES == 1) || (std::is_same_v<T, float> && COLOR_PLANES == 3),
                  "CircularTensor<float3, 1, ...> (packed) and CircularTensor<float, 3, ...> (planar) are the circular tensors the B200 kernels implement");
    static_assert(CP_MODE == ColorPlanes::Standard || std::is_same_v<T, float>, "a transposed circular tensor stores planar channels");
    static_assert(BATCH >= 2, "a circular tensor holds at least two images");
    ParentType m_tempTensor;
    int m_nextUpdateIdx{0};

public:
    using StoreT = float3;
    CircularTensor() = default;
    CircularTensor(const uint& width_, const uint& height_, const MemType& type_ = defaultMemType, const int& deviceID_ = 0)
        : ParentType(width_, height_, BATCH, COLOR_PLANES, type_, deviceID_), m_tempTensor(width_, height_, BATCH, COLOR_PLANES, type_, deviceID_) {}

    template <typename... IOps>
    void update(Stream_<ParArch::GPU_NVIDIA>& stream, const IOps&... iops) {
        if (!(this->getMemType() == MemType::Device || this->getMemType() == MemType::DeviceAndPinned))
            throw std::runtime_error("CircularTensor operations on Device memory only supported if the CircularTensor is MemType::Device or MemType::DeviceAndPinned");
        const auto low = detail::lower_sequence(std::make_tuple(iops...));
        if (low.n_planes != 1) throw std::runtime_error("CircularTensor::update takes a chain that produces one image");
        if (low.wr.data != this->ptr().data) throw std::runtime_error("CircularTensor::update: the chain must write into this tensor");
        if (CP_MODE == ColorPlanes::Transposed && low.wr.write_kind != FKB_WRITE_SPLIT)
            throw std::runtime_error("Need to use TensorTSplitWrite as write function because you are using a transposed CircularTensor (CP_MODE = Transposed)");
        const size_t plane_step = low.wr.plane_stride;
        uint8_t* const out = reinterpret_cast<uint8_t*>(this->ptr().data);
        uint8_t* const ring = reinterpret_cast<uint8_t*>(m_tempTensor.ptr().data);
        fkb_chain_desc chains[2] = {low.chain, fkb_chain_desc{}};
        fkb_chain_desc& copy = chains[1];
        copy.src_format = low.wr.write_kind == FKB_WRITE_PACKED ? FKB_PIX_F32C3 : FKB_PIX_F32P3;
        copy.geometry = FKB_GEOM_NONE; copy.dst_format = FKB_PIX_F32C3; copy.write_kind = low.wr.write_kind;
        std::vector<fkb_plane_desc> planes;
        // the update sequence owns one plane of the output: the first (newest first) or the last (oldest first) ...
        constexpr int zu = CT_ORDER == CircularTensorOrder::NewestFirst ? 0 : BATCH - 1;
        fkb_plane_desc d = low.plane(0, 0);
        d.dst = out + static_cast<size_t>(zu) * plane_step;
        planes.push_back(d);
        // ... and stores the same image at (zu + first) mod BATCH of the ring (CircularTensorWrite<Ascendent>)
        d.dst = ring + static_cast<size_t>((zu + m_nextUpdateIdx) % BATCH) * plane_step;
        planes.push_back(d);
        for (int z = 0; z < BATCH; ++z) {
            if (z == zu) continue;
            // CircularTensorRead: descendent from `first` (newest first) or ascendent (oldest first), memory_operations.h:423-431
            const int zs = CT_ORDER == CircularTensorOrder::NewestFirst ? (m_nextUpdateIdx - z + BATCH) % BATCH : (z + m_nextUpdateIdx) % BATCH;
            fkb_plane_desc c{};
            c.src = ring + static_cast<size_t>(zs) * plane_step;
            if (copy.src_format == FKB_PIX_F32P3) c.src_chroma = static_cast<const uint8_t*>(c.src) + low.wr.channel_stride;
            c.src_pitch = low.wr.pitch; c.src_w = low.wr.width; c.src_h = low.wr.height;
            c.crop_w = static_cast<int>(low.wr.width); c.crop_h = static_cast<int>(low.wr.height);
            c.dst = out + static_cast<size_t>(z) * plane_step;
            c.dst_w = low.wr.width; c.dst_h = low.wr.height; c.dst_pitch = low.wr.pitch; c.dst_channel_stride = low.wr.channel_stride;
            c.chain = 1;
            planes.push_back(c);
        }
        detail::check(fkb_launch_divergent(chains, 2, planes.data(), static_cast<uint32_t>(planes.size()), stream.getCUDAStream()));
        m_nextUpdateIdx = (m_nextUpdateIdx + 1) % BATCH;
    }
};

}  // namespace fk
