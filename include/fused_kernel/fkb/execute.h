// Front end, part 4: lowering of a built chain to include/fkb/fkb.h descriptors and the executors.
//
// Reference entry points mirrored (paths relative to the reference's include/fused_kernel/):
//   fk::executeOperations<DPP>(stream, iops...) .................. fused_kernel.h:22-25
//   Executor<TransformDPP<PA,TF>>::executeOperations ............. core/execution_model/executors.h:311-358
//   BackFuser::fuse_back (everything up to the last ReadBack is folded into the Read)
//                                                                  core/execution_model/operation_model/iop_fuser.h:137-193
//   buildOperationSequence / IOpSequence ......................... core/data/tuple.h:360-371
//   Executor<DivergentBatchTransformDPP<PA,Selector>>::executeOperations
//                                                                  executors.h:360-411, data_parallel_patterns.h:322-331
// Behaviour kept: asynchronous on the stream, no synchronisation; a failing launch throws std::runtime_error (the
// reference's gpuErrchk does, core/utils/utils.h:100-114); the first IOp must be a Read, the last a Write, and the
// value types of neighbouring operations must match (static_assert, a compile error in the reference too).
#pragma once
#include <tuple>

#include "ops.h"

namespace fk {

template <ParArch PA = defaultParArch, TF TFEN = TF::DISABLED>
struct TransformDPP {
    static constexpr ParArch PAR_ARCH = PA;
};
template <ParArch PA, typename SequenceSelector>
struct DivergentBatchTransformDPP {
    static constexpr ParArch PAR_ARCH = PA;
};

template <typename... IOps>
struct IOpSequence {
    std::tuple<IOps...> iops;
};
template <typename... IOps>
constexpr auto buildOperationSequence(const IOps&... iops) { return IOpSequence<IOps...>{{iops...}}; }

namespace detail {

inline void check(int status) {
    if (status != FKB_OK) {
        std::string msg = std::string("GPU Error: fkb status ") + std::to_string(status) + " (" + fkb_status_string(status) + ")";
        if (status == FKB_ERR_CUDA) msg += std::string(": ") + cudaGetErrorString(static_cast<cudaError_t>(fkb_last_cuda_error()));
        throw std::runtime_error(msg);
    }
}

// folds [Read, (Crop|Resize|compute)...] into one ReadIOp, exactly the order the caller gave
template <typename R>
auto fold_chain(const R& read) { return read; }
template <typename R, typename Next, typename... Rest>
auto fold_chain(const R& read, const Next& next, const Rest&... rest) {
    // operations listed after the read keep a conditional batch read conditional; only an explicit .then(compute) by
    // the caller re-batches the read with PROCESS_ALL, as the reference's fuser does
    auto fused = read.then(next);
    fused.st.used_planes = read.st.used_planes;
    return fold_chain(fused, rest...);
}

template <typename Tuple, size_t... I>
auto fold_all_but_last(const Tuple& t, std::index_sequence<I...>) { return fold_chain(std::get<I>(t)...); }

// A lowered chain: the descriptor plus a function that fills the descriptor of one plane.
template <typename OutT, size_t BATCH, typename WT>
struct Lowered {
    fkb_chain_desc chain{};
    ReadState st;
    WriteIOp<WT> wr;
    uint32_t n_planes{1};
    std::vector<int> op_slot;  // per op: -1 immediate, else plane slot

    Lowered(const ReadIOp<OutT, BATCH>& r, const WriteIOp<WT>& w) : st(r.st), wr(w) {
        static_assert(std::is_same_v<OutT, WT>, "the Write's InputType is not the OutputType of the last operation");
        static_assert(std::is_same_v<WT, uchar3> || std::is_same_v<WT, float3> || std::is_same_v<WT, uchar4> || std::is_same_v<WT, float4> ||
                      std::is_same_v<WT, uchar> || std::is_same_v<WT, float>,
                      "uchar3, float3, uchar4, float4 and (after a gray conversion) uchar and float are the pixel types the B200 kernels write");
        n_planes = r.params.activeThreads.z;
        chain.src_format = st.src_format;
        chain.geometry = !st.has_resize ? FKB_GEOM_NONE
                       : st.ar == AspectRatio::IGNORE_AR ? FKB_GEOM_RESIZE_IGNORE_AR
                       : st.ar == AspectRatio::PRESERVE_AR_RN_EVEN ? FKB_GEOM_RESIZE_PRESERVE_AR_RN_EVEN
                       : st.ar == AspectRatio::PRESERVE_AR_LEFT ? FKB_GEOM_RESIZE_PRESERVE_AR_LEFT : FKB_GEOM_RESIZE_PRESERVE_AR;
        chain.dst_format = std::is_same_v<WT, float3> ? FKB_PIX_F32C3 : std::is_same_v<WT, uchar3> ? FKB_PIX_U8C3
                         : std::is_same_v<WT, float4> ? FKB_PIX_F32C4 : std::is_same_v<WT, uchar4> ? FKB_PIX_U8C4
                         : std::is_same_v<WT, float> ? FKB_PIX_F32C1 : FKB_PIX_U8C1;
        chain.write_kind = wr.write_kind;
        if (st.ops.size() > FKB_MAX_OPS) check(FKB_ERR_UNSUPPORTED);
        chain.n_ops = static_cast<uint32_t>(st.ops.size());
        chain.n_pre_ops = static_cast<uint32_t>(st.has_resize ? st.n_pre_ops : 0);
        chain.border = st.border; chain.border_at = static_cast<uint32_t>(st.border_at);
        for (int i = 0; i < 3; ++i) chain.border_value[i] = st.border_value[i];
        chain.border_value_w = st.border_value[3];
        for (int i = 0; i < 9; ++i) chain.ccm2[i] = st.ccm2[i];
        for (int i = 0; i < 3; ++i) chain.yuv_add[i] = st.yuv_add[i];
        for (int i = 0; i < 9; ++i) chain.ccm[i] = st.ccm[i];
        for (int i = 0; i < 3; ++i) chain.yuv_sub[i] = st.yuv_sub[i];
        int next_slot = 0;
        for (size_t k = 0; k < st.ops.size(); ++k) {
            const OpRec& op = st.ops[k];
            bool same = true;
            for (const auto& v : op.v) same = same && v == op.v[0];
            int slot = -1;
            if (!same) {  // operands differ between planes: they travel in the plane descriptors
                if (next_slot >= static_cast<int>(FKB_MAX_PLANE_PARAMS)) check(FKB_ERR_UNSUPPORTED);
                slot = next_slot++;
            }
            op_slot.push_back(slot);
            chain.ops[k].code = op.code;
            chain.ops[k].plane_slot = static_cast<int16_t>(slot);
            for (int c = 0; c < 3; ++c) chain.ops[k].v[c] = op.v[0][c];
            chain.op_w[k] = op.v[0][3];
        }
    }

    // descriptor of global plane z (batched parameters are indexed by z, shared ones by 0)
    fkb_plane_desc plane(uint32_t z, uint32_t chain_index) const {
        fkb_plane_desc d{};
        auto pick = [z](const auto& vec) -> const auto& {
            if (vec.size() == 1) return vec[0];
            if (z >= vec.size()) throw std::runtime_error("plane index beyond the batch of an operation of this sequence");
            return vec[z];
        };
        const SrcPlane& s = pick(st.src);
        d.src = s.data; d.src_pitch = s.pitch; d.src_w = s.w; d.src_h = s.h;
        if (st.src_format == FKB_PIX_NV12 || st.src_format == FKB_PIX_NV21 || st.src_format == FKB_PIX_P010 || st.src_format == FKB_PIX_P210)
            d.src_chroma = static_cast<const uint8_t*>(s.data) + static_cast<size_t>(s.pitch) * s.h;
        if (st.crops.empty()) { d.crop_x = 0; d.crop_y = 0; d.crop_w = static_cast<int>(s.w); d.crop_h = static_cast<int>(s.h); }
        else { const Rect& r = pick(st.crops); d.crop_x = r.x; d.crop_y = r.y; d.crop_w = r.width; d.crop_h = r.height; }
        if (st.has_resize) { d.dst_w = st.dst_size.width; d.dst_h = st.dst_size.height; }
        else { d.dst_w = d.crop_w; d.dst_h = d.crop_h; }
        if (d.dst_w > wr.width || d.dst_h > wr.height) throw std::runtime_error("the output of the chain is larger than the Write's buffer");
        if (z >= wr.planes) throw std::runtime_error("plane index beyond the planes of the Write's buffer");
        d.dst = static_cast<uint8_t*>(wr.data) + static_cast<size_t>(z) * wr.plane_stride;
        d.dst_pitch = wr.pitch;
        d.dst_channel_stride = wr.channel_stride;
        d.dst_y = wr.data_y; d.dst_z = wr.data_z;
        d.bg[0] = st.bg[0]; d.bg[1] = st.bg[1]; d.bg[2] = st.bg[2]; d.bg_w = st.bg[3];
        d.chain = chain_index;
        if (st.used_planes >= 0 && z >= static_cast<uint32_t>(st.used_planes)) {
            d.chain |= FKB_PLANE_DEFAULT;
            d.bg[0] = st.dflt[0]; d.bg[1] = st.dflt[1]; d.bg[2] = st.dflt[2]; d.bg_w = st.dflt[3];
        }
        for (size_t k = 0; k < st.ops.size(); ++k)
            if (op_slot[k] >= 0) { const auto& v = pick(st.ops[k].v); for (int c = 0; c < 3; ++c) d.params[op_slot[k]][c] = v[c]; d.params_w[op_slot[k]] = v[3]; }
        if (st.has_resize && !(d.chain & FKB_PLANE_DEFAULT)) check(fkb_resize_params(chain.geometry, &d));
        return d;
    }
};

template <typename... IOps>
auto lower_sequence(const std::tuple<IOps...>& t) {
    constexpr size_t N = sizeof...(IOps);
    static_assert(N >= 2, "a chain needs at least a Read and a Write");
    using First = std::decay_t<std::tuple_element_t<0, std::tuple<IOps...>>>;  // (the tuple may hold references)
    using Last = std::decay_t<std::tuple_element_t<N - 1, std::tuple<IOps...>>>;
    static_assert(isReadIOp<First>, "The first IOp must be a complete Read operation");
    static_assert(isWriteIOp<Last>, "The last IOp must be a Write operation");
    const auto read = fold_all_but_last(t, std::make_index_sequence<N - 1>{});
    using R = std::decay_t<decltype(read)>;
    return Lowered<typename R::OutputType, R::batch, typename Last::InputType>(read, std::get<N - 1>(t));
}

}  // namespace detail

template <typename DPP>
struct Executor;

template <ParArch PA, TF TFEN>
struct Executor<TransformDPP<PA, TFEN>> {
    static_assert(PA == ParArch::GPU_NVIDIA, "this library executes on ParArch::GPU_NVIDIA only (there is no CPU path)");
    template <typename... IOps>
    static void executeOperations(Stream_<ParArch::GPU_NVIDIA>& stream, const IOps&... iops) {
        const auto low = detail::lower_sequence(std::tie(iops...));
        // (the descriptor array is kept per thread: a fresh allocation of its size is page-faulted in on every call)
        static thread_local std::vector<fkb_plane_desc> planes;
        planes.resize(low.n_planes);
        for (uint32_t z = 0; z < low.n_planes; ++z) planes[z] = low.plane(z, 0);
        detail::check(fkb_launch_transform(&low.chain, planes.data(), low.n_planes, stream.getCUDAStream()));
    }
};

template <ParArch PA, typename Selector>
struct Executor<DivergentBatchTransformDPP<PA, Selector>> {
    static_assert(PA == ParArch::GPU_NVIDIA, "this library executes on ParArch::GPU_NVIDIA only (there is no CPU path)");
    template <typename... Seqs>
    static void executeOperations(Stream_<ParArch::GPU_NVIDIA>& stream, const Seqs&... seqs) {
        static_assert(sizeof...(Seqs) >= 1 && sizeof...(Seqs) <= FKB_MAX_CHAINS, "between 1 and FKB_MAX_CHAINS sequences");
        const auto lows = std::make_tuple(detail::lower_sequence(seqs.iops)...);
        std::vector<fkb_chain_desc> chains;
        uint32_t total = 0;
        std::apply([&](const auto&... l) { ((chains.push_back(l.chain), total += l.n_planes), ...); }, lows);
        // grid z = the sum of the sequences' planes; plane z runs sequence Selector::at(z) and keeps its global index
        std::vector<fkb_plane_desc> planes(total);
        for (uint32_t z = 0; z < total; ++z) {
            const uint32_t k = Selector::at(z);
            if (k >= sizeof...(Seqs)) throw std::runtime_error("SequenceSelector returned an index beyond the sequences");
            uint32_t i = 0;
            std::apply([&](const auto&... l) { ((i++ == k ? void(planes[z] = l.plane(z, k)) : void()), ...); }, lows);
        }
        detail::check(fkb_launch_divergent(chains.data(), static_cast<uint32_t>(chains.size()), planes.data(), total, stream.getCUDAStream()));
    }
};

template <typename DPPType, typename... Args>
inline void executeOperations(Stream_<DPPType::PAR_ARCH>& stream, const Args&... args) {
    Executor<DPPType>::executeOperations(stream, args...);
}
// the conveniences of core/execution_model/executors.h:67-78 (one source, optionally one destination) ...
template <typename DPPType, ND D, typename I, typename... IOps>
inline void executeOperations(const Ptr<D, I>& input, Stream_<DPPType::PAR_ARCH>& stream, const IOps&... iOps) {
    Executor<DPPType>::executeOperations(stream, PerThreadRead<D, I>::build(input), iOps...);
}
template <typename DPPType, ND D, typename I, typename O, typename... IOps>
inline void executeOperations(const Ptr<D, I>& input, const Ptr<D, O>& output, Stream_<DPPType::PAR_ARCH>& stream, const IOps&... iOps) {
    Executor<DPPType>::executeOperations(stream, PerThreadRead<D, I>::build(input), iOps..., PerThreadWrite<D, O>::build(output));
}
// ... and the batch conveniences of :80-114
template <typename DPPType, typename I, size_t BATCH, typename... IOps>
inline void executeOperations(const std::array<Ptr2D<I>, BATCH>& input, const int& activeBatch, const I& defaultValue,
                              Stream_<DPPType::PAR_ARCH>& stream, const IOps&... iOps) {
    Executor<DPPType>::executeOperations(stream, PerThreadRead<ND::_2D, I>::build(activeBatch, defaultValue, input), iOps...);
}
template <typename DPPType, typename I, size_t BATCH, typename... IOps>
inline void executeOperations(const std::array<Ptr2D<I>, BATCH>& input, Stream_<DPPType::PAR_ARCH>& stream, const IOps&... iOps) {
    Executor<DPPType>::executeOperations(stream, PerThreadRead<ND::_2D, I>::build(input), iOps...);
}
template <typename DPPType, typename I, typename O, size_t BATCH, typename... IOps>
inline void executeOperations(const std::array<Ptr2D<I>, BATCH>& input, const int& activeBatch, const I& defaultValue,
                              const Tensor<O>& output, Stream_<DPPType::PAR_ARCH>& stream, const IOps&... iOps) {
    Executor<DPPType>::executeOperations(stream, PerThreadRead<ND::_2D, I>::build(activeBatch, defaultValue, input), iOps...,
                                         TensorWrite<O>::build(output));
}
template <typename DPPType, typename I, typename O, size_t BATCH, typename... IOps>
inline void executeOperations(const std::array<Ptr2D<I>, BATCH>& input, const Tensor<O>& output, Stream_<DPPType::PAR_ARCH>& stream,
                              const IOps&... iOps) {
    Executor<DPPType>::executeOperations(stream, PerThreadRead<ND::_2D, I>::build(input), iOps..., TensorWrite<O>::build(output));
}

}  // namespace fk
