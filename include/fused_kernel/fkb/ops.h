// Front end, part 3: the operations ("IOps") a chain is built from, with the reference's builder spellings.
//
// Reference builders mirrored (paths relative to the reference's include/fused_kernel/):
//   PerThreadRead<ND::_2D,T>::build(ptr | std::array<Ptr2D,N>) ... algorithms/basic_ops/memory_operations.h:27-67,
//                                                                 core/execution_model/operation_model/batch_operations.h:523-543
//   ReadYUV<PixelFormat::NV12>::build(image) ..................... algorithms/image_processing/color_conversion.h:206-294
//   Crop<>::build(Rect | std::array<Rect,N>) ..................... algorithms/image_processing/crop.h:62-91
//   Resize<INTER_LINEAR, AR>::build(Size[, background]) .......... algorithms/image_processing/resize.h:159-162, 262-264
//   Cast / Mul / Add / Sub / Div / SaturateCast / ColorConversion / ConvertYUVToRGB ::build(...)
//                                                                  core/execution_model/operation_model/parent_operations.h:55, 84-85
//   PerThreadWrite / TensorWrite / TensorSplit ::build(ptr) ...... algorithms/basic_ops/memory_operations.h:85-212
//   iop.then(next) ............................................... core/execution_model/operation_model/instantiable_operations.h:43-52
//   BatchRead<PlanePolicy::PROCESS_ALL>::build(std::array<IOp,N>)  batch_operations.h:395-425
// In the reference an IOp's type encodes the operation and its value holds the parameters; ill-typed chains fail to
// compile.  Here the static types carry just enough (value type flowing through the chain, batch size) to keep those
// compile-time rejections, and the parameters live in a small run-time record that is lowered to include/fkb/fkb.h.
#pragma once
#include <memory>
#include <array>
#include <vector>

#include "fkb/fkb.h"
#include "memory.h"

namespace fk {

enum class InterpolationType { INTER_LINEAR = 1 };
enum class AspectRatio { PRESERVE_AR = 0, IGNORE_AR = 1, PRESERVE_AR_RN_EVEN = 2, PRESERVE_AR_LEFT = 3 };  // resize.h:42
// border_reader.h:25-36
enum class BorderType : int { CONSTANT = 0, REPLICATE = 1, REFLECT = 2, WRAP = 3, REFLECT_101 = 4, TRANSPARENT_ = 5, DEFAULT = REFLECT_101, ISOLATED = 16 };
enum class PlanePolicy { PROCESS_ALL = 0, CONDITIONAL_WITH_DEFAULT = 1 };  // batch_operations.h:75
// (color_conversion.h:408-426; the codes that discard the alpha channel of a four-channel source are the ones beside BGR<->RGB)
enum class ColorConversionCodes { COLOR_BGR2RGB, COLOR_RGB2BGR, COLOR_BGRA2BGR, COLOR_RGBA2RGB, COLOR_BGRA2RGB, COLOR_RGBA2BGR, COLOR_BGRA2RGBA, COLOR_RGBA2BGRA,
                                  COLOR_BGR2BGRA, COLOR_RGB2RGBA = COLOR_BGR2BGRA, COLOR_BGR2RGBA, COLOR_RGB2BGRA = COLOR_BGR2RGBA,
                                  COLOR_BGR2GRAY, COLOR_RGB2GRAY, COLOR_BGRA2GRAY, COLOR_RGBA2GRAY };

namespace detail {
struct SrcPlane { const void* data{nullptr}; uint pitch{0}, w{0}, h{0}; };
struct OpRec {
    uint16_t code{0};
    std::vector<std::array<float, 4>> v;  // one operand per plane, or a single one shared by all planes (fourth component: four-channel chains)
};
// A vector that is shared between the copies of a ReadState until one of them changes it: every .then() of a chain
// copies the state, and the per-plane vectors of a batch of thousands of planes need not be copied with it.
template <typename T>
class SharedVec {
    std::shared_ptr<std::vector<T>> p_;
    static const std::vector<T>& none() { static const std::vector<T> e; return e; }
public:
    const std::vector<T>& get() const { return p_ ? *p_ : none(); }
    std::vector<T>& mut() {  // a private copy from here on
        if (!p_) p_ = std::make_shared<std::vector<T>>();
        else if (p_.use_count() > 1) p_ = std::make_shared<std::vector<T>>(*p_);
        return *p_;
    }
    void assign(std::vector<T> v) { p_ = std::make_shared<std::vector<T>>(std::move(v)); }
    size_t size() const { return get().size(); }
    bool empty() const { return get().empty(); }
    const T& operator[](size_t i) const { return get()[i]; }
    auto begin() const { return get().begin(); }
    auto end() const { return get().end(); }
};
// Everything a chain knows before its Write: the run-time image of the reference's fused Read IOp.
struct ReadState {
    uint32_t src_format{FKB_PIX_U8C3};
    SharedVec<SrcPlane> src;     // 1 entry (shared) or one per plane
    SharedVec<Rect> crops;       // empty (whole frame), 1 entry, or one per plane
    bool has_resize{false};
    AspectRatio ar{AspectRatio::IGNORE_AR};
    Size dst_size;
    float bg[4]{0.f, 0.f, 0.f, 0.f};
    std::vector<OpRec> ops;
    size_t n_pre_ops{0};         // ops that were chained before the Resize run on the taps
    float ccm[9]{};
    float yuv_sub[3]{};
    float ccm2[9]{};             // ConvertRGBToYUV: matrix and offsets
    float yuv_add[3]{};
    // BatchRead<CONDITIONAL_WITH_DEFAULT>: planes >= used_planes yield dflt instead of reading (-1: every plane reads)
    int used_planes{-1};
    float dflt[4]{0.f, 0.f, 0.f, 0.f};
    // BorderReader between the first border_at ops and the Crop (0 = none, else FKB_BORDER_*)
    uint32_t border{0};
    size_t border_at{0};
    float border_value[4]{0.f, 0.f, 0.f, 0.f};
};
inline std::array<float, 4> f3(const float3& v, float w = 0.f) { return {v.x, v.y, v.z, w}; }
// fourth component of a vector value, or 0 for the three-channel types
template <typename V> float w_of(const V& v) { if constexpr (cn<V> == 4) return static_cast<float>(v.w); else return 0.f; }
template <typename T, typename = void> struct has_read_state : std::false_type {};
template <typename T> struct has_read_state<T, std::void_t<decltype(std::declval<T>().st)>> : std::true_type {};
}  // namespace detail

// ---- compute IOps -------------------------------------------------------------------------------------------------
template <uint16_t CODE, typename I, typename O>
struct ComputeIOp {
    using InputType = I;
    using OutputType = O;
    static constexpr uint16_t code = CODE;
    float3 params{0.f, 0.f, 0.f};
    float ccm[9]{};
    float yuv_sub[3]{};
    float w{0.f};  // fourth operand (four-channel chains)
};
template <typename T> constexpr bool isComputeIOp = false;
template <uint16_t C, typename I, typename O> constexpr bool isComputeIOp<ComputeIOp<C, I, O>> = true;

template <typename I, typename O>
struct Cast {
    static_assert((std::is_same_v<I, uchar3> && std::is_same_v<O, float3>) || (std::is_same_v<I, uchar4> && std::is_same_v<O, float4>) ||
                  (std::is_same_v<I, uchar> && std::is_same_v<O, float>),
                  "the B200 kernels implement Cast<uchar3,float3>, Cast<uchar4,float4> and (after a gray conversion) Cast<uchar,float>");
    static constexpr auto build() { return ComputeIOp<FKB_OP_CAST_F32, I, O>{}; }
};
#define FKB_BINARY_OP(Name, CODE)                                                                                     \
    template <typename I, typename P = I, typename O = I>                                                             \
    struct Name {                                                                                                     \
        static_assert((std::is_same_v<I, float3> || std::is_same_v<I, float4> || std::is_same_v<I, float>) && std::is_same_v<P, I> && std::is_same_v<O, I>, \
                      "the B200 kernels implement " #Name "<float3>, " #Name "<float4> and (after a gray conversion) " #Name "<float>");   \
        static constexpr auto build(const I& params) {                                                                            \
            if constexpr (cn<I> == 1) {                                                                                           \
                return ComputeIOp<CODE, I, O>{float3{params, params, params}};                                                    \
            } else {                                                                                                              \
                ComputeIOp<CODE, I, O> op{float3{params.x, params.y, params.z}};                                                  \
                if constexpr (cn<I> == 4) op.w = params.w;                                                                        \
                return op;                                                                                                        \
            }                                                                                                                     \
        }                                                                                                                         \
    };
FKB_BINARY_OP(Mul, FKB_OP_MUL)
FKB_BINARY_OP(Add, FKB_OP_ADD)
FKB_BINARY_OP(Sub, FKB_OP_SUB)
FKB_BINARY_OP(Div, FKB_OP_DIV)
#undef FKB_BINARY_OP
template <typename I, typename O>
struct SaturateCast {
    static_assert((std::is_same_v<I, float3> && std::is_same_v<O, uchar3>) || (std::is_same_v<I, float4> && std::is_same_v<O, uchar4>) ||
                  (std::is_same_v<I, float> && std::is_same_v<O, uchar>),
                  "the B200 kernels implement SaturateCast<float3,uchar3>, SaturateCast<float4,uchar4> and SaturateCast<float,uchar>");
    static constexpr auto build() { return ComputeIOp<FKB_OP_SATCAST_U8, I, O>{}; }
};
// A step of a chain that changes the number of channels without arithmetic: the alpha channel of a uchar4 / float4 is
// dropped, or an opaque one is appended to a uchar3 / float3 (AddOpaqueAlpha, color_conversion.h:81-94)
template <typename I, typename O>
struct RetypeIOp {
    using InputType = I;
    using OutputType = O;
    bool reorder;          // BGRA2RGB / RGBA2BGR / BGR2RGBA / RGB2BGRA: the three colour channels are also reversed
    bool add_alpha{false};
    float alpha{0.f};      // maxDepthValue<CD>
    bool gray{false};      // RGB2Gray: the three colour channels become one (a fourth channel of the input is ignored)
};
// RGB2Gray<I, O, GrayFormula::CCIR_601> (color_conversion.h:44-79): 0.299 x + 0.587 y + 0.114 z, rounded to the nearest integer.
enum class GrayFormula { CCIR_601 };
template <typename I, typename O = VBase<I>, GrayFormula GF = GrayFormula::CCIR_601>
struct RGB2Gray {
    static_assert((std::is_same_v<O, uchar> && (std::is_same_v<I, uchar3> || std::is_same_v<I, uchar4>)) ||
                  (std::is_same_v<O, float> && (std::is_same_v<I, uchar3> || std::is_same_v<I, uchar4> || std::is_same_v<I, float3> || std::is_same_v<I, float4>)),
                  "RGB2Gray takes uchar3 / uchar4 to uchar, or uchar3 / uchar4 / float3 / float4 to float");
    static constexpr auto build() { return RetypeIOp<I, O>{false, false, 0.f, true}; }
};
template <ColorConversionCodes CODE, typename I, typename O = I, ColorDepth CD = ColorDepth::p8bit>
struct ColorConversion {
    static constexpr bool swap4 = CODE == ColorConversionCodes::COLOR_BGRA2RGBA || CODE == ColorConversionCodes::COLOR_RGBA2BGRA;
    static constexpr bool swap3 = CODE == ColorConversionCodes::COLOR_BGR2RGB || CODE == ColorConversionCodes::COLOR_RGB2BGR || swap4;
    static constexpr bool add = CODE == ColorConversionCodes::COLOR_BGR2BGRA || CODE == ColorConversionCodes::COLOR_BGR2RGBA;
    static constexpr bool gray = CODE == ColorConversionCodes::COLOR_BGR2GRAY || CODE == ColorConversionCodes::COLOR_RGB2GRAY ||
                                 CODE == ColorConversionCodes::COLOR_BGRA2GRAY || CODE == ColorConversionCodes::COLOR_RGBA2GRAY;
    static constexpr bool drop = !swap3 && !add && !gray;
    static_assert(!gray || ((CODE == ColorConversionCodes::COLOR_BGR2GRAY || CODE == ColorConversionCodes::COLOR_RGB2GRAY) == (cn<I> == 3)),
                  "BGR2GRAY / RGB2GRAY take three channels, BGRA2GRAY / RGBA2GRAY four");
    static_assert(!add || (std::is_same_v<I, uchar3> && std::is_same_v<O, uchar4>) || (std::is_same_v<I, float3> && std::is_same_v<O, float4>),
                  "BGR2BGRA / RGB2RGBA / BGR2RGBA / RGB2BGRA take uchar3 -> uchar4 or float3 -> float4");
    static_assert(!add || CD == ColorDepth::p8bit || CD == ColorDepth::fn8bit, "the appended alpha is that of an 8-bit depth (255) or of a normalised one (1)");
    static_assert(!swap3 || swap4 || (std::is_same_v<I, O> && (std::is_same_v<I, float3> || std::is_same_v<I, uchar3>)),
                  "BGR<->RGB on uchar3 or float3 is the three-channel colour conversion the B200 kernels implement");
    static_assert(!swap4 || (std::is_same_v<I, O> && (std::is_same_v<I, float4> || std::is_same_v<I, uchar4>)),
                  "BGRA<->RGBA takes uchar4 or float4 and leaves the fourth channel in place");
    static_assert(!drop || (std::is_same_v<I, uchar4> && std::is_same_v<O, uchar3>) || (std::is_same_v<I, float4> && std::is_same_v<O, float3>),
                  "BGRA2BGR / RGBA2RGB / BGRA2RGB / RGBA2BGR take uchar4 -> uchar3 or float4 -> float3");
    static constexpr auto build() {
        if constexpr (gray) {  // (color_conversion.h:484-502: a channel reversal first for the BGR orders)
            auto op = RGB2Gray<I, O>::build();
            op.reorder = CODE == ColorConversionCodes::COLOR_BGR2GRAY || CODE == ColorConversionCodes::COLOR_BGRA2GRAY;
            return op;
        }
        else if constexpr (swap3) return ComputeIOp<FKB_OP_REORDER_ZYX, I, O>{};
        else if constexpr (add) return RetypeIOp<I, O>{CODE == ColorConversionCodes::COLOR_BGR2RGBA, true, CD == ColorDepth::p8bit ? 255.f : 1.f};
        else return RetypeIOp<I, O>{CODE == ColorConversionCodes::COLOR_BGRA2RGB || CODE == ColorConversionCodes::COLOR_RGBA2BGR};
    }
};
// YCbCr -> RGB: the matrix and offsets of <range, primitives> as the reference evaluates them in fp32
// (algorithms/image_processing/itu_color.h:185-258, color_conversion.h:150-174), from fkb_ycbcr_to_rgb.
template <ColorDepth CD, ColorRange CR, ColorPrimitives CP>
struct ConvertYUVToRGB {
    static_assert(CD == ColorDepth::p8bit || CD == ColorDepth::p10bit, "8-bit and 10-bit YCbCr are the depths the B200 kernels convert");
    static auto build() {
        ComputeIOp<FKB_OP_YUV2RGB, ColorDepthPixelType<CD>, float3> op{};
        const uint32_t prim = CP == ColorPrimitives::bt601 ? FKB_PRIMITIVES_BT601 : CP == ColorPrimitives::bt709 ? FKB_PRIMITIVES_BT709 : FKB_PRIMITIVES_BT2020;
        if (fkb_ycbcr_to_rgb_bits(CD == ColorDepth::p8bit ? 8u : 10u, CR == ColorRange::Full ? FKB_RANGE_FULL : FKB_RANGE_LIMITED, prim,
                                  op.ccm, op.yuv_sub) != FKB_OK)
            throw std::runtime_error("ConvertYUVToRGB: colour description refused");
        return op;
    }
};

// RGB -> YCbCr (color_conversion.h:176-199); the matrix and offsets come from fkb_rgb_to_ycbcr.
template <ColorDepth CD, ColorRange CR, ColorPrimitives CP>
struct ConvertRGBToYUV {
    static_assert(CD == ColorDepth::p8bit, "8-bit YCbCr is the depth the B200 kernels convert");
    static auto build() {
        ComputeIOp<FKB_OP_RGB2YUV, uchar3, float3> op{};
        const uint32_t prim = CP == ColorPrimitives::bt601 ? FKB_PRIMITIVES_BT601 : CP == ColorPrimitives::bt709 ? FKB_PRIMITIVES_BT709 : FKB_PRIMITIVES_BT2020;
        if (fkb_rgb_to_ycbcr(CR == ColorRange::Full ? FKB_RANGE_FULL : FKB_RANGE_LIMITED, prim, op.ccm, op.yuv_sub) != FKB_OK)
            throw std::runtime_error("ConvertRGBToYUV: colour description refused");
        return op;  // (ccm / yuv_sub of the IOp carry the matrix and the offsets to add)
    }
};

// ---- BorderReader (algorithms/image_processing/border_reader.h) ------------------------------------------------
struct BorderIOp {
    uint32_t mode;     // FKB_BORDER_*
    float value[4];    // CONSTANT only
};
template <BorderType BT>
struct BorderReader {
    static_assert(BT == BorderType::CONSTANT || BT == BorderType::REPLICATE || BT == BorderType::REFLECT || BT == BorderType::WRAP ||
                  BT == BorderType::REFLECT_101, "CONSTANT, REPLICATE, REFLECT, WRAP and REFLECT_101 are the border modes the reference implements");
    static constexpr uint32_t mode = static_cast<uint32_t>(BT) + 1u;
    static auto build() {
        static_assert(BT != BorderType::CONSTANT, "BorderReader<CONSTANT> needs its value: build(value)");
        return BorderIOp{mode, {0.f, 0.f, 0.f, 0.f}};
    }
    // build(value): the incomplete CONSTANT reader; build(readIOp): the complete form of the other modes
    template <typename A>
    static auto build(const A& a) {
        if constexpr (detail::has_read_state<A>::value) {
            return a.then(build());
        } else {
            static_assert(BT == BorderType::CONSTANT, "only BorderReader<CONSTANT> takes a value");
            return BorderIOp{mode, {static_cast<float>(a.x), static_cast<float>(a.y), static_cast<float>(a.z), detail::w_of(a)}};
        }
    }
    template <typename R, typename V>
    static auto build(const R& read, const V& value) { return read.then(build(value)); }
};

// ---- incomplete ReadBack IOps ----------------------------------------------------------------------------------
template <size_t BATCH>
struct CropIOp {
    std::vector<Rect> rects;
};
template <typename BackIOp = void>
struct Crop {
    static auto build(const Rect& rect) { return CropIOp<0>{{rect}}; }
    template <size_t N>
    static auto build(const std::array<Rect, N>& rects) { return CropIOp<N>{std::vector<Rect>(rects.begin(), rects.end())}; }
};
struct ResizeIOp {
    AspectRatio ar;
    Size dst_size;
    float3 bg;
    float bg_w{0.f};  // fourth channel of the background (four-channel chains)
};
template <InterpolationType IT = InterpolationType::INTER_LINEAR, AspectRatio AR = AspectRatio::IGNORE_AR, typename DefaultType = void>
struct Resize {
    static_assert(IT == InterpolationType::INTER_LINEAR, "INTER_LINEAR is the interpolation the B200 kernels implement");
    static auto build(const Size& dstSize) {
        static_assert(AR == AspectRatio::IGNORE_AR, "PRESERVE_AR needs a background value: build(Size, float3)");
        return ResizeIOp{AR, dstSize, float3{0.f, 0.f, 0.f}};
    }
    static auto build(const Size& dstSize, const float3& backgroundValue) { return ResizeIOp{AR, dstSize, backgroundValue}; }
    static auto build(const Size& dstSize, const float4& backgroundValue) {
        return ResizeIOp{AR, dstSize, float3{backgroundValue.x, backgroundValue.y, backgroundValue.z}, backgroundValue.w};
    }
};

// ---- Read IOps -------------------------------------------------------------------------------------------------
// OutT: the value type the chain currently produces; BATCH: 0 = not batched, else the number of planes.
template <typename OutT, size_t BATCH>
struct ReadIOp {
    using OutputType = OutT;
    static constexpr size_t batch = BATCH;
    detail::ReadState st;
    struct Params { ActiveThreads activeThreads; } params;  // .activeThreads.z may be narrowed (divergent launches)

    ReadIOp() = default;
    explicit ReadIOp(detail::ReadState s) : st(std::move(s)) { refresh(); }

    void refresh() {
        const Size g = geometry();
        params.activeThreads = {static_cast<uint>(g.width), static_cast<uint>(g.height), static_cast<uint>(BATCH ? BATCH : 1)};
    }
    Size geometry() const {
        if (st.has_resize) return st.dst_size;
        if (!st.crops.empty()) { int w = 0, h = 0; for (const Rect& r : st.crops) { w = std::max(w, r.width); h = std::max(h, r.height); } return Size(w, h); }
        if (!st.src.empty()) return Size(static_cast<int>(st.src[0].w), static_cast<int>(st.src[0].h));
        return Size(0, 0);
    }
    ActiveThreads getActiveThreads() const { return params.activeThreads; }

    auto then(const BorderIOp& b) const {
        if (st.has_resize || !st.crops.empty() || st.border)
            throw std::runtime_error("a BorderReader directly on the Read (before any Crop or Resize) is the placement the B200 kernels implement");
        detail::ReadState s = st;
        s.border = b.mode; s.border_at = s.ops.size();
        for (int c = 0; c < 4; ++c) s.border_value[c] = b.value[c];
        return ReadIOp<OutT, BATCH>(std::move(s));
    }
    template <size_t N>
    auto then(const CropIOp<N>& c) const {
        static_assert(BATCH == 0 || N == 0 || BATCH == N, "Fusing two batch operations of different BATCH size is not allowed.");
        if (st.has_resize) throw std::runtime_error("Crop after Resize is not a chain the B200 kernels implement");
        detail::ReadState s = st;
        if (s.crops.empty()) s.crops.assign(c.rects);
        else {  // a crop of a crop: offsets add up
            std::vector<Rect> out(std::max(s.crops.size(), c.rects.size()));
            for (size_t i = 0; i < out.size(); ++i) {
                const Rect& a = s.crops[s.crops.size() == 1 ? 0 : i];
                const Rect& b = c.rects[c.rects.size() == 1 ? 0 : i];
                out[i] = Rect(a.x + b.x, a.y + b.y, b.width, b.height);
            }
            s.crops.assign(std::move(out));
        }
        return ReadIOp<OutT, (BATCH ? BATCH : N)>(std::move(s));
    }
    auto then(const ResizeIOp& r) const {
        if (st.has_resize) throw std::runtime_error("two Resize operations in one chain are not implemented by the B200 kernels");
        detail::ReadState s = st;
        s.has_resize = true; s.ar = r.ar; s.dst_size = r.dst_size;
        s.bg[0] = r.bg.x; s.bg[1] = r.bg.y; s.bg[2] = r.bg.z; s.bg[3] = r.bg_w;
        s.n_pre_ops = s.ops.size();
        return ReadIOp<std::conditional_t<cn<OutT> == 4, float4, float3>, BATCH>(std::move(s));  // the interpolation returns float_<cn>
    }
    template <typename I, typename O>
    auto then(const RetypeIOp<I, O>& r) const {
        static_assert(std::is_same_v<I, OutT>, "the operation's InputType is not the OutputType of the operation before it");
        detail::ReadState s = st;
        if (r.reorder) s.ops.push_back(detail::OpRec{FKB_OP_REORDER_ZYX, {{0.f, 0.f, 0.f, 0.f}}});
        if (r.add_alpha) s.ops.push_back(detail::OpRec{FKB_OP_ADD_ALPHA, {{r.alpha, 0.f, 0.f, 0.f}}});
        if (r.gray) s.ops.push_back(detail::OpRec{FKB_OP_RGB2GRAY, {{std::is_same_v<O, uchar> ? 1.f : 0.f, 0.f, 0.f, 0.f}}});
        return ReadIOp<O, BATCH>(std::move(s));
    }
    template <uint16_t C, typename I, typename O>
    auto then(const ComputeIOp<C, I, O>& op) const {
        static_assert(std::is_same_v<I, OutT>, "the operation's InputType is not the OutputType of the operation before it");
        detail::ReadState s = st;
        // the reference's fuser rebuilds a batch of fused per-plane reads here with PROCESS_ALL (iop_fuser.h:89-95):
        // a conditional batch read stops being conditional when a compute operation is fused into it
        s.used_planes = -1;
        s.ops.push_back(detail::OpRec{C, {detail::f3(op.params, op.w)}});
        if (C == FKB_OP_YUV2RGB) { for (int i = 0; i < 9; ++i) s.ccm[i] = op.ccm[i]; for (int i = 0; i < 3; ++i) s.yuv_sub[i] = op.yuv_sub[i]; }
        if (C == FKB_OP_RGB2YUV) { for (int i = 0; i < 9; ++i) s.ccm2[i] = op.ccm[i]; for (int i = 0; i < 3; ++i) s.yuv_add[i] = op.yuv_sub[i]; }
        return ReadIOp<O, BATCH>(std::move(s));
    }
};
// readIOp & nextIOp: the reference's other spelling of .then()
template <typename O, size_t B, typename Next>
auto operator&(const ReadIOp<O, B>& read, const Next& next) -> decltype(read.then(next)) { return read.then(next); }
template <typename T> constexpr bool isReadIOp = false;
template <typename O, size_t B> constexpr bool isReadIOp<ReadIOp<O, B>> = true;

template <ND D, typename T>
struct PerThreadRead {
    static_assert(D == ND::_2D && (std::is_same_v<T, uchar3> || std::is_same_v<T, uchar4>),
                  "PerThreadRead<ND::_2D, uchar3> (and uchar4, whose alpha channel the chain must discard) are the reads the B200 kernels implement");
    static constexpr uint32_t fmt = std::is_same_v<T, uchar4> ? FKB_PIX_U8C4 : FKB_PIX_U8C3;
    static auto build(const RawPtr<ND::_2D, T>& p) {
        detail::ReadState s;
        s.src_format = fmt;
        s.src.mut().push_back({p.data, p.dims.pitch, p.dims.width, p.dims.height});
        return ReadIOp<T, 0>(std::move(s));
    }
    static auto build(const Ptr<ND::_2D, T>& p) { return build(p.ptr()); }
    template <size_t N>
    static auto build(const std::array<Ptr2D<T>, N>& ptrs) {
        detail::ReadState s;
        s.src_format = fmt;
        auto& src = s.src.mut();
        src.reserve(N);
        for (const auto& p : ptrs) { const auto r = p.ptr(); src.push_back({r.data, r.dims.pitch, r.dims.width, r.dims.height}); }
        return ReadIOp<T, N>(std::move(s));
    }
    // BatchRead<CONDITIONAL_WITH_DEFAULT> (batch_operations.h:221-281, builder :530-534): planes >= usedPlanes yield
    // defaultValue; a Resize fused behind it passes the value on as its float3 cast (iop_fuser.h:71-88)
    template <size_t N>
    static auto build(const int& usedPlanes, const T& defaultValue, const std::array<Ptr2D<T>, N>& ptrs) {
        auto r = build(ptrs);
        r.st.used_planes = usedPlanes;
        r.st.dflt[0] = static_cast<float>(defaultValue.x); r.st.dflt[1] = static_cast<float>(defaultValue.y); r.st.dflt[2] = static_cast<float>(defaultValue.z);
        r.st.dflt[3] = detail::w_of(defaultValue);
        return r;
    }
};
template <PixelFormat PF>
struct ReadYUV {
    static auto build(const Image<PF>& img) { return build(img.ptr()); }
    static auto build(const RawImage<PF>& raw) {
        static_assert(PixelFormatTraits<PF>::supported, "NV12, NV21, UYVY, P010, P210 and Y210 are the formats the B200 kernels read");
        detail::ReadState s;
        s.src_format = PixelFormatTraits<PF>::code;
        s.src.mut().push_back({raw.data.data, raw.data.dims.pitch, raw.width, raw.height});
        return ReadIOp<ColorDepthPixelType<PixelFormatTraits<PF>::depth>, 0>(std::move(s));
    }
};
// A batch whose planes are complete read chains of the same shape but different parameters (their own source,
// their own operands): the operands that differ travel per plane.
template <PlanePolicy PP = PlanePolicy::PROCESS_ALL>
struct BatchRead {
    template <typename O, size_t N>
    static auto build(const std::array<ReadIOp<O, 0>, N>& iops) {
        detail::ReadState s = iops[0].st;
        for (auto& op : s.ops) op.v.resize(N);
        if (!s.crops.empty()) s.crops.mut().resize(N);
        s.src.mut().resize(N);
        for (size_t i = 0; i < N; ++i) {
            const detail::ReadState& e = iops[i].st;
            if (e.ops.size() != s.ops.size() || e.src_format != s.src_format || e.has_resize != s.has_resize ||
                e.n_pre_ops != s.n_pre_ops || e.crops.empty() != iops[0].st.crops.empty() ||
                (e.has_resize && (e.dst_size.width != s.dst_size.width || e.dst_size.height != s.dst_size.height || e.ar != s.ar)))
                throw std::runtime_error("BatchRead: the planes are not chains of the same operations");
            s.src.mut()[i] = e.src[0];
            if (!e.crops.empty()) s.crops.mut()[i] = e.crops[0];
            for (size_t k = 0; k < s.ops.size(); ++k) {
                if (e.ops[k].code != s.ops[k].code) throw std::runtime_error("BatchRead: the planes are not chains of the same operations");
                s.ops[k].v[i] = e.ops[k].v[0];
            }
        }
        return ReadIOp<O, N>(std::move(s));
    }
};

// ---- Write IOps ------------------------------------------------------------------------------------------------
template <typename T>
struct WriteIOp {
    using InputType = T;
    uint32_t write_kind{FKB_WRITE_PACKED};
    void* data{nullptr};
    uint width{0}, height{0}, pitch{0}, planes{1};
    size_t plane_stride{0};    // bytes between consecutive planes (tensors)
    size_t channel_stride{0};  // TensorSplit: bytes between channel planes
    void* data_y{nullptr};     // SplitWrite: the second and third channel plane
    void* data_z{nullptr};
};
template <typename T> constexpr bool isWriteIOp = false;
template <typename T> constexpr bool isWriteIOp<WriteIOp<T>> = true;

template <ND D, typename T>
struct PerThreadWrite {
    static_assert(D == ND::_2D, "PerThreadWrite<ND::_2D, T> is the 2-D write the B200 kernels implement");
    static auto build(const RawPtr<ND::_2D, T>& p) { return WriteIOp<T>{FKB_WRITE_PACKED, p.data, p.dims.width, p.dims.height, p.dims.pitch, 1, 0, 0}; }
    static auto build(const Ptr<ND::_2D, T>& p) { return build(p.ptr()); }
};
template <typename T>
struct TensorWrite {
    static auto build(const RawPtr<ND::_3D, T>& p) {
        return WriteIOp<T>{FKB_WRITE_PACKED, p.data, p.dims.width, p.dims.height, p.dims.pitch, p.dims.planes,
                           static_cast<size_t>(p.dims.plane_pitch) * p.dims.color_planes, 0};
    }
    static auto build(const Ptr<ND::_3D, T>& p) { return build(p.ptr()); }
};
template <typename T>
struct TensorSplit {
    static_assert(std::is_same_v<T, float3> || std::is_same_v<T, uchar3>, "TensorSplit<float3|uchar3> are the planar writes the B200 kernels implement");
    using Base = std::conditional_t<std::is_same_v<T, float3>, float, uchar>;
    static auto build(const RawPtr<ND::_3D, Base>& p) {
        // memory_operations.h:189-205: channel c of pixel (x,y) lies width*height elements after channel c-1
        return WriteIOp<T>{FKB_WRITE_SPLIT, p.data, p.dims.width, p.dims.height, p.dims.pitch, p.dims.planes,
                           static_cast<size_t>(p.dims.plane_pitch) * p.dims.color_planes,
                           static_cast<size_t>(p.dims.width) * p.dims.height * sizeof(Base)};
    }
    static auto build(const Ptr<ND::_3D, Base>& p) { return build(p.ptr()); }
};
// (Y,Cb,Cr) byte triples into a YCbCr image (color_conversion.h:296-406).
template <PixelFormat PF>
struct WriteYUV {
    static_assert(PF == PixelFormat::NV12 || PF == PixelFormat::NV21 || PF == PixelFormat::UYVY, "NV12, NV21 and UYVY are the images the B200 kernels write");
    static auto build(const Image<PF>& img) { return build(img.ptr()); }
    static auto build(const RawImage<PF>& raw) {
        constexpr uint32_t kind = PF == PixelFormat::NV12 ? FKB_WRITE_NV12 : PF == PixelFormat::NV21 ? FKB_WRITE_NV21 : FKB_WRITE_UYVY;
        WriteIOp<uchar3> w{kind, raw.data.data, raw.width, raw.height, raw.data.dims.pitch, 1, 0, 0};
        if (PF != PixelFormat::UYVY) w.data_y = reinterpret_cast<uint8_t*>(raw.data.data) + static_cast<size_t>(raw.data.dims.pitch) * raw.height;
        return w;
    }
};
// Three separate 2-D planes, one per channel (memory_operations.h:360-393).
template <ND D, typename T>
struct SplitWrite {
    static_assert(D == ND::_2D && (std::is_same_v<T, float3> || std::is_same_v<T, uchar3>),
                  "SplitWrite<ND::_2D, float3|uchar3> is the split write the B200 kernels implement");
    using Base = std::conditional_t<std::is_same_v<T, float3>, float, uchar>;
    static auto build(const std::vector<Ptr2D<Base>>& output) {
        const auto x = output.at(0).ptr(), y = output.at(1).ptr(), z = output.at(2).ptr();
        if (y.dims.pitch != x.dims.pitch || z.dims.pitch != x.dims.pitch || y.dims.width != x.dims.width || z.dims.width != x.dims.width ||
            y.dims.height != x.dims.height || z.dims.height != x.dims.height)
            throw std::runtime_error("SplitWrite: the three planes must have the same size and pitch");
        WriteIOp<T> w{FKB_WRITE_SPLIT_PLANES, x.data, x.dims.width, x.dims.height, x.dims.pitch, 1, 0, 0};
        w.data_y = y.data; w.data_z = z.data;
        return w;
    }
};
// The same planar write into a colour-plane-transposed tensor (memory_operations.h:214-241): channel c of image z lies
// at c * color_planes_pitch + z * plane_pitch (core/data/rawptr.h:229-239).
template <typename T>
struct TensorTSplit {
    static_assert(std::is_same_v<T, float3> || std::is_same_v<T, uchar3>, "TensorTSplit<float3|uchar3> are the planar writes the B200 kernels implement");
    using Base = std::conditional_t<std::is_same_v<T, float3>, float, uchar>;
    static auto build(const RawPtr<ND::T3D, Base>& p) {
        return WriteIOp<T>{FKB_WRITE_SPLIT, p.data, p.dims.width, p.dims.height, p.dims.pitch, p.dims.planes,
                           static_cast<size_t>(p.dims.plane_pitch), static_cast<size_t>(p.dims.color_planes_pitch)};
    }
    static auto build(const Ptr<ND::T3D, Base>& p) { return build(p.ptr()); }
};

}  // namespace fk
