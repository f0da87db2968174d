/*
 * fkb.h — C ABI of the B200 (sm_100a) fused image-transform kernels.
 *
 * FusedKernelLibrary (FKL) is header-only C++: it has no ABI of its own.  A user lists
 * `Op::build(...)` objects and calls `fk::executeOperations<TransformDPP<>>(stream, iops...)`
 * (include/fused_kernel/fused_kernel.h:22-54); the type system turns the list into one templated
 * kernel (core/execution_model/executor_details/executor_kernels.h:20-30).  This header is the
 * boundary that sits beneath that source-level API in this library: the C++ front end
 * (include/fused_kernel/) lowers a built chain to the plain structs below and calls one of the
 * `fkb_launch_*` entry points.  Every struct is POD, every pointer is a plain device (or host)
 * address, no C++ or torch type crosses the boundary, and no entry point throws.
 *
 * What each piece replaces in the reference (paths relative to include/fused_kernel/):
 *   fkb_chain_desc   — the *types* of the IOps of one chain, i.e. the template argument list of
 *                      launchTransformDPP_Kernel (executor_kernels.h:26-30).
 *   fkb_plane_desc   — the *values*: one OperationData per batch plane as held by BatchRead
 *                      (core/execution_model/operation_model/batch_operations.h:101-105, 205-212):
 *                      RawPtr of the frame (core/data/rawptr.h:135-141), Crop rect
 *                      (algorithms/image_processing/crop.h:36-39), ResizeParams
 *                      (algorithms/image_processing/resize.h:44-58), and the RawPtr of the write
 *                      (algorithms/basic_ops/memory_operations.h:85-107, 160-212).
 *   fkb_launch_transform  — Executor<TransformDPP<GPU_NVIDIA>>::executeOperations_helper
 *                      (core/execution_model/executors.h:316-351).
 *   fkb_launch_divergent  — Executor<DivergentBatchTransformDPP<GPU_NVIDIA,Sel>>::executeOperations
 *                      (executors.h:360-411); the selector result is stored per plane
 *                      (fkb_plane_desc.chain, 0-based like Selector::at, data_parallel_patterns.h:322-331).
 *   fkb_resize_params — the host arithmetic of Resize<>::build (resize.h:164-233, 266-278).
 *
 * Arithmetic contract: every value inside a chain is carried as three fp32 numbers; the order of
 * operations is the reference's, without FMA contraction, with IEEE division, and
 * SaturateCast rounds half to even (core/constexpr_libs/constexpr_saturate.h:28-150).  Results are
 * bit-identical to the reference CPU backend compiled with -O2 -ffp-contract=off.
 */
#ifndef FKB_FKB_H
#define FKB_FKB_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FKB_ABI_VERSION 3u
#define FKB_PLANE_DEFAULT 0x80000000u
#define FKB_MAX_OPS 12u          /* compute ops per chain */
#define FKB_MAX_PLANE_PARAMS 4u  /* per-plane float3 operands a chain may refer to */
#define FKB_MAX_CHAINS 8u        /* chains of one divergent launch */

/* Status codes.  0 is success; everything else is negative.  fkb_status_string() names them. */
enum {
    FKB_OK = 0,
    FKB_ERR_NULL = -1,          /* a required pointer is null */
    FKB_ERR_INVALID = -2,       /* a descriptor is inconsistent (sizes, pitches, rect outside the frame ...) */
    FKB_ERR_UNSUPPORTED = -3,   /* well-formed, but not a chain these kernels implement */
    FKB_ERR_CUDA = -4,          /* a CUDA runtime call failed; fkb_last_cuda_error() has the code */
    FKB_ERR_TOO_LARGE = -5,     /* more planes / bytes than the entry point accepts */
    FKB_ERR_DEVICE_WAIT = -6,   /* a bounded device-side wait gave up (reported by fkb_device_status) */
    FKB_ERR_DEVICE_CHECK = -7   /* the self-checking build of the library (compiled with -DFKB_DEBUG) found an address or a
                                   size outside its buffer, or misaligned, and skipped that access (reported by
                                   fkb_device_status); the release build has no such checks */
};

/* Pixel formats.  A source is U8C3 (PerThreadRead<_2D,uchar3>, memory_operations.h:27-38) or NV12
 * (ReadYUV<NV12>, algorithms/image_processing/color_conversion.h:219-238).  A destination is U8C3 or F32C3. */
enum { FKB_PIX_U8C3 = 1, FKB_PIX_F32C3 = 2, FKB_PIX_NV12 = 3,
       /* two more 8-bit sources of ReadYUV (color_conversion.h:240-268): NV21 is NV12 with the chroma bytes in the
        * order V,U; UYVY is one plane of 4-byte groups U Y0 V Y1 (two pixels), 2*width bytes per row, no src_chroma */
       FKB_PIX_NV21 = 4, FKB_PIX_UYVY = 5,
       /* a uchar4 source (PerThreadRead<_2D,uchar4>) of which the first three channels enter the chain: the alpha
        * channel is dropped, as ColorConversion<COLOR_BGRA2BGR | COLOR_RGBA2RGB> = Discard does (color_conversion.h:448-452;
        * with the BGRA2RGB / RGBA2BGR codes, :460-464, the chain also carries FKB_OP_REORDER_ZYX).  Where in the chain the
        * reference discards the channel does not change the other three: every op here acts per channel. */
       FKB_PIX_U8C4 = 6,
       /* Four-channel chains: a chain whose dst_format is U8C4 or F32C4 keeps all four channels of its U8C4 source to the
        * Write (PerThreadRead<_2D,uchar4> ... TensorWrite<uchar4 | float4>, e.g. tests/examples/compiler_explorer_example.h:23-46).
        * Its ops are Cast, Mul / Add / Sub / Div (fourth operands in op_w / params_w), BGRA<->RGBA (FKB_OP_REORDER_ZYX leaves the
        * fourth channel in place: VectorReorder<T,2,1,0,3>, color_conversion.h:472-476) and SaturateCast; the write is PACKED. */
       FKB_PIX_F32C4 = 7,
       /* Float sources: FKB_PIX_F32C3 as src_format is a packed float3 image or tensor plane (TensorRead<float3>,
        * memory_operations.h:124-157); FKB_PIX_F32P3 is three float planes, channel c at src + c * (src_chroma - src)
        * (TensorPack, memory_operations.h:243-290; TensorTPack, :292-335).  They feed chains that start in float: the copy sequence
        * of CircularTensor::update (core/data/circular_tensor.h:111-161) is such a chain without ops. */
       FKB_PIX_F32P3 = 8,
       /* 10-bit YCbCr sources of ReadYUV, 16-bit containers read as they are stored (color_conversion.h:219-238, 255-265):
        * P010 = NV12's layout with ushort samples (4:2:0), P210 the same with full-height chroma (4:2:2), Y210 one plane of
        * ushort4 groups Y0 U Y1 V.  src_pitch in bytes; P010 / P210 take src_chroma.  The matrix and offsets of their
        * FKB_OP_YUV2RGB come from fkb_ycbcr_to_rgb_bits(10, ...). */
       FKB_PIX_P010 = 9, FKB_PIX_P210 = 10, FKB_PIX_Y210 = 11,
       /* One-channel destinations (PerThreadWrite<_2D, uchar | float>, TensorWrite<uchar | float>): what a chain writes
        * after FKB_OP_RGB2GRAY has reduced it to one channel.  As dst_format only; the write is PACKED. */
       FKB_PIX_U8C1 = 12, FKB_PIX_F32C1 = 13 };

/* Geometry of the ReadBack stage.  The crop rectangle is always applied (a chain without Crop
 * passes the whole frame as the rectangle).  NONE: output pixel (x,y) reads crop pixel (x,y).
 * RESIZE_*: bilinear INTER_LINEAR through the parameters of fkb_resize_params. */
enum { FKB_GEOM_NONE = 0, FKB_GEOM_RESIZE_IGNORE_AR = 1, FKB_GEOM_RESIZE_PRESERVE_AR = 2,
       /* the two other letterbox placements of the reference (resize.h:42): the target width rounded down to an even
        * number (resize.h:212-222), and the image flush with the left edge (resize.h:176-189).  On the device they are
        * PRESERVE_AR with other x1..y2; only fkb_resize_params tells them apart. */
       FKB_GEOM_RESIZE_PRESERVE_AR_RN_EVEN = 3, FKB_GEOM_RESIZE_PRESERVE_AR_LEFT = 4 };

/* BorderType of the reference (border_reader.h:25-36), shifted by one so that 0 means "no BorderReader". */
enum { FKB_BORDER_NONE = 0, FKB_BORDER_CONSTANT = 1, FKB_BORDER_REPLICATE = 2, FKB_BORDER_REFLECT = 3, FKB_BORDER_WRAP = 4,
       FKB_BORDER_REFLECT_101 = 5 };

/* Write kinds.  PACKED: interleaved pixels in pitched rows — PerThreadWrite<_2D,T> and
 * TensorWrite<T> (memory_operations.h:85-107, 160-179).  SPLIT: TensorSplit<float3>
 * (memory_operations.h:182-212): channel c of pixel (x,y) at dst + c*dst_channel_stride + y*dst_pitch + x*4. */
enum { FKB_WRITE_PACKED = 1, FKB_WRITE_SPLIT = 2,
       /* SplitWrite<_2D,T> (memory_operations.h:360-393): three unrelated planes dst (x), dst_y, dst_z, one base element
        * per pixel each, all with the pitch dst_pitch */
       FKB_WRITE_SPLIT_PLANES = 3,
       /* WriteYUV<NV12|NV21|UYVY> (color_conversion.h:296-406) of (Y,Cb,Cr) byte triples; dst_format is U8C3.
        * NV12 / NV21: dst is the luma plane, dst_y the interleaved chroma rows (reference: dst + pitch * height), both
        * with the pitch dst_pitch.  NV12 takes the chroma pair of the pixel with even x and even y.  The reference's
        * NV21 branch lets every pixel of a 2x2 block store its pair (the last store wins; on its CPU backend that is the
        * last pixel of the block in raster order) — that pixel is the one written here.  UYVY: dst holds U Y0 V Y1
        * groups, U and V from the even pixel. */
       FKB_WRITE_NV12 = 4, FKB_WRITE_NV21 = 5, FKB_WRITE_UYVY = 6 };

/* Compute ops.  The value type is tracked like the reference's Input/OutputType: it starts as
 * uchar3, ops that need float3 are rejected on uchar3 and vice versa. */
enum {
    FKB_OP_CAST_F32 = 1,     /* Cast<uchar3,float3>            (basic_ops/cast.h:22-33)            u8 -> f32 */
    FKB_OP_MUL = 2,          /* Mul<float3>: in * v            (basic_ops/arithmetic.h:23-137)     f32 */
    FKB_OP_ADD = 3,          /* Add<float3>: in + v                                                f32 */
    FKB_OP_SUB = 4,          /* Sub<float3>: in - v                                                f32 */
    FKB_OP_DIV = 5,          /* Div<float3>: in / v, IEEE                                          f32 */
    FKB_OP_REORDER_ZYX = 6,  /* ColorConversion<COLOR_BGR2RGB|COLOR_RGB2BGR> = VectorReorder<T,2,1,0>
                                (color_conversion.h:473-476, basic_ops/vector_ops.h:43-56)         any */
    FKB_OP_YUV2RGB = 7,      /* ConvertYUVToRGB<p8bit,CR,CP> (color_conversion.h:150-174): subtracts
                                chain.yuv_sub, multiplies by chain.ccm rows, sums (x+y)+z          u8 -> f32 */
    FKB_OP_SATCAST_U8 = 8,   /* SaturateCast<float3,uchar3>    (image_processing/saturate.h:25-36) f32 -> u8 */
    FKB_OP_RGB2YUV = 9,      /* ConvertRGBToYUV<p8bit,CR,CP> (color_conversion.h:176-199): ccm2 x (R,G,B), then adds
                                yuv_add to (Y,Cb,Cr)                                                   u8 -> f32 */
    FKB_OP_RGB2GRAY = 11,    /* RGB2Gray<I,O,CCIR_601> (color_conversion.h:46-79), also the second half of
                                ColorConversion<COLOR_BGR2GRAY | COLOR_BGRA2GRAY> (after FKB_OP_REORDER_ZYX; :484-502):
                                (x * 0.299f + y * 0.587f) + z * 0.114f in fp32, then rounded to the nearest integer, ties
                                to even — for every output type: the reference rounds whenever std::is_signed_v<O> or
                                std::is_unsigned_v<O> holds, and std::is_signed_v<float> does, so its float result is the
                                rounded luminance too (std::nearbyint on the host, __float2int_rn on the device).
                                v[0] != 0: the result is a uchar (O = uchar, from a uchar3 / uchar4 input only);
                                v[0] == 0: it is a float (O = float).
                                From here on the chain carries ONE channel: Mul / Add / Sub / Div use v[0] only,
                                SaturateCast acts on that channel, and the destination is FKB_PIX_U8C1 / F32C1.
                                At most once per chain, after the interpolation when the geometry is a RESIZE.     any */
    FKB_OP_ADD_ALPHA = 10    /* AddOpaqueAlpha<I,CD> (color_conversion.h:81-94), the second half of
                                ColorConversion<COLOR_BGR2BGRA|COLOR_RGB2RGBA> (and, after FKB_OP_REORDER_ZYX, of
                                COLOR_BGR2RGBA|COLOR_RGB2BGRA): appends a fourth channel v[0] = maxDepthValue<CD> (255
                                for p8bit, 1 for fn8bit).  Exactly once in a chain from a three-channel source
                                (FKB_PIX_U8C3) to a four-channel write; ops before it work on three channels,
                                ops after it on four                                                any */
};

typedef struct fkb_op {
    uint16_t code;       /* FKB_OP_* */
    int16_t plane_slot;  /* -1: operand is v[]; k >= 0: operand is planes[z].params[k] (per-plane values, as
                            when the op was fused into each plane's Read with .then()) */
    float v[3];
} fkb_op;

typedef struct fkb_chain_desc {
    uint32_t src_format;  /* FKB_PIX_U8C3 | FKB_PIX_NV12 */
    uint32_t geometry;    /* FKB_GEOM_* */
    uint32_t dst_format;  /* FKB_PIX_U8C3 | FKB_PIX_F32C3 */
    uint32_t write_kind;  /* FKB_WRITE_* */
    uint32_t n_ops;       /* <= FKB_MAX_OPS */
    uint32_t n_pre_ops;   /* ops[0..n_pre_ops) were fused into the Read: with a RESIZE geometry they run on each of
                             the four source taps before the interpolation; the rest run on the interpolated value */
    fkb_op ops[FKB_MAX_OPS];
    float ccm[9];         /* FKB_OP_YUV2RGB: row-major 3x3 (algorithms/image_processing/itu_color.h:185-258) */
    float yuv_sub[3];     /* FKB_OP_YUV2RGB: subtracted from (Y,U,V) first; Full range 8 bit = (0,128,128) */
    float ccm2[9];        /* FKB_OP_RGB2YUV: row-major 3x3 (itu_color.h:185-258, direction RGB2YCbCr) */
    float yuv_add[3];     /* FKB_OP_RGB2YUV: added to (Y,Cb,Cr) afterwards; Full range 8 bit = (0,128,128) */
    uint32_t border;      /* FKB_BORDER_*: a BorderReader between the Read and the Crop
                             (algorithms/image_processing/border_reader.h:25-334).  With one, the crop rectangle may leave
                             the frame: a frame coordinate outside [0,src_w) x [0,src_h) is remapped by the mode, or
                             (CONSTANT) the read yields border_value.  crop_x / crop_y are then taken as signed, as
                             Crop::exec casts them (crop.h:36-39). */
    uint32_t border_at;   /* ops[0..border_at) sit before the BorderReader (border_at <= n_pre_ops with a RESIZE
                             geometry): CONSTANT's value replaces their result, the later ops still run on it */
    float border_value[3];
    float op_w[FKB_MAX_OPS]; /* four-channel chains: the fourth operand of ops[i] (v holds the first three) */
    float border_value_w;    /* four-channel chains: the fourth channel of border_value */
} fkb_chain_desc;

typedef struct fkb_plane_desc {
    const void* src;         /* first byte of the source frame (Y plane for NV12) */
    const void* src_chroma;  /* NV12: first byte of the interleaved UV rows (reference: src + pitch*height); else null */
    void* dst;               /* first byte of this plane of the output */
    uint32_t src_pitch;      /* bytes between source rows (NV12: shared by the Y and the UV rows) */
    uint32_t src_w, src_h;   /* frame size in pixels */
    uint32_t crop_x, crop_y; /* Rect (core/data/rect.h:23-32): origin unsigned ... */
    int32_t crop_w, crop_h;  /* ... extent signed; must lie inside the frame */
    uint32_t dst_w, dst_h;   /* pixels this plane writes */
    uint32_t dst_pitch;      /* bytes between destination rows */
    uint64_t dst_channel_stride; /* FKB_WRITE_SPLIT: bytes between channel planes; else 0 */
    float fx, fy;            /* ResizeParams::src_conv_factors (resize.h:44-58); fx * dst_w and fy * dst_h must stay below
                                2^22 (source coordinates of four million and more are FKB_ERR_UNSUPPORTED) */
    int32_t x1, y1, x2, y2;  /* PRESERVE_AR: inclusive rectangle of the resized image inside dst */
    float bg[3];             /* PRESERVE_AR: ResizeParams::defaultValue outside that rectangle */
    uint32_t chain;          /* bits 0..30: divergent launch: which chain runs on this plane (0-based); else 0.
                                bit 31 (FKB_PLANE_DEFAULT): a plane beyond usedPlanes of
                                BatchRead<CONDITIONAL_WITH_DEFAULT> (batch_operations.h:221-281): its read — with a
                                RESIZE geometry, the resized read — yields bg for every pixel and the remaining ops
                                (all ops without a Resize, ops[n_pre_ops..) with one) run on that value; src, crop and
                                the resize parameters are ignored.  Without a Resize the read is uchar3, so bg must
                                hold integers in [0,255]. */
    float params[FKB_MAX_PLANE_PARAMS][3]; /* operands of ops whose plane_slot >= 0 */
    void* dst_y;             /* FKB_WRITE_SPLIT_PLANES: first byte of the second (FKB_WRITE_NV12/NV21: of the chroma rows) ... */
    void* dst_z;             /* ... and of the third channel plane; else unused */
    float bg_w;              /* four-channel chains: the fourth channel of bg ... */
    float params_w[FKB_MAX_PLANE_PARAMS]; /* ... and of params[slot] */
} fkb_plane_desc;

/* Fills plane->fx, fy, x1, y1, x2, y2 from plane->crop_w/crop_h (the size of the back operation) and
 * plane->dst_w/dst_h, exactly as Resize<INTER_LINEAR,AR>::build does on the host (resize.h:164-233 for
 * the PRESERVE_AR family, 266-278 for IGNORE_AR).  geometry = FKB_GEOM_RESIZE_*. */
int fkb_resize_params(uint32_t geometry, fkb_plane_desc* plane);

/* The 8-bit YCbCr -> RGB matrix (row-major) and the offsets subtracted from (Y,Cb,Cr) first, as ConvertYUVToRGB
 * <p8bit, range, primitives> evaluates them in fp32 (itu_color.h:112-124, 142-153, 185-258; color_conversion.h:150-174):
 * goes into fkb_chain_desc.ccm / yuv_sub of a chain with FKB_OP_YUV2RGB. */
enum { FKB_RANGE_LIMITED = 0, FKB_RANGE_FULL = 1 };
enum { FKB_PRIMITIVES_BT601 = 0, FKB_PRIMITIVES_BT709 = 1, FKB_PRIMITIVES_BT2020 = 2 };
int fkb_ycbcr_to_rgb(uint32_t range, uint32_t primitives, float ccm[9], float yuv_sub[3]);
/* The same for a colour depth of 8, 10 or 12 bits (maxDepthValue, subCoefficients and rangeLimits of itu_color.h:104-171). */
int fkb_ycbcr_to_rgb_bits(uint32_t bits, uint32_t range, uint32_t primitives, float ccm[9], float yuv_sub[3]);
/* The other direction, for fkb_chain_desc.ccm2 / yuv_add of a chain with FKB_OP_RGB2YUV (ConvertRGBToYUV). */
int fkb_rgb_to_ycbcr(uint32_t range, uint32_t primitives, float ccm2[9], float yuv_add[3]);

/* Host-only check of a launch: pointer, size, pitch, rectangle, type-flow and chain-index rules.
 * Launches run it first and return its code.  Needs no GPU. */
int fkb_validate(const fkb_chain_desc* chains, uint32_t n_chains,
                 const fkb_plane_desc* planes, uint32_t n_planes);

/* One fused launch of `chain` over n_planes planes (plane z uses planes[z]); replaces
 * executeOperations<TransformDPP<>> (executors.h:316-351).  `planes` is a host array, copied before the
 * call returns.  Asynchronous on `cuda_stream` (a cudaStream_t; null = legacy default stream), on the
 * current device; the caller keeps src/dst alive until the stream has run the work.
 * Stream capture: a launch of at most 8 planes carries its plane records in the kernel parameters and can be recorded
 * into a CUDA graph like any kernel launch.  A larger launch stages its records through buffers the library reuses from
 * call to call, which a recorded graph would read again at every replay; on a capturing stream such a launch returns
 * FKB_ERR_UNSUPPORTED and records nothing.  To put a large launch into a graph, create a plan and record fkb_plan_launch.
 * Ordering: the usual stream order.  The kernels of launches of 200 000 output pixels and more are submitted with
 * programmatic stream serialisation allowed, so that the GPU may set such a kernel up while an earlier kernel of this
 * library is still running; every kernel waits for the completion (and the visibility of the writes) of the kernel
 * before it in the stream before it reads a source or writes a destination (only plane records, which the host writes,
 * may be read earlier), so a launch may consume what the previous launch or any other earlier work in the stream
 * produced.  FKB_PDL=0 in the environment switches the attribute off. */
int fkb_launch_transform(const fkb_chain_desc* chain, const fkb_plane_desc* planes,
                         uint32_t n_planes, void* cuda_stream);

/* The same launch as fkb_launch_transform for callers that must not allocate.  (No counterpart in the reference: it is
 * an addition of this library.)  Some users of these kernels run where creating memory is off the table once start-up
 * is over: a process whose GPU memory was handed out in full to a pool or to other tenants, a service with a
 * no-allocation rule on its steady-state path, code between two points where the CUDA runtime refuses allocation calls.
 * fkb_launch_transform keeps its plane records in device and pinned buffers that it creates and grows on demand; this
 * entry point instead keeps them in a fixed array that is part of the library image on every GPU, and calls neither
 * cudaMalloc / cudaMallocHost / cudaFree nor any other allocating routine, on the device or on the host.
 *   - Limit: at most FKB_NOALLOC_MAX_PLANES planes per call; more returns FKB_ERR_TOO_LARGE and launches nothing.
 *   - Cost: FKB_NOALLOC_MAX_PLANES * 224 bytes (896 KB) of device memory on each GPU that loads the library, and the
 *     same again in host memory, until the process exits, whether or not this entry point is ever called.
 *   - The first call on a device looks up the array's device address (one cudaGetSymbolAddress, with that device
 *     current), and the first launch of each kernel lets the CUDA runtime load that kernel, which may allocate inside
 *     the driver.  Make one warm-up call per chain shape you will use before the window in which nothing may allocate,
 *     and before any stream capture begins.
 *   - On a capturing stream the call returns FKB_ERR_UNSUPPORTED (its copy of the records out of the shared host array
 *     cannot be replayed).
 *   - Planes of a conditional batch read (FKB_PLANE_DEFAULT) are accepted, as by fkb_launch_transform.
 *   - All calls share the one array.  A call overwrites every record it uses, so nothing has to be cleared, but two
 *     calls whose GPU work can overlap (different streams, no dependency between them) race on it: keep calls to this
 *     entry point ordered on the GPU, or use fkb_launch_transform / a plan for concurrent launches.
 * Source and destination buffers are still the caller's, as everywhere else in this header. */
#define FKB_NOALLOC_MAX_PLANES 4096u
int fkb_launch_transform_noalloc(const fkb_chain_desc* chain, const fkb_plane_desc* planes,
                                 uint32_t n_planes, void* cuda_stream);

/* One fused launch where plane z runs chains[planes[z].chain]; replaces
 * Executor<DivergentBatchTransformDPP<>>::executeOperations (executors.h:360-411). */
int fkb_launch_divergent(const fkb_chain_desc* chains, uint32_t n_chains,
                         const fkb_plane_desc* planes, uint32_t n_planes, void* cuda_stream);

/* A plan keeps the lowered launch (descriptor table, tile schedule) resident on the device so that a
 * pipeline that repeats the same launch pays the lowering once.  fkb_plan_launch is asynchronous and may be recorded
 * into a CUDA graph.  The reference rebuilds its IOps on every call (executors.h:53-58); a plan is the same launch, cached.
 * Launches of one plan may overlap on the GPU (different streams): each takes its own pair of work counters from a ring
 * of 64, so up to 64 launches of one plan can be in flight at a time.  They all write the same destination buffers. */
typedef struct fkb_plan fkb_plan;
int fkb_plan_create(const fkb_chain_desc* chains, uint32_t n_chains,
                    const fkb_plane_desc* planes, uint32_t n_planes, fkb_plan** out);
int fkb_plan_launch(const fkb_plan* plan, void* cuda_stream);  /* FKB_ERR_INVALID when the current device is not the plan's */
void fkb_plan_destroy(fkb_plan* plan);
/* Kernel launches one fkb_plan_launch issues (for launch accounting). */
uint32_t fkb_plan_kernel_launches(const fkb_plan* plan);

/* Reads and clears the device-side status word of the current device (synchronises the device).
 * 0, or FKB_ERR_DEVICE_WAIT when a bounded wait on a bulk copy ran out in some earlier launch. */
int fkb_device_status(void);

/* cudaError_t of the most recent failing CUDA call on this thread (0 if none). */
int fkb_last_cuda_error(void);
const char* fkb_status_string(int status);
uint32_t fkb_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FKB_FKB_H */
