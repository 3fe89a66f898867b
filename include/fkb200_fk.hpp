/* fkb200_fk.hpp - the reference's operation vocabulary on top of the fkb200 C ABI (header-only, C++17).
 *
 * User code written against FusedKernelLibrary's fused-execution path
 *
 *     const auto sender = PerThreadRead<ND::_2D, uchar3>::build(image)
 *         .then(Crop<>::build(crops))
 *         .then(Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(size, background))
 *         .then(Mul<float3>::build(m)).then(Sub<float3>::build(s)).then(Div<float3>::build(d))
 *         .then(ColorConversion<ColorConversionCodes::COLOR_RGB2BGR, float3, float3>::build());
 *     executeOperations<TransformDPP<>>(stream, sender, TensorWrite<float3>::build(output));
 *     stream.sync();
 *
 * (tests/examples/readme_test_code.h:25-71 of the reference) compiles against this header with
 * `using namespace fkb200::fk;` and runs on the library's kernels.  Names, argument meaning and
 * error behaviour follow the reference: build() factories (operation_model/parent_operations.h),
 * .then() chaining (instantiable_operations.h:44-52), batch forms taking std::array (batch_operations.h:
 * 408-421), errors as std::runtime_error (core/utils/utils.h:95-109).  What differs: a chain is a
 * run-time value here, so a chain the reference would reject at compile time (arithmetic on a
 * uchar3 value, a receiver of the wrong element type) is rejected when it is executed; and images are
 * non-owning views (RawPtr, core/data/rawptr.h:124-157) over memory the caller allocated - the owning
 * Ptr2D/Tensor classes of the reference (core/data/ptr_nd.h) are outside this path.
 *
 * Only the operations of the fused-execution path are here: PerThreadRead, ReadYUV<NV12 | NV21 | P010 | P210 | Y210 | UYVY> +
 * ConvertYUVToRGB<PF, Full, bt709 | bt601 | bt2020>, Crop, Resize<INTER_LINEAR, IGNORE_AR | PRESERVE_AR |
 * PRESERVE_AR_RN_EVEN | PRESERVE_AR_LEFT>, BorderReader, Deinterlace, Warping, Mul/Sub/Div/Add, Cast,
 * SaturateCast, ColorConversion<RGB2BGR | BGR2RGB>, PerThreadWrite, TensorWrite, TensorSplit, batches, and
 * divergent batches (several chains in one launch).
 */
#ifndef FKB200_FK_HPP
#define FKB200_FK_HPP

#include <array>
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "fkb200.h"

#if defined(__has_include)
#if __has_include(<vector_types.h>)
#include <vector_types.h>
#define FKB200_HAVE_CUDA_VECTOR_TYPES 1
#endif
#endif
#ifndef FKB200_HAVE_CUDA_VECTOR_TYPES
#define FKB200_HAVE_CUDA_VECTOR_TYPES 0
#endif

namespace fkb200 {
namespace fk {

/* ---- vector and geometry types (core/data/vector_types.h, point.h, size.h, rect.h) ---- */
#if FKB200_HAVE_CUDA_VECTOR_TYPES
using ::uchar3; /* CUDA's own, as in the reference's GPU build */
using ::float3;
#else
struct uchar3 { unsigned char x, y, z; }; /* host stand-ins, as in the reference's CPU build (vector_types.h:67-314) */
struct float3 { float x, y, z; };
#endif
template <typename T> inline T make_set(float v);
template <> inline float3 make_set<float3>(float v) { return float3{v, v, v}; }
template <typename T> inline T make_(float x, float y, float z);
template <> inline float3 make_<float3>(float x, float y, float z) { return float3{x, y, z}; }

struct Size { int width, height; Size(int w = 0, int h = 0) : width(w), height(h) {} };
/* x and y are unsigned as in the reference (core/data/rect.h:38); a crop above a BorderReader that starts outside the
   image is written Rect(-7, -5, w, h) there too, and the origin wraps back when it is added to the signed thread index */
struct Rect { unsigned x, y; int width, height; Rect(unsigned x_ = 0, unsigned y_ = 0, int w = 0, int h = 0) : x(x_), y(y_), width(w), height(h) {} };

enum class ND { _2D, _3D };
enum class InterpolationType { INTER_LINEAR };
enum class AspectRatio { PRESERVE_AR, IGNORE_AR, PRESERVE_AR_RN_EVEN, PRESERVE_AR_LEFT };
enum class ColorConversionCodes { COLOR_RGB2BGR, COLOR_BGR2RGB };
enum class PixelFormat { NV12, NV21, P010, P210, Y210, UYVY };
enum class ColorRange { Full };
enum class ColorPrimitives { bt601, bt709, bt2020 };
enum class BorderType { CONSTANT, REPLICATE, REFLECT, WRAP, REFLECT_101 };
enum class DeinterlaceType { BLEND, INTER_LINEAR };
enum class DeinterlaceLinear : bool { USE_EVEN = true, USE_ODD = false };
enum class WarpType { Affine, Perspective };
enum class ParArch { GPU_NVIDIA };
template <ParArch PA = ParArch::GPU_NVIDIA> struct TransformDPP {};

/* ---- non-owning image views (core/data/rawptr.h) ---- */
template <typename T> struct RawPtr2D { T* data; unsigned width, height, pitch; }; /* pitch in bytes */
template <typename T> struct RawTensor { T* data; unsigned width, height, planes, pitch; };          /* dense planes */
/* An NV12 frame: `height` luma rows, then height/2 rows of interleaved U,V, same pitch
   (color_conversion.h:336-341 with an Image whose dims.height is the frame height). */
struct ImageNV12 { const unsigned char* data; unsigned width, height, pitch; };
using ImageNV21 = ImageNV12; /* the same layout with V before U in the chroma rows */
/* Any other layout of ReadYUV (raw_image.h:48-106): `data` is the first plane, `pitch` the bytes between its rows; P010 and
   P210 keep their interleaved chroma rows behind the `height` luma rows, Y210 and UYVY are one packed plane. */
using ImageYUV = ImageNV12;

inline void check(int status) {
    if (status != FKB_OK) throw std::runtime_error(std::string(fkb_last_error()[0] ? fkb_last_error() : fkb_status_string(status)));
}

/* ---- stream (core/execution_model/stream.h:52-109): wraps a cudaStream_t the caller created ---- */
class Stream {
public:
    explicit Stream(void* cuda_stream = nullptr) : stream_(cuda_stream) {}
    Stream(const Stream&) = delete;
    Stream& operator=(const Stream&) = delete;
    ~Stream() { try { sync(); } catch (...) {} }
    void* getCUDAStream() const { return stream_; }
    /* Waits for the launches made on the stream; throws if a kernel gave up a bounded wait. */
    void sync() { check(fkb_async_check(stream_, nullptr)); }
private:
    void* stream_;
};

/* ---- the chain as a value ---- */
struct SourcePlane { const void* data; unsigned width, height, pitch; Rect crop; bool cropped; };
struct Sender {
    int src_format = 0;
    std::vector<SourcePlane> planes;
    int resize_mode = FKB_RESIZE_NONE;
    Size dst_size;
    float background[3] = {0.f, 0.f, 0.f};
    std::vector<fkb_op> ops;
    int n_pre_ops = 0;
    bool value_is_float = false, value_is_yuv = false;
    int border_mode = FKB_BORDER_NONE, deinterlace = FKB_DEINTERLACE_NONE;
    float border_value[3] = {0.f, 0.f, 0.f};
    float transform[9] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};

    template <typename Continuation> Sender then(const Continuation& c) const { Sender s = *this; c.apply(s); return s; }
};

namespace detail {
inline fkb_op make_op(int opcode, float3 p = float3{0.f, 0.f, 0.f}) { fkb_op o; o.opcode = opcode; o.p[0] = p.x; o.p[1] = p.y; o.p[2] = p.z; return o; }
struct Continuation { fkb_op op; bool needs_float; bool yields_float; bool yields_u8;
    void apply(Sender& s) const {
        if (needs_float && !s.value_is_float) throw std::runtime_error("fkb200: arithmetic on a value that is not float3 (add Cast<uchar3, float3> first)");
        s.ops.push_back(op);
        if (yields_float) { s.value_is_float = true; s.value_is_yuv = false; }
        if (yields_u8) s.value_is_float = false;
    } };
}  // namespace detail

/* ---- reads (core/execution_model/memory_operations.h:71-112, color_conversion.h:314-400) ---- */
template <ND D, typename T> struct PerThreadRead;
template <> struct PerThreadRead<ND::_2D, uchar3> {
    static Sender build(const RawPtr2D<uchar3>& img) { return build(std::array<RawPtr2D<uchar3>, 1>{img}); }
    template <size_t B> static Sender build(const std::array<RawPtr2D<uchar3>, B>& imgs) {
        Sender s; s.src_format = FKB_SRC_U8X3;
        for (const auto& i : imgs) s.planes.push_back(SourcePlane{i.data, i.width, i.height, i.pitch, Rect(), false});
        return s;
    }
};
template <> struct PerThreadRead<ND::_2D, float3> {
    static Sender build(const RawPtr2D<float3>& img) { return build(std::array<RawPtr2D<float3>, 1>{img}); }
    template <size_t B> static Sender build(const std::array<RawPtr2D<float3>, B>& imgs) {
        Sender s; s.src_format = FKB_SRC_F32X3; s.value_is_float = true;
        for (const auto& i : imgs) s.planes.push_back(SourcePlane{i.data, i.width, i.height, i.pitch, Rect(), false});
        return s;
    }
};
template <PixelFormat PF> struct ReadYUV {
    static Sender build(const ImageNV12& img) { return build(std::array<ImageNV12, 1>{img}); }
    template <size_t B> static Sender build(const std::array<ImageNV12, B>& imgs) {
        Sender s; s.value_is_yuv = true;
        s.src_format = PF == PixelFormat::NV12 ? FKB_SRC_NV12 : PF == PixelFormat::NV21 ? FKB_SRC_NV21 : PF == PixelFormat::P010 ? FKB_SRC_P010
                       : PF == PixelFormat::P210 ? FKB_SRC_P210 : PF == PixelFormat::Y210 ? FKB_SRC_Y210 : FKB_SRC_UYVY;
        for (const auto& i : imgs) s.planes.push_back(SourcePlane{i.data, i.width, i.height, i.pitch, Rect(), false});
        return s;
    }
};

/* ---- read-back operations (image_processing/crop.h, resize.h) ---- */
struct CropContinuation { std::vector<Rect> rects;
    void apply(Sender& s) const {
        if (s.resize_mode != FKB_RESIZE_NONE) throw std::runtime_error("fkb200: Crop after Resize is not on this path");
        /* fuseAllIOps (iop_fuser.h:77-88): one image is replicated over the batch of rects */
        if (s.planes.size() == 1 && rects.size() > 1) s.planes.resize(rects.size(), s.planes[0]);
        if (s.planes.size() != rects.size()) throw std::runtime_error("fkb200: batch sizes of the read and of Crop differ");
        for (size_t i = 0; i < rects.size(); ++i) { s.planes[i].crop = rects[i]; s.planes[i].cropped = true; }
    } };
template <typename = void> struct Crop {
    static CropContinuation build(const Rect& r) { return CropContinuation{{r}}; }
    template <size_t B> static CropContinuation build(const std::array<Rect, B>& r) { return CropContinuation{std::vector<Rect>(r.begin(), r.end())}; }
};
struct ResizeContinuation { int mode; Size size; float3 background;
    void apply(Sender& s) const {
        if (s.resize_mode != FKB_RESIZE_NONE) throw std::runtime_error("fkb200: two Resize operations in one chain");
        s.resize_mode = mode; s.dst_size = size;
        s.background[0] = background.x; s.background[1] = background.y; s.background[2] = background.z;
        s.n_pre_ops = (int)s.ops.size();   /* what came before runs on every tap (backwards vertical fusion) */
        s.value_is_float = true; s.value_is_yuv = false; /* Interpolate returns float (interpolation.h:55-57) */
    } };
template <InterpolationType I, AspectRatio AR = AspectRatio::IGNORE_AR> struct Resize {
    static constexpr int MODE = AR == AspectRatio::PRESERVE_AR ? FKB_RESIZE_PRESERVE_AR
                                : AR == AspectRatio::PRESERVE_AR_RN_EVEN ? FKB_RESIZE_PRESERVE_AR_RN_EVEN
                                : AR == AspectRatio::PRESERVE_AR_LEFT ? FKB_RESIZE_PRESERVE_AR_LEFT : FKB_RESIZE_IGNORE_AR;
    static ResizeContinuation build(const Size& dst) { return ResizeContinuation{MODE, dst, float3{0.f, 0.f, 0.f}}; }
    static ResizeContinuation build(const Size& dst, const float3& background) { return ResizeContinuation{MODE, dst, background}; }
};
/* BorderReader<BT>::build(read[, value]) (image_processing/border_reader.h:46-87): wraps the image read, so that a Crop
   above it may reach beyond the image */
template <BorderType BT> struct BorderReader {
    static constexpr int MODE = BT == BorderType::CONSTANT ? FKB_BORDER_CONSTANT : BT == BorderType::REPLICATE ? FKB_BORDER_REPLICATE
                                : BT == BorderType::REFLECT ? FKB_BORDER_REFLECT : BT == BorderType::WRAP ? FKB_BORDER_WRAP : FKB_BORDER_REFLECT_101;
    static Sender wrap(const Sender& read) {
        if (read.value_is_yuv || !read.ops.empty() || read.resize_mode != FKB_RESIZE_NONE || read.border_mode != FKB_BORDER_NONE ||
            read.deinterlace != FKB_DEINTERLACE_NONE)
            throw std::runtime_error("fkb200: BorderReader anywhere but directly above PerThreadRead is not on this path");
        for (const auto& p : read.planes) if (p.cropped) throw std::runtime_error("fkb200: BorderReader above a Crop is not on this path");
        Sender s = read; s.border_mode = MODE; return s;
    }
    static Sender build(const Sender& read) {
        static_assert(BT != BorderType::CONSTANT, "a CONSTANT border needs its value");
        return wrap(read);
    }
    template <typename V> static Sender build(const Sender& read, const V& value) {
        static_assert(BT == BorderType::CONSTANT, "only a CONSTANT border takes a value");
        Sender s = wrap(read); s.border_value[0] = (float)value.x; s.border_value[1] = (float)value.y; s.border_value[2] = (float)value.z; return s;
    }
};
/* Deinterlace<DT>::build([which field,] read) (image_processing/deinterlace.h:133-183); the value becomes float3 */
template <DeinterlaceType DT> struct Deinterlace {
    static Sender wrap(const Sender& read, int mode) {
        if (read.value_is_yuv || !read.ops.empty() || read.resize_mode != FKB_RESIZE_NONE || read.border_mode != FKB_BORDER_NONE ||
            read.deinterlace != FKB_DEINTERLACE_NONE)
            throw std::runtime_error("fkb200: Deinterlace anywhere but directly above PerThreadRead is not on this path");
        for (const auto& p : read.planes) if (p.cropped) throw std::runtime_error("fkb200: Deinterlace above a Crop is not on this path");
        Sender s = read; s.deinterlace = mode; s.value_is_float = true; return s;
    }
    static Sender build(const Sender& read) {
        static_assert(DT == DeinterlaceType::BLEND, "INTER_LINEAR needs DeinterlaceLinear::USE_EVEN or USE_ODD");
        return wrap(read, FKB_DEINTERLACE_BLEND);
    }
    static Sender build(DeinterlaceLinear field, const Sender& read) {
        static_assert(DT == DeinterlaceType::INTER_LINEAR, "only INTER_LINEAR chooses a field");
        return wrap(read, field == DeinterlaceLinear::USE_EVEN ? FKB_DEINTERLACE_LINEAR_EVEN : FKB_DEINTERLACE_LINEAR_ODD);
    }
};
/* Warping<WT>::build(params) (image_processing/warping.h:25-141): the matrix maps output to source coordinates */
template <WarpType WT> struct WarpingParameters { float transformMatrix[WT == WarpType::Affine ? 2 : 3][3]; Size dstSize; };
template <WarpType WT> struct WarpingContinuation { WarpingParameters<WT> params;
    void apply(Sender& s) const {
        if (s.resize_mode != FKB_RESIZE_NONE) throw std::runtime_error("fkb200: Warping after a Resize or another Warping is not on this path");
        if (s.value_is_yuv) throw std::runtime_error("fkb200: Warping over a YUV value is not on this path");
        s.resize_mode = WT == WarpType::Affine ? FKB_GEOMETRY_WARP_AFFINE : FKB_GEOMETRY_WARP_PERSPECTIVE;
        constexpr int rows = WT == WarpType::Affine ? 2 : 3;
        for (int r = 0; r < rows; ++r) for (int c = 0; c < 3; ++c) s.transform[3 * r + c] = params.transformMatrix[r][c];
        if (rows == 2) { s.transform[6] = 0.f; s.transform[7] = 0.f; s.transform[8] = 1.f; }
        s.dst_size = params.dstSize; s.n_pre_ops = (int)s.ops.size(); s.value_is_float = true;
    } };
template <WarpType WT> struct Warping { static WarpingContinuation<WT> build(const WarpingParameters<WT>& p) { return WarpingContinuation<WT>{p}; } };

/* ---- element-wise operations (basic_ops/arithmetic.h, cast.h, image_processing/saturate.h, color_conversion.h) ---- */
template <typename T> struct Mul { static detail::Continuation build(const float3& p) { return {detail::make_op(FKB_OP_MUL, p), true, false, false}; } };
template <typename T> struct Sub { static detail::Continuation build(const float3& p) { return {detail::make_op(FKB_OP_SUB, p), true, false, false}; } };
template <typename T> struct Div { static detail::Continuation build(const float3& p) { return {detail::make_op(FKB_OP_DIV, p), true, false, false}; } };
template <typename T> struct Add { static detail::Continuation build(const float3& p) { return {detail::make_op(FKB_OP_ADD, p), true, false, false}; } };
template <typename I, typename O> struct Cast;
template <> struct Cast<uchar3, float3> { static detail::Continuation build() { return {detail::make_op(FKB_OP_CAST_F32), false, true, false}; } };
template <typename I, typename O> struct SaturateCast;
template <> struct SaturateCast<float3, uchar3> { static detail::Continuation build() { return {detail::make_op(FKB_OP_SATURATE_CAST_U8), true, false, true}; } };
template <ColorConversionCodes CODE, typename I, typename O = I> struct ColorConversion {
    static detail::Continuation build() { return {detail::make_op(FKB_OP_SWAP_RB), false, false, false}; }
};
template <PixelFormat PF, ColorRange CR, ColorPrimitives CP, bool ALPHA = false, typename O = float3> struct ConvertYUVToRGB {
    static_assert(CR == ColorRange::Full && !ALPHA, "only full-range conversions without alpha are on this path");
    struct C { void apply(Sender& s) const {
        if (!s.value_is_yuv) throw std::runtime_error("fkb200: ConvertYUVToRGB needs the value read by ReadYUV");
        const int want = PF == PixelFormat::NV12 ? FKB_SRC_NV12 : PF == PixelFormat::NV21 ? FKB_SRC_NV21 : PF == PixelFormat::P010 ? FKB_SRC_P010
                         : PF == PixelFormat::P210 ? FKB_SRC_P210 : PF == PixelFormat::Y210 ? FKB_SRC_Y210 : FKB_SRC_UYVY;
        if (s.src_format != want) throw std::runtime_error("fkb200: ConvertYUVToRGB's pixel format differs from ReadYUV's");
        s.ops.push_back(detail::make_op(CP == ColorPrimitives::bt709 ? FKB_OP_YUV_TO_RGB_BT709_FULL
                                        : CP == ColorPrimitives::bt601 ? FKB_OP_YUV_TO_RGB_BT601_FULL : FKB_OP_YUV_TO_RGB_BT2020_FULL));
        s.value_is_yuv = false; s.value_is_float = true;
    } };
    static C build() { return C{}; }
};

/* ---- receivers (memory_operations.h:114-137,173-226) ---- */
struct Receiver { int dst_format; void* data; unsigned width, height, planes, pitch; };
template <ND D, typename T> struct PerThreadWrite;
template <> struct PerThreadWrite<ND::_2D, float3> { static Receiver build(const RawPtr2D<float3>& p) { return {FKB_DST_F32X3_PACKED, p.data, p.width, p.height, 1, p.pitch}; } };
template <> struct PerThreadWrite<ND::_2D, uchar3> { static Receiver build(const RawPtr2D<uchar3>& p) { return {FKB_DST_U8X3_PACKED, p.data, p.width, p.height, 1, p.pitch}; } };
template <typename T> struct TensorWrite;
template <> struct TensorWrite<float3> { static Receiver build(const RawTensor<float3>& t) { return {FKB_DST_F32X3_PACKED, t.data, t.width, t.height, t.planes, t.pitch}; } };
template <> struct TensorWrite<uchar3> { static Receiver build(const RawTensor<uchar3>& t) { return {FKB_DST_U8X3_PACKED, t.data, t.width, t.height, t.planes, t.pitch}; } };
/* planar N x 3 x H x W (memory_operations.h:203-219): the view is over float elements */
template <typename T> struct TensorSplit;
template <> struct TensorSplit<float3> { static Receiver build(const RawTensor<float>& t) { return {FKB_DST_F32_PLANAR3, t.data, t.width, t.height, t.planes, t.pitch}; } };

/* ---- execution (fused_kernel.h:22-54, executors.h:252-287) ---- */
namespace detail {
struct Lowered { std::vector<fkb_sequence> seqs; std::vector<fkb_plane> planes; };
inline void lower_into(const Sender& s, const Receiver& r, Lowered& out, std::vector<std::vector<fkb_op>>& op_store) {
    /* the reference rejects this at compile time (TensorWrite<float3> after a uchar3 value, ...) */
    const bool want_u8 = r.dst_format == FKB_DST_U8X3_PACKED;
    if (want_u8 == s.value_is_float) throw std::runtime_error("fkb200: the chain's value type does not match the receiver's element type");
    if (s.planes.size() != r.planes) throw std::runtime_error("fkb200: the chain has " + std::to_string(s.planes.size()) + " planes but the receiver " + std::to_string(r.planes));
    op_store.push_back(s.ops);
    fkb_sequence q{};
    q.src_format = s.src_format; q.dst_format = r.dst_format; q.resize_mode = s.resize_mode;
    q.n_ops = (int32_t)s.ops.size(); q.n_pre_ops = s.resize_mode == FKB_RESIZE_NONE ? 0 : s.n_pre_ops;
    q.background[0] = s.background[0]; q.background[1] = s.background[1]; q.background[2] = s.background[2];
    q.border_mode = s.border_mode; q.deinterlace = s.deinterlace;
    for (int k = 0; k < 3; ++k) q.border_value[k] = s.border_value[k];
    for (int k = 0; k < 9; ++k) q.transform[k] = s.transform[k];
    q.ops = nullptr; /* fixed up by the caller once op_store stops growing */
    const int seq_index = (int)out.seqs.size();
    out.seqs.push_back(q);
    const size_t plane_bytes = r.dst_format == FKB_DST_F32_PLANAR3 ? (size_t)r.pitch * r.height * 3 : (size_t)r.pitch * r.height;
    for (size_t i = 0; i < s.planes.size(); ++i) {
        const SourcePlane& sp = s.planes[i];
        fkb_plane p{};
        p.src = sp.data; p.src_width = sp.width; p.src_height = sp.height; p.src_pitch = sp.pitch;
        p.crop_x = sp.cropped ? (int)sp.crop.x : 0; p.crop_y = sp.cropped ? (int)sp.crop.y : 0;
        p.crop_width = sp.cropped ? sp.crop.width : (int)sp.width; p.crop_height = sp.cropped ? sp.crop.height : (int)sp.height;
        p.dst = static_cast<unsigned char*>(r.data) + i * plane_bytes;
        p.dst_width = r.width; p.dst_height = r.height; p.dst_pitch = r.pitch;
        p.dst_channel_stride = r.dst_format == FKB_DST_F32_PLANAR3 ? r.pitch * r.height : 0;
        p.sequence = seq_index;
        out.planes.push_back(p);
    }
}
inline void launch(Stream& stream, Lowered& low, std::vector<std::vector<fkb_op>>& op_store) {
    for (size_t k = 0; k < low.seqs.size(); ++k) low.seqs[k].ops = op_store[k].empty() ? nullptr : op_store[k].data();
    fkb_plan_desc d{low.seqs.data(), (int32_t)low.seqs.size(), low.planes.data(), (int32_t)low.planes.size()};
    /* lowering, one stream-ordered copy of the descriptor table from pinned memory, the launch: no
       allocation and no synchronisation, like the reference's launch site */
    check(fkb_execute_async(&d, stream.getCUDAStream()));
}
}  // namespace detail

/* One sender chain, one receiver: asynchronous on the stream, like the reference (executors.h:284-285). */
template <typename DPP = TransformDPP<>>
inline void executeOperations(Stream& stream, const Sender& sender, const Receiver& receiver) {
    detail::Lowered low;
    std::vector<std::vector<fkb_op>> op_store;
    detail::lower_into(sender, receiver, low, op_store);
    detail::launch(stream, low, op_store);
}

/* Divergent horizontal fusion (data_parallel_patterns.h:301-353): several chains, each with its own
   receiver, in one launch.  The reference has the device code but no host launcher for it. */
struct OperationSequence { Sender sender; Receiver receiver; };
inline OperationSequence buildOperationSequence(const Sender& s, const Receiver& r) { return OperationSequence{s, r}; }
template <typename DPP = TransformDPP<>>
inline void executeDivergentOperations(Stream& stream, const std::vector<OperationSequence>& sequences) {
    detail::Lowered low;
    std::vector<std::vector<fkb_op>> op_store;
    op_store.reserve(sequences.size());
    for (const auto& q : sequences) detail::lower_into(q.sender, q.receiver, low, op_store);
    detail::launch(stream, low, op_store);
}

/* ---- CircularTensor (core/data/circular_tensor.h:86-161): the newest BATCH results of a chain, kept in order ----
 * update(stream, sender, receiver) runs the sender once for the new image and leaves the tensor's planes as the last
 * BATCH results, newest first or oldest first, in one launch (fkb_circular_tensor_update).  The tensor owns its device
 * memory, like the reference's; ptr() is what TensorWrite / TensorSplit take as the receiver of update().  Only the
 * Standard colour-plane mode is here. */
enum class CircularTensorOrder { NewestFirst, OldestFirst };
enum class ColorPlanes { Standard };
template <typename T, int COLOR_PLANES, int BATCH, CircularTensorOrder CT_ORDER, ColorPlanes CP_MODE = ColorPlanes::Standard>
class CircularTensor {
    static_assert(COLOR_PLANES == 3 || COLOR_PLANES == 1, "three colour planes of a base type (TensorSplit) or one plane of a three-channel type (TensorWrite)");
public:
    CircularTensor(unsigned width, unsigned height, int dst_format) : width_(width), height_(height), dst_format_(dst_format) {
        fkb_circular_tensor_desc d{};
        d.width = width; d.height = height; d.batch = BATCH;
        d.order = CT_ORDER == CircularTensorOrder::NewestFirst ? FKB_CIRCULAR_NEWEST_FIRST : FKB_CIRCULAR_OLDEST_FIRST;
        d.dst_format = dst_format;
        check(fkb_circular_tensor_create(&d, &ct_));
    }
    CircularTensor(const CircularTensor&) = delete;
    CircularTensor& operator=(const CircularTensor&) = delete;
    ~CircularTensor() { fkb_circular_tensor_destroy(ct_); }
    /* the visible tensor as a receiver's view: BATCH dense planes */
    RawTensor<T> ptr() const {
        const unsigned px = dst_format_ == FKB_DST_U8X3_PACKED ? 3u : dst_format_ == FKB_DST_F32_PLANAR3 ? 4u : 12u;
        return RawTensor<T>{static_cast<T*>(fkb_circular_tensor_data(ct_)), width_, height_, (unsigned)BATCH, width_ * px};
    }
    void update(Stream& stream, const Sender& sender, const Receiver& receiver) {
        if (receiver.data != fkb_circular_tensor_data(ct_) || receiver.dst_format != dst_format_)
            throw std::runtime_error("fkb200: update() takes a receiver built on this tensor's ptr()");
        if (sender.planes.size() != 1) throw std::runtime_error("fkb200: update() takes the chain of one new image");
        detail::Lowered low;
        std::vector<std::vector<fkb_op>> op_store;
        Receiver one = receiver; one.planes = 1;
        detail::lower_into(sender, one, low, op_store);
        low.seqs[0].ops = op_store[0].empty() ? nullptr : op_store[0].data();
        check(fkb_circular_tensor_update(ct_, &low.seqs[0], &low.planes[0], stream.getCUDAStream()));
    }
private:
    fkb_circular_tensor* ct_ = nullptr;
    unsigned width_, height_;
    int dst_format_;
};

}  // namespace fk
}  // namespace fkb200

#endif /* FKB200_FK_HPP */
