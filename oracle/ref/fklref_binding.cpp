/* The reference-side binding (include/fkb200_executor.h) compiled against the UNMODIFIED reference headers.
 *
 * TEST INFRASTRUCTURE ONLY.  Compiled by oracle/Makefile with nvcc (the reference defines
 * Stream_<ParArch::GPU_NVIDIA> only there) into oracle/_ref/libfklref_binding.so, which links
 * libfkb200.so.  Every entry point builds a sender chain with the reference's REAL types, exactly as
 * a user of the reference writes it - PerThreadRead<_2D, uchar3>::build(...).then(Crop<>::build(...))
 * .then(Resize<...>::build(...))... - and then either
 *   mode 0: runs it with fk::executeOperations<fkb200::TransformDPP>(stream, sender, receiver), i.e.
 *           through the Executor specialisation of fkb200_executor.h and libfkb200's kernels, or
 *   mode 1: only lowers it (no device is touched) and keeps the plan for inspection, so that a CPU
 *           test can compare it with the plan the Python harness builds for the same chain.
 * All image pointers are DEVICE pointers in mode 0; in mode 1 they are never dereferenced.
 */
#include <array>
#include <cstdint>
#include <cstring>
#include <string>

#include <fused_kernel/fused_kernel.h>
#include <fused_kernel/algorithms/algorithms.h>
#include <fused_kernel/algorithms/image_processing/image.h>
#include <fused_kernel/core/data/circular_tensor.h>

#include <fkb200_executor.h>

using namespace fk;

namespace {

thread_local fkb200::binding::LoweredPlan g_last;
thread_local std::string g_error;

constexpr auto LINEAR = InterpolationType::INTER_LINEAR;

RawPtr<ND::_2D, uchar3> raw_u8x3(const void* d, int w, int h, int pitch) {
    return RawPtr<ND::_2D, uchar3>{reinterpret_cast<uchar3*>(const_cast<void*>(d)), PtrDims<ND::_2D>((uint)w, (uint)h, (uint)pitch)};
}
template <typename T> RawPtr<ND::_3D, T> raw_tensor(void* d, int w, int h, int planes, int color_planes) {
    return RawPtr<ND::_3D, T>{reinterpret_cast<T*>(d), PtrDims<ND::_3D>((uint)w, (uint)h, (uint)planes, (uint)color_planes, (uint)(sizeof(T) * w))};
}
float3 f3(const float* p) { return float3{p[0], p[1], p[2]}; }

/* mode 0: execute through the binding; mode 1: lower only */
template <typename... IOps> int run(int mode, void* stream, const IOps&... iops) {
    try {
        if (mode == 1) {
            g_last = fkb200::binding::lower(iops...);
            (void)g_last.desc();
        } else {
            Stream_<ParArch::GPU_NVIDIA> s(static_cast<cudaStream_t>(stream));
            executeOperations<fkb200::TransformDPP>(s, iops...);
        }
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

template <size_t B, AspectRatio AR>
auto cropped_resized(const void* const* frames, int w, int h, int pitch, const int* rects, int dw, int dh, const float* bg) {
    std::array<RawPtr<ND::_2D, uchar3>, B> srcs;
    std::array<Rect, B> crops;
    for (size_t i = 0; i < B; ++i) {
        srcs[i] = raw_u8x3(frames[i], w, h, pitch);
        crops[i] = Rect(rects[4 * i + 0], rects[4 * i + 1], rects[4 * i + 2], rects[4 * i + 3]);
    }
    const auto cropped = PerThreadRead<ND::_2D, uchar3>::build(srcs).then(Crop<>::build(crops));
    if constexpr (AR == AspectRatio::IGNORE_AR) return cropped.then(Resize<LINEAR, AR>::build(Size(dw, dh)));
    else return cropped.then(Resize<LINEAR, AR>::build(Size(dw, dh), f3(bg)));
}

/* PerThreadRead -> BorderReader<border> -> Crop(rect beyond the image) -> Resize dw x dh -> PerThreadWrite<float3>.
   border: 1 CONSTANT(value) 2 REPLICATE 3 REFLECT 4 WRAP 5 REFLECT_101 */
template <BorderType BT>
int border_crop_resize(int mode, const void* src, int w, int h, int pitch, const uint8_t* value, const int* rect, int dw, int dh,
                              float* out, void* stream) {
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, pitch));
    using ReadIOp = std::decay_t<decltype(read)>;
    const auto bordered = [&] {
        if constexpr (BT == BorderType::CONSTANT) return BorderReader<BT, ReadIOp>::build(read, uchar3{value[0], value[1], value[2]});
        else return BorderReader<BT, ReadIOp>::build(read);
    }();
    const auto sender = bordered.then(Crop<>::build(Rect(rect[0], rect[1], rect[2], rect[3]))).then(Resize<LINEAR>::build(Size(dw, dh)));
    return run(mode, stream, sender, PerThreadWrite<ND::_2D, float3>::build(
        RawPtr<ND::_2D, float3>{reinterpret_cast<float3*>(out), PtrDims<ND::_2D>((uint)dw, (uint)dh, (uint)(dw * 12))}));
}

/* ReadYUV<PF> -> ConvertYUVToRGB<PF, Full, bt601, false, float3> -> Resize dw x dh -> Mul -> PerThreadWrite<float3>, one image of
   a layout beyond NV12 / NV21.  format as fkb_src_format: 5 P010, 6 P210, 7 Y210, 8 UYVY. */
template <PixelFormat PF>
int yuv_layout_chain(int mode, const void* frame, int w, int h, int pitch, int dw, int dh, const float* mul, float* out, void* stream) {
    using Img = Image<PF>;
    using Base = typename Img::BaseType;
    Ptr<ND::_2D, Base> view(reinterpret_cast<Base*>(const_cast<void*>(frame)), PtrDims<ND::_2D>((uint)w, (uint)h, (uint)pitch), MemType::Device, 0);
    const Img img(view, (uint)w, (uint)h);
    const auto sender = ReadYUV<PF>::build(img)
                            .then(ConvertYUVToRGB<PF, ColorRange::Full, ColorPrimitives::bt601, false, float3>::build())
                            .then(Resize<LINEAR>::build(Size(dw, dh)))
                            .then(Mul<float3>::build(f3(mul)));
    return run(mode, stream, sender, PerThreadWrite<ND::_2D, float3>::build(
        RawPtr<ND::_2D, float3>{reinterpret_cast<float3*>(out), PtrDims<ND::_2D>((uint)dw, (uint)dh, (uint)(dw * 12))}));
}

}  // namespace

extern "C" {

const char* fklbind_last_error(void) { return g_error.c_str(); }

/* the README example (README.md; tests/examples/readme_test_code.h:25-71): one frame, five crops, 60x60 */
int fklbind_readme5(int mode, const void* frame, int w, int h, int pitch, const int* rects, const float* bg, const float* mul,
                    const float* sub, const float* div, float* out, void* stream) {
    const void* frames[5] = {frame, frame, frame, frame, frame};
    const auto sender = cropped_resized<5, AspectRatio::PRESERVE_AR>(frames, w, h, pitch, rects, 60, 60, bg)
                            .then(Mul<float3>::build(f3(mul)))
                            .then(Sub<float3>::build(f3(sub)))
                            .then(Div<float3>::build(f3(div)))
                            .then(ColorConversion<ColorConversionCodes::COLOR_RGB2BGR, float3, float3>::build());
    const auto receiver = TensorWrite<float3>::build(raw_tensor<float3>(out, 60, 60, 5, 1));
    return run(mode, stream, sender, receiver);
}

/* 16 crops of several frames -> PRESERVE_AR dw x dh -> Div, Sub, Div -> TensorSplit (16 x 3 x dh x dw) */
int fklbind_norm_planar16(int mode, const void* const* frames, int w, int h, int pitch, const int* rects, int dw, int dh,
                          const float* bg, const float* d0, const float* mean, const float* stdv, float* out, void* stream) {
    const auto sender = cropped_resized<16, AspectRatio::PRESERVE_AR>(frames, w, h, pitch, rects, dw, dh, bg)
                            .then(Div<float3>::build(f3(d0)))
                            .then(Sub<float3>::build(f3(mean)))
                            .then(Div<float3>::build(f3(stdv)));
    const auto receiver = TensorSplit<float3>::build(raw_tensor<float>(out, dw, dh, 16, 3));
    return run(mode, stream, sender, receiver);
}

/* two NV12 frames -> ConvertYUVToRGB<Full, bt709> -> Resize dw x dh -> Div -> TensorWrite<float3> */
int fklbind_nv12_2(int mode, const void* const* frames, int w, int h, int pitch, int dw, int dh, const float* div, float* out,
                   void* stream) {
    using Img = Image<PixelFormat::NV12>;
    auto make = [&](size_t i) {
        Ptr<ND::_2D, uchar> view(reinterpret_cast<uchar*>(const_cast<void*>(frames[i])), PtrDims<ND::_2D>((uint)w, (uint)h, (uint)pitch),
                                 MemType::Device, 0);
        return Img(view, (uint)w, (uint)h);
    };
    std::array<Img, 2> imgs{make(0), make(1)};
    const auto sender = ReadYUV<PixelFormat::NV12>::build(imgs)
                            .then(ConvertYUVToRGB<PixelFormat::NV12, ColorRange::Full, ColorPrimitives::bt709, false, float3>::build())
                            .then(Resize<LINEAR>::build(Size(dw, dh)))
                            .then(Div<float3>::build(f3(div)));
    const auto receiver = TensorWrite<float3>::build(raw_tensor<float3>(out, dw, dh, 2, 1));
    return run(mode, stream, sender, receiver);
}

/* one image, the operations handed over one by one (the parameter-pack form of fused_kernel.h:22-25) */
int fklbind_cast_mul_sub_div(int mode, const void* src, int w, int h, int spitch, const float* mul, const float* sub, const float* div,
                             float* dst, int dpitch, void* stream) {
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, spitch));
    const auto write = PerThreadWrite<ND::_2D, float3>::build(
        RawPtr<ND::_2D, float3>{reinterpret_cast<float3*>(dst), PtrDims<ND::_2D>((uint)w, (uint)h, (uint)dpitch)});
    return run(mode, stream, read, Cast<uchar3, float3>::build(), Mul<float3>::build(f3(mul)), Sub<float3>::build(f3(sub)),
               Div<float3>::build(f3(div)), write);
}

/* the shape of the reference's run-time test (tests/operation/test_instantiable_operations.h:236-264):
   Cast -> Resize -> Add -> Cast<float3,uint3> -> PerThreadWrite<uint3> */
int fklbind_cast_resize_add_cast_uint3(int mode, const void* src, int w, int h, int spitch, int dw, int dh, const float* add,
                                       uint32_t* dst, int dpitch, void* stream) {
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, spitch))
                            .then(Cast<uchar3, float3>::build())
                            .then(Resize<LINEAR>::build(Size(dw, dh)))
                            .then(Add<float3>::build(f3(add)))
                            .then(Cast<float3, uint3>::build());
    const auto write = PerThreadWrite<ND::_2D, uint3>::build(
        RawPtr<ND::_2D, uint3>{reinterpret_cast<uint3*>(dst), PtrDims<ND::_2D>((uint)dw, (uint)dh, (uint)dpitch)});
    return run(mode, stream, sender, write);
}

/* RGB2BGR(uchar3) -> Cast -> Mul -> SaturateCast<float3,uchar3> -> PerThreadWrite<uchar3> */
int fklbind_bgr_cast_mul_saturate(int mode, const void* src, int w, int h, int spitch, const float* mul, uint8_t* dst, int dpitch,
                                  void* stream) {
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, spitch))
                            .then(ColorConversion<ColorConversionCodes::COLOR_RGB2BGR, uchar3, uchar3>::build())
                            .then(Cast<uchar3, float3>::build())
                            .then(Mul<float3>::build(f3(mul)))
                            .then(SaturateCast<float3, uchar3>::build());
    return run(mode, stream, sender, PerThreadWrite<ND::_2D, uchar3>::build(raw_u8x3(dst, w, h, dpitch)));
}

/* two NV21 frames -> ConvertYUVToRGB<Full, bt601> -> Resize dw x dh -> Div -> TensorWrite<float3> */
int fklbind_nv21_bt601_2(int mode, const void* const* frames, int w, int h, int pitch, int dw, int dh, const float* div, float* out,
                         void* stream) {
    using Img = Image<PixelFormat::NV21>;
    auto make = [&](size_t i) {
        Ptr<ND::_2D, uchar> view(reinterpret_cast<uchar*>(const_cast<void*>(frames[i])), PtrDims<ND::_2D>((uint)w, (uint)h, (uint)pitch),
                                 MemType::Device, 0);
        return Img(view, (uint)w, (uint)h);
    };
    std::array<Img, 2> imgs{make(0), make(1)};
    const auto sender = ReadYUV<PixelFormat::NV21>::build(imgs)
                            .then(ConvertYUVToRGB<PixelFormat::NV21, ColorRange::Full, ColorPrimitives::bt601, false, float3>::build())
                            .then(Resize<LINEAR>::build(Size(dw, dh)))
                            .then(Div<float3>::build(f3(div)));
    return run(mode, stream, sender, TensorWrite<float3>::build(raw_tensor<float3>(out, dw, dh, 2, 1)));
}

/* four crops -> PRESERVE_AR_LEFT dw x dh -> Div, Sub, Div -> TensorTSplit (3 x 4 x dh x dw, channel-major over the batch) */
int fklbind_left_tsplit4(int mode, const void* const* frames, int w, int h, int pitch, const int* rects, int dw, int dh, const float* bg,
                         const float* d0, const float* mean, const float* stdv, float* out, void* stream) {
    const auto sender = cropped_resized<4, AspectRatio::PRESERVE_AR_LEFT>(frames, w, h, pitch, rects, dw, dh, bg)
                            .then(Div<float3>::build(f3(d0)))
                            .then(Sub<float3>::build(f3(mean)))
                            .then(Div<float3>::build(f3(stdv)));
    PtrDims<ND::T3D> dims((uint)dw, (uint)dh, 4u, 3u);
    dims.pitch = (uint)(dw * sizeof(float));
    dims.plane_pitch = dims.pitch * (uint)dh;
    dims.color_planes_pitch = dims.plane_pitch * 4u;
    const auto receiver = TensorTSplit<float3>::build(RawPtr<ND::T3D, float>{out, dims});
    return run(mode, stream, sender, receiver);
}

/* a partly filled batch of four images (BatchRead<4, CONDITIONAL_WITH_DEFAULT>): Cast -> Mul -> TensorWrite<float3> */
int fklbind_batch4_default_cast_mul(int mode, const void* const* srcs, int w, int h, int spitch, int used, const uint8_t* default_value,
                                    const float* mul, float* dst, void* stream) {
    std::array<RawPtr<ND::_2D, uchar3>, 4> a;
    for (size_t i = 0; i < 4; ++i) a[i] = raw_u8x3(srcs[i], w, h, spitch);
    const uchar3 dv{default_value[0], default_value[1], default_value[2]};
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(used, dv, a);
    return run(mode, stream, read, Cast<uchar3, float3>::build(), Mul<float3>::build(f3(mul)),
               TensorWrite<float3>::build(raw_tensor<float3>(dst, w, h, 4, 1)));
}

/* border: 1 CONSTANT(value) 2 REPLICATE 3 REFLECT 4 WRAP 5 REFLECT_101 */
int fklbind_border_crop_resize(int mode, const void* src, int w, int h, int pitch, int border, const uint8_t* value, const int* rect, int dw,
                               int dh, float* out, void* stream) {
    switch (border) {
        case 1: return border_crop_resize<BorderType::CONSTANT>(mode, src, w, h, pitch, value, rect, dw, dh, out, stream);
        case 2: return border_crop_resize<BorderType::REPLICATE>(mode, src, w, h, pitch, value, rect, dw, dh, out, stream);
        case 3: return border_crop_resize<BorderType::REFLECT>(mode, src, w, h, pitch, value, rect, dw, dh, out, stream);
        case 4: return border_crop_resize<BorderType::WRAP>(mode, src, w, h, pitch, value, rect, dw, dh, out, stream);
        case 5: return border_crop_resize<BorderType::REFLECT_101>(mode, src, w, h, pitch, value, rect, dw, dh, out, stream);
        default: g_error = "unknown border"; return -1;
    }
}

/* PerThreadRead -> Warping<Affine | Perspective>(matrix, dw x dh) -> Mul -> PerThreadWrite<float3> */
int fklbind_warp(int mode, const void* src, int w, int h, int pitch, int perspective, const float* matrix, int dw, int dh, const float* mul,
                 float* out, void* stream) {
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, pitch));
    const auto write = PerThreadWrite<ND::_2D, float3>::build(
        RawPtr<ND::_2D, float3>{reinterpret_cast<float3*>(out), PtrDims<ND::_2D>((uint)dw, (uint)dh, (uint)(dw * 12))});
    if (perspective) {
        WarpingParameters<WarpType::Perspective> p{};
        for (int r = 0; r < 3; ++r) for (int c = 0; c < 3; ++c) p.transformMatrix.data[r][c] = matrix[3 * r + c];
        p.dstSize = Size(dw, dh);
        return run(mode, stream, read.then(Warping<WarpType::Perspective>::build(p)).then(Mul<float3>::build(f3(mul))), write);
    }
    WarpingParameters<WarpType::Affine> p{};
    for (int r = 0; r < 2; ++r) for (int c = 0; c < 3; ++c) p.transformMatrix.data[r][c] = matrix[3 * r + c];
    p.dstSize = Size(dw, dh);
    return run(mode, stream, read.then(Warping<WarpType::Affine>::build(p)).then(Mul<float3>::build(f3(mul))), write);
}

/* PerThreadRead -> Deinterlace -> Mul -> PerThreadWrite<float3>.  kind: 1 BLEND, 2 INTER_LINEAR keeping even lines, 3 odd */
int fklbind_deinterlace(int mode, const void* src, int w, int h, int pitch, int kind, const float* mul, float* out, void* stream) {
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, pitch));
    const auto write = PerThreadWrite<ND::_2D, float3>::build(
        RawPtr<ND::_2D, float3>{reinterpret_cast<float3*>(out), PtrDims<ND::_2D>((uint)w, (uint)h, (uint)(w * 12))});
    if (kind == 1) return run(mode, stream, Deinterlace<DeinterlaceType::BLEND>::build(read).then(Mul<float3>::build(f3(mul))), write);
    const auto lin = kind == 2 ? DeinterlaceLinear::USE_EVEN : DeinterlaceLinear::USE_ODD;
    return run(mode, stream, Deinterlace<DeinterlaceType::INTER_LINEAR>::build(lin, read).then(Mul<float3>::build(f3(mul))), write);
}

/* format as fkb_src_format: 5 P010, 6 P210, 7 Y210, 8 UYVY */
int fklbind_yuv_layout(int mode, int format, const void* frame, int w, int h, int pitch, int dw, int dh, const float* mul, float* out,
                       void* stream) {
    switch (format) {
        case 5: return yuv_layout_chain<PixelFormat::P010>(mode, frame, w, h, pitch, dw, dh, mul, out, stream);
        case 6: return yuv_layout_chain<PixelFormat::P210>(mode, frame, w, h, pitch, dw, dh, mul, out, stream);
        case 7: return yuv_layout_chain<PixelFormat::Y210>(mode, frame, w, h, pitch, dw, dh, mul, out, stream);
        case 8: return yuv_layout_chain<PixelFormat::UYVY>(mode, frame, w, h, pitch, dw, dh, mul, out, stream);
        default: g_error = "unknown layout"; return -1;
    }
}

/* ---- the reference's own CircularTensor class (core/data/circular_tensor.h), its update() running through the binding ---- */
using RefCircularNewest = CircularTensor<float, 3, 6, CircularTensorOrder::NewestFirst, ColorPlanes::Standard>;
using RefCircularOldest = CircularTensor<float, 3, 6, CircularTensorOrder::OldestFirst, ColorPlanes::Standard>;
struct CircularHandle { int order; RefCircularNewest newest; RefCircularOldest oldest; };

/* a 6-plane tensor of 3 x h x w floats in device memory that the reference's Tensor class allocates */
void* fklbind_circular_create(int order, int w, int h) {
    try {
        auto* c = new CircularHandle{order, {}, {}};
        if (order == 0) c->newest.Alloc((uint)w, (uint)h, MemType::Device); else c->oldest.Alloc((uint)w, (uint)h, MemType::Device);
        return c;
    } catch (const std::exception& e) { g_error = e.what(); return nullptr; }
}
void* fklbind_circular_data(void* handle) {
    auto* c = static_cast<CircularHandle*>(handle);
    return c->order == 0 ? (void*)c->newest.ptr().data : (void*)c->oldest.ptr().data;
}
/* CircularTensor::update(stream, crop -> PRESERVE_AR resize -> Div, Sub, Div, TensorSplit(this tensor)) */
int fklbind_circular_update(void* handle, const void* frame, int w, int h, int pitch, const int* rect, const float* bg, const float* d0,
                            const float* mean, const float* stdv, void* stream) {
    auto* c = static_cast<CircularHandle*>(handle);
    try {
        Stream_<ParArch::GPU_NVIDIA> s(static_cast<cudaStream_t>(stream));
        auto run = [&](auto& tensor) {
            const auto dims = tensor.ptr().dims;
            const auto sender = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(frame, w, h, pitch))
                                    .then(Crop<>::build(Rect(rect[0], rect[1], rect[2], rect[3])))
                                    .then(Resize<LINEAR, AspectRatio::PRESERVE_AR>::build(Size((int)dims.width, (int)dims.height), f3(bg)))
                                    .then(Div<float3>::build(f3(d0)))
                                    .then(Sub<float3>::build(f3(mean)))
                                    .then(Div<float3>::build(f3(stdv)));
            tensor.update(s, sender, TensorSplit<float3>::build(tensor.ptr()));
        };
        if (c->order == 0) run(c->newest); else run(c->oldest);
        return 0;
    } catch (const std::exception& e) { g_error = e.what(); return -1; }
}
void fklbind_circular_destroy(void* handle) { delete static_cast<CircularHandle*>(handle); }

/* The two sequences update() builds (circular_tensor.h:121-134) over tensors of the caller, lowered only: for the
   comparison of the plan with fkb_circular_tensor_plan_update on a machine without a GPU. */
int fklbind_circular_describe6(int order, const void* frame, int w, int h, int pitch, const int* rect, int dw, int dh, const float* bg,
                               const float* d0, const float* mean, const float* stdv, float* visible, float* hidden, int first) {
    try {
        const auto v = raw_tensor<float>(visible, dw, dh, 6, 3), t = raw_tensor<float>(hidden, dw, dh, 6, 3);
        const auto sender = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(frame, w, h, pitch))
                                .then(Crop<>::build(Rect(rect[0], rect[1], rect[2], rect[3])))
                                .then(Resize<LINEAR, AspectRatio::PRESERVE_AR>::build(Size(dw, dh), f3(bg)))
                                .then(Div<float3>::build(f3(d0)))
                                .then(Sub<float3>::build(f3(mean)))
                                .then(Div<float3>::build(f3(stdv)));
        const auto write = TensorSplit<float3>::build(v);
        MidWrite<CircularTensorWrite<CircularDirection::Ascendent, TensorSplit<float3>, 6>> toHidden;
        toHidden.params.first = first;
        toHidden.params.opData.params = t;
        const auto updateOps = buildOperationSequence(sender, toHidden, write);
        if (order == 0) {
            Read<CircularTensorRead<CircularDirection::Descendent, TensorPack<float3>, 6>> fromHidden;
            fromHidden.params.first = first; fromHidden.params.opData.params = t;
            g_last = fkb200::binding::lower_divergent<SequenceSelectorType<CircularTensorOrder::NewestFirst, 6>>(updateOps, buildOperationSequence(fromHidden, write));
        } else {
            Read<CircularTensorRead<CircularDirection::Ascendent, TensorPack<float3>, 6>> fromHidden;
            fromHidden.params.first = first; fromHidden.params.opData.params = t;
            g_last = fkb200::binding::lower_divergent<SequenceSelectorType<CircularTensorOrder::OldestFirst, 6>>(updateOps, buildOperationSequence(fromHidden, write));
        }
        (void)g_last.desc();
        return 0;
    } catch (const std::exception& e) { g_error = e.what(); return -1; }
}

/* ---- inspection of the plan of the last mode-1 call on this thread ---- */
int fklbind_last_counts(int* n_planes, int* n_sequences) {
    *n_planes = (int)g_last.planes.size();
    *n_sequences = (int)g_last.sequences.size();
    return 0;
}
int fklbind_last_plane(int i, fkb_plane* out) {
    if (i < 0 || i >= (int)g_last.planes.size()) return -1;
    *out = g_last.planes[i];
    return 0;
}
/* ops_out receives up to `capacity` operations; returns the sequence's operation count */
int fklbind_last_sequence(int s, fkb_sequence* out, fkb_op* ops_out, int capacity) {
    if (s < 0 || s >= (int)g_last.sequences.size()) return -1;
    *out = g_last.sequences[s];
    out->ops = nullptr;
    const int n = (int)g_last.sequence_ops[s].size();
    for (int k = 0; k < n && k < capacity; ++k) ops_out[k] = g_last.sequence_ops[s][k];
    return n;
}
/* what the reference's own Resize::build stored in the operation (resize.h:105-166) for plane i */
int fklbind_last_reference_resize(int i, fkb_resize_params* out) {
    if (i < 0 || i >= (int)g_last.states.size() || !g_last.states[i].has_reference_resize) return -1;
    *out = g_last.states[i].reference_resize;
    return 0;
}

}  // extern "C"
