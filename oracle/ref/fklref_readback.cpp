/* extern "C" entry points around the UNMODIFIED reference headers (CPU backend): the other read-back operations.
 *
 * TEST INFRASTRUCTURE ONLY (see fklref_common.h).  BorderReader (image_processing/border_reader.h:136-279), Warping
 * (warping.h:43-141) and Deinterlace (deinterlace.h:41-183), each in a chain a user of the reference would write and
 * run with fk::executeOperations<TransformDPP<ParArch::CPU>>.  Host build only.
 */
#include "fklref_common.h"

namespace {

template <BorderType BT, bool RESIZE>
void border_crop(const uint8_t* src, int w, int h, int pitch, const uint8_t* value, const int* rect, int dw, int dh, void* out) {
    RefStream stream = make_stream();
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, pitch));
    /* the complete form: the incomplete builder BorderReader<BT>::build(read) is ambiguous for every type but CONSTANT
       (border_reader.h:56 matches two specialisations) */
    using ReadIOp = std::decay_t<decltype(read)>;
    const auto bordered = [&] {
        if constexpr (BT == BorderType::CONSTANT) return BorderReader<BT, ReadIOp>::build(read, uchar3{value[0], value[1], value[2]});
        else return BorderReader<BT, ReadIOp>::build(read);
    }();
    const auto cropped = bordered.then(Crop<>::build(Rect(rect[0], rect[1], rect[2], rect[3])));
    if constexpr (RESIZE) {
        const auto sender = cropped.then(Resize<LINEAR>::build(Size(dw, dh)));
        executeOperations<RefDPP>(stream, sender, PerThreadWrite<ND::_2D, float3>::build(raw_f32x3((const float*)out, dw, dh, dw * 12)));
    } else {
        executeOperations<RefDPP>(stream, cropped, PerThreadWrite<ND::_2D, uchar3>::build(raw_u8x3((const uint8_t*)out, rect[2], rect[3], rect[2] * 3)));
    }
    finish(stream);
}

template <bool RESIZE>
int border_dispatch(int border, const uint8_t* src, int w, int h, int pitch, const uint8_t* value, const int* rect, int dw, int dh, void* out) {
    switch (border) {
        case 1: border_crop<BorderType::CONSTANT, RESIZE>(src, w, h, pitch, value, rect, dw, dh, out); return 0;
        case 2: border_crop<BorderType::REPLICATE, RESIZE>(src, w, h, pitch, value, rect, dw, dh, out); return 0;
        case 3: border_crop<BorderType::REFLECT, RESIZE>(src, w, h, pitch, value, rect, dw, dh, out); return 0;
        case 4: border_crop<BorderType::WRAP, RESIZE>(src, w, h, pitch, value, rect, dw, dh, out); return 0;
        case 5: border_crop<BorderType::REFLECT_101, RESIZE>(src, w, h, pitch, value, rect, dw, dh, out); return 0;
        default: return -1;
    }
}

/* ReadYUV<PF> -> ConvertYUVToRGB<PF, Full, CP, false, float3> [-> Resize(dw, dh)] -> Mul -> PerThreadWrite<float3>, one image.
   The view's data height is the image height, so that a chroma plane is addressed at data + pitch * h
   (color_conversion.h:336-341); its element type is the format's base type (uchar, or ushort for the 10-bit formats). */
template <PixelFormat PF, ColorPrimitives CP>
void yuv_chain(const void* frame, int w, int h, int pitch, int dw, int dh, const float* mul, float* out) {
    RefStream stream = make_stream();
    using Img = Image<PF>;
    using Base = typename Img::BaseType;
    Ptr<ND::_2D, Base> view(reinterpret_cast<Base*>(const_cast<void*>(frame)), PtrDims<ND::_2D>((uint)w, (uint)h, (uint)pitch), REF_MEM, 0);
    const Img img(view, (uint)w, (uint)h);
    const auto converted = ReadYUV<PF>::build(img).then(ConvertYUVToRGB<PF, ColorRange::Full, CP, false, float3>::build());
    if (dw == w && dh == h) {
        executeOperations<RefDPP>(stream, converted.then(Mul<float3>::build(f3(mul))), PerThreadWrite<ND::_2D, float3>::build(raw_f32x3(out, w, h, w * 12)));
    } else {
        executeOperations<RefDPP>(stream, converted.then(Resize<LINEAR>::build(Size(dw, dh))).then(Mul<float3>::build(f3(mul))),
                                  PerThreadWrite<ND::_2D, float3>::build(raw_f32x3(out, dw, dh, dw * 12)));
    }
    finish(stream);
}
template <PixelFormat PF>
int yuv_chain_primitives(int primitives, const void* frame, int w, int h, int pitch, int dw, int dh, const float* mul, float* out) {
    switch (primitives) {
        case 0: yuv_chain<PF, ColorPrimitives::bt709>(frame, w, h, pitch, dw, dh, mul, out); return 0;
        case 1: yuv_chain<PF, ColorPrimitives::bt601>(frame, w, h, pitch, dw, dh, mul, out); return 0;
        case 2: yuv_chain<PF, ColorPrimitives::bt2020>(frame, w, h, pitch, dw, dh, mul, out); return 0;
        default: return -1;
    }
}

}  // namespace

extern "C" {

/* One image of a YUV layout beyond NV12 / NV21, converted to RGB, optionally resized, multiplied.  format: 5 P010 (4:2:0,
   10 bits in the top of 16, luma plane then interleaved chroma), 6 P210 (the same, 4:2:2), 7 Y210 (packed 4:2:2, 16-bit
   Y0 U Y1 V), 8 UYVY (packed 4:2:2, 8-bit U Y0 V Y1); primitives 0 bt709, 1 bt601, 2 bt2020.  No resize when dw x dh = w x h. */
int FKLREF_FN(yuv_format_chain)(int format, int primitives, const void* frame, int w, int h, int pitch, int dw, int dh, const float* mul,
                                float* out) {
    switch (format) {
        case 5: return yuv_chain_primitives<PixelFormat::P010>(primitives, frame, w, h, pitch, dw, dh, mul, out);
        case 6: return yuv_chain_primitives<PixelFormat::P210>(primitives, frame, w, h, pitch, dw, dh, mul, out);
        case 7: return yuv_chain_primitives<PixelFormat::Y210>(primitives, frame, w, h, pitch, dw, dh, mul, out);
        case 8: return yuv_chain_primitives<PixelFormat::UYVY>(primitives, frame, w, h, pitch, dw, dh, mul, out);
        default: return -1;
    }
}

/* PerThreadRead<uchar3> -> BorderReader<border> -> Crop(rect, may reach beyond the image) -> PerThreadWrite<uchar3>.
   border: 1 CONSTANT(value) 2 REPLICATE 3 REFLECT 4 WRAP 5 REFLECT_101. */
int FKLREF_FN(border_crop)(const uint8_t* src, int w, int h, int pitch, int border, const uint8_t* value, const int* rect, uint8_t* out) {
    return border_dispatch<false>(border, src, w, h, pitch, value, rect, 0, 0, out);
}

/* The same followed by Resize<INTER_LINEAR>(dw, dh) -> PerThreadWrite<float3>. */
int FKLREF_FN(border_crop_resize)(const uint8_t* src, int w, int h, int pitch, int border, const uint8_t* value, const int* rect, int dw,
                                  int dh, float* out) {
    return border_dispatch<true>(border, src, w, h, pitch, value, rect, dw, dh, out);
}

/* PerThreadRead<uchar3> -> Warping<Affine | Perspective>(matrix, dw x dh) -> Mul -> PerThreadWrite<float3>.
   matrix: rows of three floats; an affine warp reads the first two rows. */
int FKLREF_FN(warp)(const uint8_t* src, int w, int h, int pitch, int perspective, const float* matrix, int dw, int dh, const float* mul,
                    float* out) {
    RefStream stream = make_stream();
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, pitch));
    const auto write = PerThreadWrite<ND::_2D, float3>::build(raw_f32x3(out, dw, dh, dw * 12));
    if (perspective) {
        WarpingParameters<WarpType::Perspective> p{};
        for (int r = 0; r < 3; ++r) for (int c = 0; c < 3; ++c) p.transformMatrix.data[r][c] = matrix[3 * r + c];
        p.dstSize = Size(dw, dh);
        executeOperations<RefDPP>(stream, read.then(Warping<WarpType::Perspective>::build(p)).then(Mul<float3>::build(f3(mul))), write);
    } else {
        WarpingParameters<WarpType::Affine> p{};
        for (int r = 0; r < 2; ++r) for (int c = 0; c < 3; ++c) p.transformMatrix.data[r][c] = matrix[3 * r + c];
        p.dstSize = Size(dw, dh);
        executeOperations<RefDPP>(stream, read.then(Warping<WarpType::Affine>::build(p)).then(Mul<float3>::build(f3(mul))), write);
    }
    finish(stream);
    return 0;
}

/* PerThreadRead<uchar3> -> Deinterlace -> Mul -> PerThreadWrite<float3>.  kind: 1 BLEND, 2 INTER_LINEAR keeping the even
   lines, 3 INTER_LINEAR keeping the odd lines. */
int FKLREF_FN(deinterlace)(const uint8_t* src, int w, int h, int pitch, int kind, const float* mul, float* out) {
    RefStream stream = make_stream();
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, pitch));
    const auto write = PerThreadWrite<ND::_2D, float3>::build(raw_f32x3(out, w, h, w * 12));
    if (kind == 1) {
        executeOperations<RefDPP>(stream, Deinterlace<DeinterlaceType::BLEND>::build(read).then(Mul<float3>::build(f3(mul))), write);
    } else if (kind == 2 || kind == 3) {
        const auto lin = kind == 2 ? DeinterlaceLinear::USE_EVEN : DeinterlaceLinear::USE_ODD;
        executeOperations<RefDPP>(stream, Deinterlace<DeinterlaceType::INTER_LINEAR>::build(lin, read).then(Mul<float3>::build(f3(mul))), write);
    } else {
        return -1;
    }
    finish(stream);
    return 0;
}

}  // extern "C"
