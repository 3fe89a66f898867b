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

}  // namespace

extern "C" {

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
