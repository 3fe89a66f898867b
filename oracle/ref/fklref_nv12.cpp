/* extern "C" entry points around the UNMODIFIED reference headers (CPU backend; CUDA backend with -DFKLREF_GPU).
 *
 * TEST INFRASTRUCTURE ONLY.  Compiled by oracle/Makefile against the reference's include
 * tree where it lies (never copied); the shared objects go to oracle/_ref/.  Only tests,
 * the smoke check and the CPU-baseline legs of the benchmark load them; the product path
 * never does.
 *
 * Every entry point builds the sender chain a user of the reference would write
 * (Op::build(...).then(...)), closes it with a receiver and runs it with
 * fk::executeOperations<TransformDPP<ParArch::CPU>> (fused_kernel.h:22-25,
 * core/execution_model/executors.h:147-173, data_parallel_patterns.h:272-299).
 */
#include "fklref_common.h"

namespace {

/* ---- NV12 -> RGB -> resize -> Div -> TensorWrite, one chunk ------------------------ */

template <size_t B, PixelFormat PF = PixelFormat::NV12, ColorPrimitives CP = ColorPrimitives::bt709>
void nv12_chunk(const uint8_t* const* frames, int w, int h, int pitch, int dw, int dh, const float* div,
                float* out) {
    RefStream stream = make_stream();
    using Img = Image<PF>;
    /* Wrap each frame as a view whose data height equals the image height so that the chroma
       plane is addressed at data + pitch*h (color_conversion.h:336-341, image.h:35-38). */
    auto make = [&](size_t i) {
        Ptr<ND::_2D, uchar> view(const_cast<uint8_t*>(frames[i]), PtrDims<ND::_2D>((uint)w, (uint)h, (uint)pitch),
                                 REF_MEM, 0);
        return Img(view, (uint)w, (uint)h);
    };
    std::array<Img, B> imgs = [&]<size_t... I>(std::index_sequence<I...>) {
        return std::array<Img, B>{make(I)...};
    }(std::make_index_sequence<B>{});
    const auto sender =
        ReadYUV<PF>::build(imgs)
            .then(ConvertYUVToRGB<PF, ColorRange::Full, CP, false, float3>::build())
            .then(Resize<LINEAR>::build(Size(dw, dh)))
            .then(Div<float3>::build(f3(div)));
    const auto receiver = TensorWrite<float3>::build(raw_tensor<float3>(out, dw, dh, (int)B, 1));
    executeOperations<RefDPP>(stream, sender, receiver);
    finish(stream);
}

}  // namespace

extern "C" {

/* ReadYUV<NV12>[B] -> ConvertYUVToRGB<NV12,Full,bt709,false,float3> -> Resize<INTER_LINEAR>(dw,dh) -> Div
   -> TensorWrite<float3> (dw x dh x B).  Each frame: h rows of luma then h/2 rows of interleaved chroma, one pitch. */
void FKLREF_FN(nv12_resize)(const uint8_t* const* frames, int w, int h, int pitch, int batch, int dw, int dh,
                        const float* div, float* out) {
    const size_t plane_floats = (size_t)dw * dh * 3;
    int i = 0;
#ifdef FKLREF_GPU
    for (; i + 32 <= batch; i += 32) nv12_chunk<32>(frames + i, w, h, pitch, dw, dh, div, out + plane_floats * i);
#endif
    for (; i + 4 <= batch; i += 4) nv12_chunk<4>(frames + i, w, h, pitch, dw, dh, div, out + plane_floats * i);
    for (; i + 2 <= batch; i += 2) nv12_chunk<2>(frames + i, w, h, pitch, dw, dh, div, out + plane_floats * i);
    if (i < batch) {
        if (batch >= 2) {
            nv12_chunk<2>(frames + batch - 2, w, h, pitch, dw, dh, div, out + plane_floats * (batch - 2));
        } else {
#ifndef FKLREF_GPU
            const uint8_t* two[2] = {frames[0], frames[0]};
            float* scratch = new float[plane_floats * 2];
            nv12_chunk<2>(two, w, h, pitch, dw, dh, div, scratch);
            std::memcpy(out, scratch, plane_floats * sizeof(float));
            delete[] scratch;
#endif
        }
    }
}

#ifndef FKLREF_GPU
/* The same chain for other layouts and matrices, pairs of frames: layout 0 = NV12, 1 = NV21 (color_conversion.h:347-359);
   primitives 0 = bt709, 1 = bt601 (:137-140, luma offset :266-269), 2 = bt2020 (:165-168).  Host build only; batch even. */
int FKLREF_FN(nv_resize_ex)(const uint8_t* const* frames, int w, int h, int pitch, int batch, int dw, int dh, int layout,
                            int primitives, const float* div, float* out) {
    const size_t plane_floats = (size_t)dw * dh * 3;
    if (batch % 2) return -1;
    for (int i = 0; i < batch; i += 2) {
        float* o = out + plane_floats * i;
        if (layout == 0 && primitives == 1) nv12_chunk<2, PixelFormat::NV12, ColorPrimitives::bt601>(frames + i, w, h, pitch, dw, dh, div, o);
        else if (layout == 0 && primitives == 2) nv12_chunk<2, PixelFormat::NV12, ColorPrimitives::bt2020>(frames + i, w, h, pitch, dw, dh, div, o);
        else if (layout == 1 && primitives == 0) nv12_chunk<2, PixelFormat::NV21, ColorPrimitives::bt709>(frames + i, w, h, pitch, dw, dh, div, o);
        else if (layout == 1 && primitives == 1) nv12_chunk<2, PixelFormat::NV21, ColorPrimitives::bt601>(frames + i, w, h, pitch, dw, dh, div, o);
        else return -1;
    }
    return 0;
}
#endif

}  // extern "C"
