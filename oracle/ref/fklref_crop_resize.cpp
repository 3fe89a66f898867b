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

/* ---- crop -> resize -> chain, one chunk of B planes ------------------------------- */

enum class Tail { README_PACKED, NORM_PLANAR };

template <size_t B, AspectRatio AR, Tail TAIL>
void crop_resize_chunk(const uint8_t* const* frames, int w, int h, int pitch, const int* rects,
                       int dw, int dh, const float* bg, const float* p0, const float* p1,
                       const float* p2, float* out) {
    RefStream stream = make_stream();
    std::array<RawPtr<ND::_2D, uchar3>, B> srcs;
    std::array<Rect, B> crops;
    for (size_t i = 0; i < B; ++i) {
        srcs[i] = raw_u8x3(frames[i], w, h, pitch);
        crops[i] = Rect(rects[4 * i + 0], rects[4 * i + 1], rects[4 * i + 2], rects[4 * i + 3]);
    }
    const Size dst(dw, dh);
    const auto cropped = PerThreadRead<ND::_2D, uchar3>::build(srcs).then(Crop<>::build(crops));
    const auto resized = [&] {
        if constexpr (AR == AspectRatio::IGNORE_AR) {
            return cropped.then(Resize<LINEAR, AR>::build(dst));
        } else {
            return cropped.then(Resize<LINEAR, AR>::build(dst, f3(bg)));
        }
    }();
    if constexpr (TAIL == Tail::README_PACKED) {
        const auto sender = resized.then(Mul<float3>::build(f3(p0)))
                                .then(Sub<float3>::build(f3(p1)))
                                .then(Div<float3>::build(f3(p2)))
                                .then(ColorConversion<ColorConversionCodes::COLOR_RGB2BGR, float3, float3>::build());
        const auto receiver = TensorWrite<float3>::build(raw_tensor<float3>(out, dw, dh, (int)B, 1));
        executeOperations<RefDPP>(stream, sender, receiver);
    } else {
        const auto sender = resized.then(Div<float3>::build(f3(p0)))
                                .then(Sub<float3>::build(f3(p1)))
                                .then(Div<float3>::build(f3(p2)));
        const auto receiver = TensorSplit<float3>::build(raw_tensor<float>(out, dw, dh, (int)B, 3));
        executeOperations<RefDPP>(stream, sender, receiver);
    }
    finish(stream);
}

template <AspectRatio AR, Tail TAIL>
void crop_resize_all(const uint8_t* const* frames, int w, int h, int pitch, const int* rects, int batch,
                     int dw, int dh, const float* bg, const float* p0, const float* p1, const float* p2,
                     float* out) {
    const size_t plane_floats = (size_t)dw * dh * 3;
    int i = 0;
    if (batch == 5) { /* the README example's own batch size (README.md; tests/examples/readme_test_code.h): one launch */
        crop_resize_chunk<5, AR, TAIL>(frames, w, h, pitch, rects, dw, dh, bg, p0, p1, p2, out);
        return;
    }
#if FKLREF_BIG_CHUNK > 16
    for (; i + FKLREF_BIG_CHUNK <= batch; i += FKLREF_BIG_CHUNK) {
        crop_resize_chunk<FKLREF_BIG_CHUNK, AR, TAIL>(frames + i, w, h, pitch, rects + 4 * i, dw, dh, bg, p0, p1, p2,
                                                      out + plane_floats * i);
    }
#endif
    for (; i + 16 <= batch; i += 16) {
        crop_resize_chunk<16, AR, TAIL>(frames + i, w, h, pitch, rects + 4 * i, dw, dh, bg, p0, p1, p2,
                                        out + plane_floats * i);
    }
    for (; i + 2 <= batch; i += 2) {
        crop_resize_chunk<2, AR, TAIL>(frames + i, w, h, pitch, rects + 4 * i, dw, dh, bg, p0, p1, p2,
                                       out + plane_floats * i);
    }
    if (i < batch) { /* odd tail: run the last two planes again as a pair (idempotent) */
        if (batch >= 2) {
            crop_resize_chunk<2, AR, TAIL>(frames + batch - 2, w, h, pitch, rects + 4 * (batch - 2), dw, dh, bg,
                                           p0, p1, p2, out + plane_floats * (batch - 2));
        } else {
#ifdef FKLREF_GPU
            /* a batch of one plane is not instantiated for the CUDA build (the tests use two or more) */
#else
            /* batch == 1: a pair made of the same plane twice, second copy into scratch */
            const uint8_t* two_frames[2] = {frames[0], frames[0]};
            int two_rects[8];
            std::memcpy(two_rects, rects, 4 * sizeof(int));
            std::memcpy(two_rects + 4, rects, 4 * sizeof(int));
            float* scratch = new float[plane_floats * 2];
            crop_resize_chunk<2, AR, TAIL>(two_frames, w, h, pitch, two_rects, dw, dh, bg, p0, p1, p2, scratch);
            std::memcpy(out, scratch, plane_floats * sizeof(float));
            delete[] scratch;
#endif
        }
    }
}

}  // namespace

/* FKLREF_ONLY = 1, 2 or 3 compiles one entry point alone, so that the CUDA build (128 planes per
   launch, minutes per instantiation) can compile the three in parallel. */
#ifndef FKLREF_ONLY
#define FKLREF_ONLY 0
#endif

extern "C" {

#if FKLREF_ONLY == 0 || FKLREF_ONLY == 1
/* PerThreadRead<uchar3>[B] -> Crop[B] -> Resize<INTER_LINEAR,PRESERVE_AR>(dw,dh,bg) -> Mul -> Sub -> Div -> RGB2BGR
   -> TensorWrite<float3> (dw x dh x B, packed).  frames[i] is the source of plane i; rects = {x,y,w,h} per plane. */
void FKLREF_FN(crop_resize_readme)(const uint8_t* const* frames, int w, int h, int pitch, const int* rects, int batch,
                               int dw, int dh, const float* bg, const float* mul, const float* sub, const float* div,
                               float* out) {
    crop_resize_all<AspectRatio::PRESERVE_AR, Tail::README_PACKED>(frames, w, h, pitch, rects, batch, dw, dh, bg, mul,
                                                                   sub, div, out);
}

#endif
#if FKLREF_ONLY == 0 || FKLREF_ONLY == 2
/* Same read path, then Div(d0) -> Sub(mean) -> Div(std) -> TensorSplit<float3> (B x 3 x dh x dw, planar). */
void FKLREF_FN(crop_resize_norm_planar)(const uint8_t* const* frames, int w, int h, int pitch, const int* rects, int batch,
                                    int dw, int dh, const float* bg, const float* d0, const float* mean,
                                    const float* stdv, float* out) {
    crop_resize_all<AspectRatio::PRESERVE_AR, Tail::NORM_PLANAR>(frames, w, h, pitch, rects, batch, dw, dh, bg, d0,
                                                                 mean, stdv, out);
}

#endif
#if FKLREF_ONLY == 0 || FKLREF_ONLY == 3
/* Same as fklref_crop_resize_readme with Resize<INTER_LINEAR, IGNORE_AR> (no background). */
void FKLREF_FN(crop_resize_readme_ignore_ar)(const uint8_t* const* frames, int w, int h, int pitch, const int* rects,
                                         int batch, int dw, int dh, const float* mul, const float* sub,
                                         const float* div, float* out) {
    crop_resize_all<AspectRatio::IGNORE_AR, Tail::README_PACKED>(frames, w, h, pitch, rects, batch, dw, dh, nullptr,
                                                                 mul, sub, div, out);
}
#endif

#if FKLREF_ONLY == 0 && !defined(FKLREF_GPU)
/* The normalise-planar chain with the other aspect-ratio modes: mode 3 = PRESERVE_AR_RN_EVEN (target rounded down to an
   even size, resize.h:200-210), 4 = PRESERVE_AR_LEFT (region at column 0, resize.h:132-147).  Host build only. */
int FKLREF_FN(crop_resize_norm_planar_mode)(const uint8_t* const* frames, int w, int h, int pitch, const int* rects, int batch,
                                            int dw, int dh, int mode, const float* bg, const float* d0, const float* mean,
                                            const float* stdv, float* out) {
    if (mode == 3) crop_resize_all<AspectRatio::PRESERVE_AR_RN_EVEN, Tail::NORM_PLANAR>(frames, w, h, pitch, rects, batch, dw, dh, bg, d0, mean, stdv, out);
    else if (mode == 4) crop_resize_all<AspectRatio::PRESERVE_AR_LEFT, Tail::NORM_PLANAR>(frames, w, h, pitch, rects, batch, dw, dh, bg, d0, mean, stdv, out);
    else return -1;
    return 0;
}
#endif

}  // extern "C"
