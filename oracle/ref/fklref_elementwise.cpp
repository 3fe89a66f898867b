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

#ifdef FKLREF_GPU
namespace fklref {
cudaStream_t& current_stream() { static thread_local cudaStream_t s = nullptr; return s; }
long& launch_counter() { static thread_local long n = 0; return n; }
}  // namespace fklref

extern "C" {
/* Stream of the calling thread's next launches (NULL = the default stream). */
void fklref_gpu_set_stream(void* stream) { fklref::current_stream() = static_cast<cudaStream_t>(stream); }
/* Kernels launched by the calling thread so far (one per executeOperations call). */
long fklref_gpu_launches(void) { return fklref::launch_counter(); }
}
#endif

namespace {

/* ---- the element-wise chains on a batch of B images of one size, one launch (horizontal fusion:
 * PerThreadRead::build(std::array) distributes the continuation over the planes, iop_fuser.h:89-118) */
template <size_t B>
std::array<RawPtr<ND::_2D, uchar3>, B> batch_u8x3(const uint8_t* const* srcs, int w, int h, int pitch) {
    std::array<RawPtr<ND::_2D, uchar3>, B> a;
    for (size_t i = 0; i < B; ++i) a[i] = raw_u8x3(srcs[i], w, h, pitch);
    return a;
}

}  // namespace

extern "C" {

/* B = 16 images: Cast -> Mul -> Sub -> Div -> TensorWrite<float3> (16 x h x w packed) */
void FKLREF_FN(cast_mul_sub_div_batch16)(const uint8_t* const* srcs, int w, int h, int spitch, const float* mul,
                                         const float* sub, const float* div, float* dst) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(batch_u8x3<16>(srcs, w, h, spitch))
                            .then(Cast<uchar3, float3>::build())
                            .then(Mul<float3>::build(f3(mul)))
                            .then(Sub<float3>::build(f3(sub)))
                            .then(Div<float3>::build(f3(div)));
    executeOperations<RefDPP>(stream, sender, TensorWrite<float3>::build(raw_tensor<float3>(dst, w, h, 16, 1)));
    finish(stream);
}

/* B = 16: Cast -> Mul -> Sub -> TensorWrite<float3> */
void FKLREF_FN(cast_mul_sub_batch16)(const uint8_t* const* srcs, int w, int h, int spitch, const float* mul,
                                     const float* sub, float* dst) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(batch_u8x3<16>(srcs, w, h, spitch))
                            .then(Cast<uchar3, float3>::build())
                            .then(Mul<float3>::build(f3(mul)))
                            .then(Sub<float3>::build(f3(sub)));
    executeOperations<RefDPP>(stream, sender, TensorWrite<float3>::build(raw_tensor<float3>(dst, w, h, 16, 1)));
    finish(stream);
}

/* B = 16: Cast -> Add -> Div -> TensorWrite<float3> */
void FKLREF_FN(cast_add_div_batch16)(const uint8_t* const* srcs, int w, int h, int spitch, const float* add,
                                     const float* div, float* dst) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(batch_u8x3<16>(srcs, w, h, spitch))
                            .then(Cast<uchar3, float3>::build())
                            .then(Add<float3>::build(f3(add)))
                            .then(Div<float3>::build(f3(div)));
    executeOperations<RefDPP>(stream, sender, TensorWrite<float3>::build(raw_tensor<float3>(dst, w, h, 16, 1)));
    finish(stream);
}

/* B = 16: RGB2BGR(uchar3) -> Cast -> Mul -> SaturateCast<float3,uchar3> -> TensorWrite<uchar3> */
void FKLREF_FN(bgr_cast_mul_saturate_batch16)(const uint8_t* const* srcs, int w, int h, int spitch, const float* mul,
                                              uint8_t* dst) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(batch_u8x3<16>(srcs, w, h, spitch))
                            .then(ColorConversion<ColorConversionCodes::COLOR_RGB2BGR, uchar3, uchar3>::build())
                            .then(Cast<uchar3, float3>::build())
                            .then(Mul<float3>::build(f3(mul)))
                            .then(SaturateCast<float3, uchar3>::build());
    executeOperations<RefDPP>(stream, sender, TensorWrite<uchar3>::build(raw_tensor<uchar3>(dst, w, h, 16, 1)));
    finish(stream);
}

/* B = 16: Cast -> Resize<INTER_LINEAR, IGNORE_AR>(dw,dh) -> TensorWrite<float3> */
void FKLREF_FN(cast_resize_batch16)(const uint8_t* const* srcs, int w, int h, int spitch, int dw, int dh, float* dst) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(batch_u8x3<16>(srcs, w, h, spitch))
                            .then(Cast<uchar3, float3>::build())
                            .then(Resize<LINEAR>::build(Size(dw, dh)));
    executeOperations<RefDPP>(stream, sender, TensorWrite<float3>::build(raw_tensor<float3>(dst, dw, dh, 16, 1)));
    finish(stream);
}

#ifndef FKLREF_GPU
/* A partly filled batch of four images: planes at or beyond `used` read `default_value` instead of their image
   (BatchRead<4, CONDITIONAL_WITH_DEFAULT>, batch_operations.h:217-241); Cast -> Mul -> TensorWrite<float3>, the
   continuation handed over operation by operation so that it applies to the default value as well. */
void FKLREF_FN(batch4_default_cast_mul)(const uint8_t* const* srcs, int w, int h, int spitch, int used, const uint8_t* default_value,
                                        const float* mul, float* dst) {
    RefStream stream = make_stream();
    const uchar3 dv{default_value[0], default_value[1], default_value[2]};
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(used, dv, batch_u8x3<4>(srcs, w, h, spitch));
    executeOperations<RefDPP>(stream, read, Cast<uchar3, float3>::build(), Mul<float3>::build(f3(mul)),
                              TensorWrite<float3>::build(raw_tensor<float3>(dst, w, h, 4, 1)));
    finish(stream);
}
#endif

/* 1 when this library was built with the device-branch prelude, 0 for the literal CPU build. */
int FKLREF_FN(is_device_branch)(void) {
#ifdef FKLREF_DEVICE_BRANCH_PRELUDE_H
    return 1;
#else
    return 0;
#endif
}

/* PerThreadRead<uchar3> -> Cast<uchar3,float3> -> Mul -> Sub -> Div -> PerThreadWrite<float3> */
void FKLREF_FN(cast_mul_sub_div)(const uint8_t* src, int w, int h, int spitch, const float* mul, const float* sub,
                             const float* div, float* dst, int dpitch) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, spitch))
                            .then(Cast<uchar3, float3>::build())
                            .then(Mul<float3>::build(f3(mul)))
                            .then(Sub<float3>::build(f3(sub)))
                            .then(Div<float3>::build(f3(div)));
    const auto receiver = PerThreadWrite<ND::_2D, float3>::build(raw_f32x3(dst, w, h, dpitch));
    executeOperations<RefDPP>(stream, sender, receiver);
    finish(stream);
}

/* PerThreadRead<uchar3> -> Cast -> Mul -> Sub -> PerThreadWrite<float3> */
void FKLREF_FN(cast_mul_sub)(const uint8_t* src, int w, int h, int spitch, const float* mul, const float* sub,
                         float* dst, int dpitch) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, spitch))
                            .then(Cast<uchar3, float3>::build())
                            .then(Mul<float3>::build(f3(mul)))
                            .then(Sub<float3>::build(f3(sub)));
    const auto receiver = PerThreadWrite<ND::_2D, float3>::build(raw_f32x3(dst, w, h, dpitch));
    executeOperations<RefDPP>(stream, sender, receiver);
    finish(stream);
}

/* PerThreadRead<uchar3> -> Cast -> Add -> Div -> PerThreadWrite<float3> */
void FKLREF_FN(cast_add_div)(const uint8_t* src, int w, int h, int spitch, const float* add, const float* div,
                         float* dst, int dpitch) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, spitch))
                            .then(Cast<uchar3, float3>::build())
                            .then(Add<float3>::build(f3(add)))
                            .then(Div<float3>::build(f3(div)));
    const auto receiver = PerThreadWrite<ND::_2D, float3>::build(raw_f32x3(dst, w, h, dpitch));
    executeOperations<RefDPP>(stream, sender, receiver);
    finish(stream);
}

/* PerThreadRead<uchar3> -> RGB2BGR(uchar3) -> Cast -> Mul -> SaturateCast<float3,uchar3> -> PerThreadWrite<uchar3> */
void FKLREF_FN(bgr_cast_mul_saturate)(const uint8_t* src, int w, int h, int spitch, const float* mul, uint8_t* dst,
                                  int dpitch) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, spitch))
                            .then(ColorConversion<ColorConversionCodes::COLOR_RGB2BGR, uchar3, uchar3>::build())
                            .then(Cast<uchar3, float3>::build())
                            .then(Mul<float3>::build(f3(mul)))
                            .then(SaturateCast<float3, uchar3>::build());
    const auto receiver = PerThreadWrite<ND::_2D, uchar3>::build(raw_u8x3(dst, w, h, dpitch));
    executeOperations<RefDPP>(stream, sender, receiver);
    finish(stream);
}

/* PerThreadRead<uchar3> -> Cast<uchar3,float3> -> Mul -> Sub -> Cast<float3,int3> -> PerThreadWrite<int3> */
void FKLREF_FN(cast_mul_sub_cast_int3)(const uint8_t* src, int w, int h, int spitch, const float* mul, const float* sub,
                                       int32_t* dst, int dpitch) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, spitch))
                            .then(Cast<uchar3, float3>::build())
                            .then(Mul<float3>::build(f3(mul)))
                            .then(Sub<float3>::build(f3(sub)))
                            .then(Cast<float3, int3>::build());
    const auto receiver = PerThreadWrite<ND::_2D, int3>::build(
        RawPtr<ND::_2D, int3>{reinterpret_cast<int3*>(dst), PtrDims<ND::_2D>((uint)w, (uint)h, (uint)dpitch)});
    executeOperations<RefDPP>(stream, sender, receiver);
    finish(stream);
}

/* PerThreadRead<uchar3> -> Cast<uchar3,float3> -> Resize<INTER_LINEAR>(dw,dh) -> Mul -> Cast<float3,uint3>
   -> PerThreadWrite<uint3> (the shape of tests/operation/test_instantiable_operations.h:236-264) */
void FKLREF_FN(cast_resize_mul_cast_uint3)(const uint8_t* src, int w, int h, int spitch, int dw, int dh, const float* mul,
                                           uint32_t* dst, int dpitch) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, spitch))
                            .then(Cast<uchar3, float3>::build())
                            .then(Resize<LINEAR>::build(Size(dw, dh)))
                            .then(Mul<float3>::build(f3(mul)))
                            .then(Cast<float3, uint3>::build());
    const auto receiver = PerThreadWrite<ND::_2D, uint3>::build(
        RawPtr<ND::_2D, uint3>{reinterpret_cast<uint3*>(dst), PtrDims<ND::_2D>((uint)dw, (uint)dh, (uint)dpitch)});
    executeOperations<RefDPP>(stream, sender, receiver);
    finish(stream);
}

/* PerThreadRead<uchar3> -> Cast<uchar3,float3> -> Resize<INTER_LINEAR, IGNORE_AR>(dw,dh) -> PerThreadWrite<float3> */
void FKLREF_FN(cast_resize)(const uint8_t* src, int w, int h, int spitch, int dw, int dh, float* dst, int dpitch) {
    RefStream stream = make_stream();
    const auto sender = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(src, w, h, spitch))
                            .then(Cast<uchar3, float3>::build())
                            .then(Resize<LINEAR>::build(Size(dw, dh)));
    const auto receiver = PerThreadWrite<ND::_2D, float3>::build(raw_f32x3(dst, dw, dh, dpitch));
    executeOperations<RefDPP>(stream, sender, receiver);
    finish(stream);
}

/* Host-side resize parameters exactly as Resize::build derives them (resize.h:105-166,196-221).
   out = {fx, fy} as floats reinterpreted, then x1,y1,x2,y2 (PRESERVE_AR only; zeros otherwise). */
void FKLREF_FN(resize_params)(int sw, int sh, int dw, int dh, int preserve_ar, float* fxy, int* roi) {
    static uchar3 dummy;
    const auto back = PerThreadRead<ND::_2D, uchar3>::build(
        RawPtr<ND::_2D, uchar3>{&dummy, PtrDims<ND::_2D>((uint)sw, (uint)sh, (uint)(sw * 3))});
    using BackT = std::decay_t<decltype(back)>;
    if (preserve_ar) {
        const auto r = Resize<LINEAR, AspectRatio::PRESERVE_AR, BackT>::build(back, Size(dw, dh), float3{0, 0, 0});
        fxy[0] = r.params.src_conv_factors.x;
        fxy[1] = r.params.src_conv_factors.y;
        roi[0] = r.params.x1; roi[1] = r.params.y1; roi[2] = r.params.x2; roi[3] = r.params.y2;
    } else {
        const auto r = Resize<LINEAR, AspectRatio::IGNORE_AR, BackT>::build(back, Size(dw, dh));
        fxy[0] = r.params.src_conv_factors.x;
        fxy[1] = r.params.src_conv_factors.y;
        roi[0] = roi[1] = roi[2] = roi[3] = 0;
    }
}

}  // extern "C"
