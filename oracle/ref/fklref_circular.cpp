/* The reference's CircularTensor update on its own CUDA backend.
 *
 * TEST INFRASTRUCTURE ONLY (see fklref_common.h).  CircularTensor::update (core/data/circular_tensor.h:111-161)
 * hands its two operation sequences to Executor<DivergentBatchTransformDPP<...>>, which the reference does not
 * define, so update() itself cannot be built.  Its device code is complete, though: this unit builds the same two
 * sequences from the reference's own types, exactly as update() does (:121-134), and launches the reference's
 * launchDivergentBatchTransformDPP_Kernel (executor_details/executor_kernels.h:20-23) with the grid and block that
 * update() keeps in a comment (:136-142).  GPU build only; `visible` and `hidden` are device tensors of BATCH planes
 * that the caller owns, `first` is the caller's copy of m_nextUpdateIdx.
 */
#include "fklref_common.h"
#include <fused_kernel/core/data/circular_tensor.h>

#ifdef FKLREF_GPU
namespace {

template <int BATCH, CircularTensorOrder ORDER, typename WriteOp, typename PackOp, typename TensorT>
void circular_update(const uint8_t* frame, int w, int h, int pitch, const int* rect, int dw, int dh, const float* bg, const float* d0,
                     const float* mean, const float* stdv, const TensorT& visible, const TensorT& hidden, int first) {
    const auto chain = PerThreadRead<ND::_2D, uchar3>::build(raw_u8x3(frame, w, h, pitch))
                           .then(Crop<>::build(Rect(rect[0], rect[1], rect[2], rect[3])))
                           .then(Resize<LINEAR, AspectRatio::PRESERVE_AR>::build(Size(dw, dh), f3(bg)))
                           .then(Div<float3>::build(f3(d0)))
                           .then(Sub<float3>::build(f3(mean)))
                           .then(Div<float3>::build(f3(stdv)));
    const auto write = WriteOp::build(visible);

    MidWrite<CircularTensorWrite<CircularDirection::Ascendent, WriteOp, BATCH>> updateWriteToTemp;   /* :121-123 */
    updateWriteToTemp.params.first = first;
    updateWriteToTemp.params.opData.params = hidden;
    const auto updateOps = buildOperationSequence(chain, updateWriteToTemp, write);

    Read<CircularTensorRead<CTReadDirection_v<ORDER>, PackOp, BATCH>> nonUpdateRead;                 /* :129-132 */
    nonUpdateRead.params.first = first;
    nonUpdateRead.params.opData.params = hidden;
    const auto copyOps = buildOperationSequence(nonUpdateRead, write);

    const dim3 block(std::min(dw, 32), std::min(dh, 8));                                             /* :136-140 */
    const dim3 grid((uint)ceil((float)dw / (float)block.x), (uint)ceil((float)dh / (float)block.y), BATCH);
    ++launch_counter();
    launchDivergentBatchTransformDPP_Kernel<ParArch::GPU_NVIDIA, SequenceSelectorType<ORDER, BATCH>><<<grid, block, 0, current_stream()>>>(updateOps, copyOps);
}

/* plane z belongs to group z / 16 of four (sequence numbers are 1-based, data_parallel_patterns.h:316-325) */
struct GroupOf16 {
    FK_HOST_DEVICE_FUSE uint at(const uint& z) { return z / 16u + 1u; }
};

template <size_t B> std::array<RawPtr<ND::_2D, uchar3>, B> all_planes(const uint8_t* const* srcs, int w, int h, int pitch) {
    std::array<RawPtr<ND::_2D, uchar3>, B> a;
    for (size_t i = 0; i < B; ++i) a[i] = raw_u8x3(srcs[i], w, h, pitch);
    return a;
}

}  // namespace

extern "C" {

/* Configuration 5B as ONE launch of the reference's divergent kernel: 64 images, four chains on four groups of 16
   (Cast-Mul-Sub | Cast-Add-Div | BGR-Cast-Mul-Saturate | Cast-Resize).  Every sequence is a 64-plane batch of which the
   selector uses 16; g0..g3 are the groups' dense output tensors (16 planes each), addressed so that plane z of the launch
   is plane z - 16 * group of its tensor.  The reference has the kernel (executor_kernels.h:20-23) and no host launcher. */
int FKLREF_FN(divergent_four_groups64)(const uint8_t* const* srcs, int w, int h, int pitch, const float* mul, const float* sub,
                                       const float* add, const float* div, int dw, int dh, float* g0, float* g1, uint8_t* g2, float* g3) {
    const auto planes = all_planes<64>(srcs, w, h, pitch);
    const auto read = PerThreadRead<ND::_2D, uchar3>::build(planes);
    const size_t fplane = (size_t)w * h * 3, rplane = (size_t)dw * dh * 3;
    const auto s0 = buildOperationSequence(read.then(Cast<uchar3, float3>::build()).then(Mul<float3>::build(f3(mul))).then(Sub<float3>::build(f3(sub))),
                                           TensorWrite<float3>::build(raw_tensor<float3>(g0, w, h, 64, 1)));
    const auto s1 = buildOperationSequence(read.then(Cast<uchar3, float3>::build()).then(Add<float3>::build(f3(add))).then(Div<float3>::build(f3(div))),
                                           TensorWrite<float3>::build(raw_tensor<float3>(g1 - 16 * fplane, w, h, 64, 1)));
    const auto s2 = buildOperationSequence(read.then(ColorConversion<ColorConversionCodes::COLOR_RGB2BGR, uchar3, uchar3>::build())
                                               .then(Cast<uchar3, float3>::build()).then(Mul<float3>::build(f3(mul))).then(SaturateCast<float3, uchar3>::build()),
                                           TensorWrite<uchar3>::build(raw_tensor<uchar3>(g2 - 32 * fplane, w, h, 64, 1)));
    const auto s3 = buildOperationSequence(read.then(Cast<uchar3, float3>::build()).then(Resize<LINEAR>::build(Size(dw, dh))),
                                           TensorWrite<float3>::build(raw_tensor<float3>(g3 - 48 * rplane, dw, dh, 64, 1)));
    const dim3 block(32, 8);
    const dim3 grid((uint)ceil((float)w / 32.f), (uint)ceil((float)h / 8.f), 64);
    ++launch_counter();
    launchDivergentBatchTransformDPP_Kernel<ParArch::GPU_NVIDIA, GroupOf16><<<grid, block, 0, current_stream()>>>(s0, s1, s2, s3);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

/* One update of a 6-plane circular tensor whose planes are 3 x dh x dw floats (TensorSplit<float3> / TensorPack<float3>).
   order: 0 NewestFirst, 1 OldestFirst. */
int FKLREF_FN(circular_update_planar6)(const uint8_t* frame, int w, int h, int pitch, const int* rect, int dw, int dh, const float* bg,
                                       const float* d0, const float* mean, const float* stdv, float* visible, float* hidden, int first,
                                       int order) {
    const auto v = raw_tensor<float>(visible, dw, dh, 6, 3), t = raw_tensor<float>(hidden, dw, dh, 6, 3);
    if (order == 0)
        circular_update<6, CircularTensorOrder::NewestFirst, TensorSplit<float3>, TensorPack<float3>>(frame, w, h, pitch, rect, dw, dh, bg, d0, mean, stdv, v, t, first);
    else
        circular_update<6, CircularTensorOrder::OldestFirst, TensorSplit<float3>, TensorPack<float3>>(frame, w, h, pitch, rect, dw, dh, bg, d0, mean, stdv, v, t, first);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

/* The same with packed float3 planes (TensorWrite<float3> / TensorRead<float3>). */
int FKLREF_FN(circular_update_packed6)(const uint8_t* frame, int w, int h, int pitch, const int* rect, int dw, int dh, const float* bg,
                                       const float* d0, const float* mean, const float* stdv, float* visible, float* hidden, int first,
                                       int order) {
    const auto v = raw_tensor<float3>(visible, dw, dh, 6, 1), t = raw_tensor<float3>(hidden, dw, dh, 6, 1);
    if (order == 0)
        circular_update<6, CircularTensorOrder::NewestFirst, TensorWrite<float3>, TensorRead<float3>>(frame, w, h, pitch, rect, dw, dh, bg, d0, mean, stdv, v, t, first);
    else
        circular_update<6, CircularTensorOrder::OldestFirst, TensorWrite<float3>, TensorRead<float3>>(frame, w, h, pitch, rect, dw, dh, bg, d0, mean, stdv, v, t, first);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
#endif
