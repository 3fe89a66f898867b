/* extern "C" entry points around the UNMODIFIED reference headers (CPU backend).
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
#ifndef FKLREF_COMMON_H
#define FKLREF_COMMON_H
#include <array>
#include <cstdint>
#include <cstring>

#include <fused_kernel/fused_kernel.h>
#include <fused_kernel/algorithms/algorithms.h>
#include <fused_kernel/algorithms/image_processing/image.h>

using namespace fk;

namespace fklref {

using CpuDPP = TransformDPP<ParArch::CPU>;
using CpuStream = Stream_<ParArch::CPU>;

constexpr auto LINEAR = InterpolationType::INTER_LINEAR;

inline float3 f3(const float* p) { return float3{p[0], p[1], p[2]}; }

inline RawPtr<ND::_2D, uchar3> raw_u8x3(const uint8_t* d, int w, int h, int pitch) {
    return RawPtr<ND::_2D, uchar3>{reinterpret_cast<uchar3*>(const_cast<uint8_t*>(d)),
                                   PtrDims<ND::_2D>((uint)w, (uint)h, (uint)pitch)};
}
inline RawPtr<ND::_2D, float3> raw_f32x3(const float* d, int w, int h, int pitch) {
    return RawPtr<ND::_2D, float3>{reinterpret_cast<float3*>(const_cast<float*>(d)),
                                   PtrDims<ND::_2D>((uint)w, (uint)h, (uint)pitch)};
}
template <typename T>
inline RawPtr<ND::_3D, T> raw_tensor(void* d, int w, int h, int planes, int color_planes) {
    return RawPtr<ND::_3D, T>{reinterpret_cast<T*>(d),
                              PtrDims<ND::_3D>((uint)w, (uint)h, (uint)planes, (uint)color_planes,
                                               (uint)(sizeof(T) * w))};
}

}  // namespace fklref

using namespace fklref;
#endif
