/* extern "C" entry points around the UNMODIFIED reference headers.
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
 *
 * The same sources are also compiled by nvcc with -DFKLREF_GPU: the chains then run on the
 * reference's own CUDA backend (TransformDPP<ParArch::GPU_NVIDIA>, executors.h:252-287,
 * executor_details/executor_kernels.h:25-29), every pointer is a device pointer, the entry points
 * are named fklref_gpu_* and return after the launch without synchronising, on the stream given
 * to fklref_gpu_set_stream.  That build is the reference's kernel on this GPU: a second checker
 * and the GPU baseline the benchmark reports.
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

#ifdef FKLREF_GPU
using RefDPP = TransformDPP<ParArch::GPU_NVIDIA>;
using RefStream = Stream_<ParArch::GPU_NVIDIA>;
constexpr MemType REF_MEM = MemType::Device;
/* the stream and the launch counter of the calling thread (fklref_elementwise.cpp) */
cudaStream_t& current_stream();
long& launch_counter();
inline RefStream make_stream() { ++launch_counter(); return RefStream(current_stream()); }
inline void finish(RefStream&) {} /* asynchronous: the caller times and synchronises */
#define FKLREF_FN(name) fklref_gpu_##name
/* planes per launch: the per-plane parameters travel in the kernel arguments (batch_operations.h:98-102),
   and about 136 bytes per plane fit the 32764-byte argument space 128 at a time */
#ifndef FKLREF_BIG_CHUNK
#define FKLREF_BIG_CHUNK 128
#endif
#else
using RefDPP = TransformDPP<ParArch::CPU>;
using RefStream = Stream_<ParArch::CPU>;
constexpr MemType REF_MEM = MemType::Host;
inline RefStream make_stream() { return RefStream(); }
inline void finish(RefStream& s) { s.sync(); }
#define FKLREF_FN(name) fklref_##name
#define FKLREF_BIG_CHUNK 16
#endif

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
