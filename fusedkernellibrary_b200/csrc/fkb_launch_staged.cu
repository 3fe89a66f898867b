/* Instantiations of fused_plan_kernel for one group of plane classes (see fkb_bodies.cuh). */
#include "fkb_bodies.cuh"

namespace fkb {

cudaError_t launch_staged(uint32_t cls, uint32_t chain, const LaunchArgs& a, size_t smem, cudaStream_t stream) {
    if (cls == CLASS_RESIZE_U8_PLANAR_STAGED) return launch_class<CLASS_RESIZE_U8_PLANAR_STAGED>(chain, a, smem, stream);
    return launch_class<CLASS_RESIZE_U8_PACKED_STAGED>(chain, a, smem, stream);
}

}  // namespace fkb
