/* Instantiations of fused_plan_kernel for one group of plane classes (see fkb_bodies.cuh). */
#include "fkb_bodies.cuh"

namespace fkb {

cudaError_t launch_flat(uint32_t cls, uint32_t chain, const LaunchArgs& a, size_t smem, cudaStream_t stream) {
    switch (cls) {
        case CLASS_FLAT_U8_F32: return launch_class<CLASS_FLAT_U8_F32>(chain, a, smem, stream);
        case CLASS_FLAT_F32_F32: return launch_class<CLASS_FLAT_F32_F32>(chain, a, smem, stream);
        default: return launch_class<CLASS_FLAT_U8_U8>(chain, a, smem, stream);
    }
}

}  // namespace fkb
