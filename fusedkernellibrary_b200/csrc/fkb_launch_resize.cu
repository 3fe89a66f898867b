/* Instantiations of fused_plan_kernel for one group of plane classes (see fkb_bodies.cuh). */
#include "fkb_bodies.cuh"

namespace fkb {

cudaError_t launch_resize(uint32_t cls, uint32_t chain, const LaunchArgs& a, size_t smem, cudaStream_t stream) {
    switch (cls) {
        case CLASS_RESIZE_U8_PLANAR: return launch_class<CLASS_RESIZE_U8_PLANAR>(chain, a, smem, stream);
        case CLASS_RESIZE_U8_PACKED: return launch_class<CLASS_RESIZE_U8_PACKED>(chain, a, smem, stream);
        default: return launch_class<CLASS_RESIZE_NV12_PACKED>(chain, a, smem, stream);
    }
}

}  // namespace fkb
