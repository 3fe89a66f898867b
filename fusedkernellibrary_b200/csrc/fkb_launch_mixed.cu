/* Instantiations of fused_plan_kernel for one group of plane classes (see fkb_bodies.cuh). */
#include "fkb_bodies.cuh"

namespace fkb {

cudaError_t launch_mixed(const LaunchArgs& a, size_t smem, cudaStream_t stream) {
    return launch_one<CLASS_MIXED, CHAIN_INTERPRET>(a, smem, stream);
}

}  // namespace fkb
