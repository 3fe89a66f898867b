/* Launcher of the fused-execution kernels: picks the instantiation of fused_plan_kernel for a
 * plan's class and continuation.  The kernels themselves are in fkb_bodies.cuh and are
 * instantiated by fkb_launch_*.cu; this unit holds the one-pixel-per-thread kernel that takes
 * anything the specialised bodies do not. */
#include "fkb_bodies.cuh"

namespace fkb {

bool chain_is_compiled(uint32_t chain) {
#define FKB_CHAIN_TEST(CH) if (chain == (CH)) return true;
    FKB_CHAIN_MENU(FKB_CHAIN_TEST)
#undef FKB_CHAIN_TEST
    return false;
}

/* launch_cls: one of CLASS_* or CLASS_MIXED; chain: a menu chain or CHAIN_INTERPRET. */
cudaError_t launch_plan_kernel(uint32_t launch_cls, uint32_t chain, const LaunchArgs& a, cudaStream_t stream) {
    const size_t ops_bytes = (size_t)(a.max_seq_ops > 0 ? a.max_seq_ops : 1) * sizeof(OpSlot);
    const size_t smem = a.staged_bytes ? ((ops_bytes + 127) & ~(size_t)127) + a.staged_bytes : ops_bytes;
    switch (launch_cls) {
        case CLASS_FLAT_U8_F32: case CLASS_FLAT_F32_F32: case CLASS_FLAT_U8_U8:
            return launch_flat(launch_cls, chain, a, smem, stream);
        case CLASS_RESIZE_U8_PLANAR: case CLASS_RESIZE_U8_PACKED: case CLASS_RESIZE_NV12_PACKED:
            return launch_resize(launch_cls, chain, a, smem, stream);
        case CLASS_RESIZE_U8_PLANAR_STAGED: case CLASS_RESIZE_U8_PACKED_STAGED:
            return launch_staged(launch_cls, chain, a, smem, stream);
        case CLASS_RESIZE_NV12_PACKED_STAGED: return launch_nv12_staged(chain, a, smem, stream);
        case CLASS_GENERIC: return launch_one<CLASS_GENERIC, CHAIN_INTERPRET>(a, smem, stream);
        default: return launch_mixed(a, smem, stream);
    }
}

}  // namespace fkb
