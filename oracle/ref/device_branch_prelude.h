/* Force-included ahead of the reference headers when building the "device branch"
 * flavour of the reference library.
 *
 * TEST INFRASTRUCTURE ONLY - never part of the product path.
 *
 * The reference selects between two source branches with `#ifdef __CUDA_ARCH__`
 * (algorithms/image_processing/interpolation.h:65-71).  The host branch derives the
 * vertical tap index from the horizontal source coordinate (interpolation.h:70), the
 * device branch does not (interpolation.h:66-67).  Defining __CUDA_ARCH__ for a g++
 * build makes the host execute the device branch of the reference's own, unmodified
 * source; the three conversion intrinsics that branch (and color_conversion.h:58,64)
 * may name are given their documented round-down / round-to-nearest-even meaning.
 */
#ifndef FKLREF_DEVICE_BRANCH_PRELUDE_H
#define FKLREF_DEVICE_BRANCH_PRELUDE_H
#include <cmath>
#define __CUDA_ARCH__ 1000
static inline int          __float2int_rd (float f) { return (int)std::floor(f); }
static inline int          __float2int_rn (float f) { return (int)std::nearbyint(f); }
static inline unsigned int __float2uint_rn(float f) { return (unsigned int)std::nearbyint(f); }
#endif
