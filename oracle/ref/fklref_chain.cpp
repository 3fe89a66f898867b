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

#include <tuple>
#include <utility>

namespace {

/* ---- alternating Add/Mul chain of compile-time length ------------------------------
 * The operations are handed to executeOperations as separate instantiable operations
 * (the parameter-pack form of fused_kernel.h:22-25; data_parallel_patterns.h:75-88 applies
 * them left to right), which computes the same values as chaining them with .then() but
 * instantiates far fewer templates for long chains. */
template <size_t... I>
void addmul_pairs(std::index_sequence<I...>, bool trailing_add, const float* src, int w, int h, int spitch,
                  const float* addv, const float* mulv, float* dst, int dpitch) {
    RefStream stream = make_stream();
    const auto read = PerThreadRead<ND::_2D, float3>::build(raw_f32x3(src, w, h, spitch));
    const auto add = Add<float3>::build(f3(addv));
    const auto mul = Mul<float3>::build(f3(mulv));
    const auto write = PerThreadWrite<ND::_2D, float3>::build(raw_f32x3(dst, w, h, dpitch));
    if (trailing_add) {
        const auto all = std::tuple_cat(std::make_tuple(read), ((void)I, std::make_tuple(add, mul))...,
                                        std::make_tuple(add, write));
        std::apply([&](const auto&... iops) { executeOperations<RefDPP>(stream, iops...); }, all);
    } else {
        const auto all = std::tuple_cat(std::make_tuple(read), ((void)I, std::make_tuple(add, mul))...,
                                        std::make_tuple(write));
        std::apply([&](const auto&... iops) { executeOperations<RefDPP>(stream, iops...); }, all);
    }
    finish(stream);
}

template <int N>
void addmul_chain(const float* src, int w, int h, int spitch, const float* addv, const float* mulv, float* dst,
                  int dpitch) {
    addmul_pairs(std::make_index_sequence<N / 2>{}, (N % 2) == 1, src, w, h, spitch, addv, mulv, dst, dpitch);
}

}  // namespace

extern "C" {

/* PerThreadRead<float3> -> n alternating Add(add)/Mul(mul) (Add first) -> PerThreadWrite<float3>.
   n must be one of 1, 2, 3, 16, 64, 256 (256: CPU build only); returns 0 on success, -1 for another n. */
int FKLREF_FN(addmul_chain)(const float* src, int w, int h, int spitch, int n, const float* addv, const float* mulv,
                        float* dst, int dpitch) {
    switch (n) {
        case 1: addmul_chain<1>(src, w, h, spitch, addv, mulv, dst, dpitch); return 0;
        case 2: addmul_chain<2>(src, w, h, spitch, addv, mulv, dst, dpitch); return 0;
        case 3: addmul_chain<3>(src, w, h, spitch, addv, mulv, dst, dpitch); return 0;
        case 16: addmul_chain<16>(src, w, h, spitch, addv, mulv, dst, dpitch); return 0;
        case 64: addmul_chain<64>(src, w, h, spitch, addv, mulv, dst, dpitch); return 0;
#ifndef FKLREF_GPU /* nvcc cannot deduce operate()'s return type at this recursion depth (data_parallel_patterns.h:86) */
        case 256: addmul_chain<256>(src, w, h, spitch, addv, mulv, dst, dpitch); return 0;
#endif
        default: return -1;
    }
}

}  // extern "C"
