/* sm_100a kernels of the fused-execution path (bodies and the kernel template; the translation
 * units fkb_launch_*.cu instantiate them class by class so that they compile in parallel).
 *
 * One grid serves a whole plan: thread block b looks up its work item (plane, tile) in a
 * device-resident table, copies that plane's descriptor and its operation sequence into
 * shared memory, and runs the body selected by the plane's class.  A plan whose planes all
 * share one class is launched with that body alone; a plan with several classes (divergent
 * horizontal fusion, data_parallel_patterns.h:315-323) is launched with a block-uniform
 * switch over the bodies.
 *
 * The element-wise continuation of a chain is either one of a menu of chains compiled into
 * the kernel (the reference compiles every chain, data_parallel_patterns.h:75-88) or, for
 * any other sequence, interpreted from the operation table with a block-uniform switch.
 *
 * Arithmetic follows the reference's per-thread function exactly (execute_thread,
 * data_parallel_patterns.h:153-181): IEEE binary32, round to nearest even, no fused
 * multiply-add except inside the proven constant division, true division otherwise; every
 * operation is spelled with the __f*_rn intrinsics so that compiler flags cannot change the
 * rounding.
 */
#ifndef FKB_BODIES_CUH
#define FKB_BODIES_CUH
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <type_traits>

#include "fkb200.h"
#include "fkb_device.h"

namespace fkb {

/* ------------------------------------------------------------------------------------ */
/* element-wise operations                                                              */
/* ------------------------------------------------------------------------------------ */

/* SaturateCast<float, uchar>: clamp, then cxp::round = (int)(x + 0.5f) for x > 0
 * (image_processing/saturate.h:27-50, constexpr_libs/constexpr_cmath.h:119-130). */
__device__ __forceinline__ float saturate_round_u8(float f) {
    /* (int)(t) of t = f + 0.5f in [0.5, 255.5] is floor(t): adding 2^23 rounded down leaves
       2^23 + floor(t), and taking 2^23 off again is exact.  Same values as a float -> int -> float
       round trip, without two trips through the quarter-rate conversion unit.  fmaxf maps NaN to
       0 as the comparisons of the reference's clamp followed by the conversion do. */
    const float t = __fadd_rn(fminf(fmaxf(f, 0.0f), 255.0f), 0.5f);
    return __fadd_rn(__fadd_rd(t, 8388608.0f), -8388608.0f);
}

/* The same result still under the exponent of 2^23 (2^23 + the byte): for a chain whose last operation it is and whose
   receiver packs bytes, which would add 2^23 again to get at the byte. */
__device__ __forceinline__ float saturate_round_u8_biased(float f) {
    return __fadd_rd(__fadd_rn(fminf(fmaxf(f, 0.0f), 255.0f), 0.5f), 8388608.0f);
}

/* Exact uchar -> float.  Converting from a 32-bit integer (not from an 8-bit one) keeps the
   conversion off the quarter-rate conversion unit. */
__device__ __forceinline__ float u8_to_float(uint32_t b) { return __int2float_rn((int)b); }

/* Lowest byte of w, as float.  Written as shift-and-mask at the call site so that the compiler
   can use the integer-to-float conversion that takes a byte of its source register directly. */
__device__ __forceinline__ float byte_to_float(uint32_t w) { return __int2float_rn((int)(w & 0xFFu)); }

/* Byte LANE of a packed word, as float: one byte permute builds 2^23 + b, one add removes 2^23. */
template <int LANE>
__device__ __forceinline__ float packed_u8_to_float(uint32_t w) {
    return __fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440 | LANE)), 8388608.0f);
}

/* Byte `lane` of a and of b as a float pair, the same way with one packed add for the two. */
__device__ __forceinline__ float2 bytes_to_float2_by_bias(uint32_t a, uint32_t b, int lane) {
    const float2 biased = make_float2(__uint_as_float(__byte_perm(a, 0x4B000000u, 0x7440 | lane)),
                                      __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7440 | lane)));
    return __fadd2_rn(biased, make_float2(-8388608.0f, -8388608.0f));
}

/* x / p for a divisor known when the plan was made: with r = RN(1/p),
 *     q0 = RN(x*r);  e = x - p*q0 (exact, one FMA);  q = RN(q0 + e*r)
 * The host emits this form only for divisors for which it has checked the sequence against
 * IEEE division on all 2^23 significands of x, and only where it has shown that x stays in
 * the range in which scaling by powers of two is exact (constant_division_is_exact and
 * advance_range in fkb_host.cu).  np is -p. */
__device__ __forceinline__ float div_by_constant(float x, float np, float r) {
    const float q0 = __fmul_rn(x, r);
    const float e = __fmaf_rn(np, q0, x);
    return __fmaf_rn(e, r, q0);
}

/* ConvertYUVToRGB<NV12, Full, bt709, false, float3> (color_conversion.h:265-308; matrix
 * :143-146; row reduction left to right, basic_ops/algebraic.h:58-64).  The reference computes
 *     R = ((y*1 + u*0) + v*1.5748) * 1,  G = ((y*1 + u*-0.1873) + v*-0.4681) * 1,  B = ((y*1 + u*1.8556) + v*0) * 1
 * with u, v already reduced by 128.  The operations dropped below cannot change a bit: x*1 is x;
 * y is a converted byte, so it is +0 or positive and y + (+-0) is y; and y + u*1.8556 is never -0
 * (a sum of a non-negative and a product rounds to +0 when it cancels), so adding v*0 = +-0 leaves
 * it as it is. */
__device__ __forceinline__ void yuv_to_rgb_bt709_full(float& a, float& b, float& c) {
    const float y = a, u = __fsub_rn(b, 128.0f), v = __fsub_rn(c, 128.0f);
    a = __fadd_rn(y, __fmul_rn(v, 1.5748f));
    b = __fadd_rn(__fadd_rn(y, __fmul_rn(u, -0.1873f)), __fmul_rn(v, -0.4681f));
    c = __fadd_rn(y, __fmul_rn(u, 1.8556f));
}

/* ConvertYUVToRGB<PF, Full, bt601, false, float3>: the luma offset 16 is subtracted as well (:266-269), matrix :137-140.
 * The dropped terms are no-ops for the same reasons: (y-16)*k is +0 or non-zero, so adding u*0 = +-0 leaves it; a sum
 * of two finite terms is never -0 unless both are, and (y-16)*k is never -0. */
__device__ __forceinline__ void yuv_to_rgb_bt601_full(float& a, float& b, float& c) {
    const float y = __fmul_rn(__fsub_rn(a, 16.0f), 1.164383562f), u = __fsub_rn(b, 128.0f), v = __fsub_rn(c, 128.0f);
    a = __fadd_rn(y, __fmul_rn(v, 1.596026786f));
    b = __fadd_rn(__fadd_rn(y, __fmul_rn(u, -0.39176229f)), __fmul_rn(v, -0.812967647f));
    c = __fadd_rn(y, __fmul_rn(u, 2.017232143f));
}
/* ConvertYUVToRGB<PF, Full, bt2020, false, float3>: matrix :165-168, otherwise as bt709. */
__device__ __forceinline__ void yuv_to_rgb_bt2020_full(float& a, float& b, float& c) {
    const float y = a, u = __fsub_rn(b, 128.0f), v = __fsub_rn(c, 128.0f);
    a = __fadd_rn(y, __fmul_rn(v, 1.4746f));
    b = __fadd_rn(__fadd_rn(y, __fmul_rn(u, -0.16455312684366f)), __fmul_rn(v, -0.57135312684366f));
    c = __fadd_rn(y, __fmul_rn(u, 1.8814f));
}
/* The conversion a sequence asks for before the interpolation (block-uniform). */
__device__ __forceinline__ void yuv_to_rgb(int pre_kind, float& a, float& b, float& c) {
    if (pre_kind == PRE_YUV_BT709) yuv_to_rgb_bt709_full(a, b, c);
    else if (pre_kind == PRE_YUV_BT601) yuv_to_rgb_bt601_full(a, b, c);
    else if (pre_kind == PRE_YUV_BT2020) yuv_to_rgb_bt2020_full(a, b, c);
}

/* Packed binary32 arithmetic (sm_100): one instruction rounds two independent products, sums
 * or fused multiply-adds, each to nearest even exactly like the scalar instruction.  Values
 * travel as pairs of horizontally adjacent pixels, one pair per channel. */
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 dup2(float a) { return make_float2(a, a); }
/* a + b as RN(a*1 + b), which is the same value for every input including signed zeros.  The
 * packed add itself cannot be used after a packed multiply: the assembler contracts
 * mul.rn.f32x2 + add.rn.f32x2 into one fused multiply-add even with contraction disabled
 * (measured on this toolchain: the fused result differs from the separately rounded one on
 * 15 % of random inputs), and a literal 1.0 is folded back into an add and contracted too.
 * `one` is therefore (1, 1) read from the plan's descriptor at run time. */
__device__ __forceinline__ float2 add2(float2 a, float2 b, float2 one) { return __ffma2_rn(a, one, b); }

/* The block's copy of its sequence's operation table, laid out for packed arithmetic: slot k
 * holds four pairs, (p0,p0) (p1,p1) (p2,p2) (opcode bits, 0), so that a per-channel parameter
 * arrives as a register pair with one 8-byte shared-memory load.  Sub is stored negated
 * (x - p == x + (-p) exactly); a division by a plan-time constant takes two slots: -p, then 1/p. */
struct OpSlot {
    float2 p[3];
    int32_t opcode;
    int32_t pad;
};
static_assert(sizeof(OpSlot) == 32, "OpSlot layout");

__device__ __forceinline__ void expand_op(const uint4 g, OpSlot* slot) {
    const int32_t opcode = (int32_t)g.x;
    float p0 = __uint_as_float(g.y), p1 = __uint_as_float(g.z), p2 = __uint_as_float(g.w);
    if (opcode == FKB_OP_SUB) { p0 = -p0; p1 = -p1; p2 = -p2; }
    reinterpret_cast<float4*>(slot)[0] = make_float4(p0, p0, p1, p1);
    reinterpret_cast<float4*>(slot)[1] = make_float4(p2, p2, __int_as_float(opcode), 0.0f);
}

/* One operation on NPAIR pixel pairs held as v[3*j + channel] = (pixel 2j, pixel 2j+1); `s` is the
   operation's slot (and s[1] the second slot of a two-slot operation). */
template <int CODE, int NPAIR, bool BIASED = false, bool UNIFORM = false>
__device__ __forceinline__ void apply_one(float2 (&v)[NPAIR * 3], const OpSlot* __restrict__ s, const float2 one) {
    if (CODE == CH_CASTI || CODE == CH_CASTU) {
        /* Cast<float3,int3> / Cast<float3,uint3>: static_cast truncates toward zero (cast_base.h:20-30); the
           integer travels on as a bit pattern in the same registers and is stored as it is */
#pragma unroll
        for (int k = 0; k < NPAIR * 3; ++k) {
            if (CODE == CH_CASTI) v[k] = make_float2(__int_as_float(__float2int_rz(v[k].x)), __int_as_float(__float2int_rz(v[k].y)));
            else v[k] = make_float2(__uint_as_float(__float2uint_rz(v[k].x)), __uint_as_float(__float2uint_rz(v[k].y)));
        }
        return;
    }
    if (CODE == CH_SWAP || CODE == CH_SAT || CODE == CH_YUV || CODE == CH_YUV601 || CODE == CH_YUV2020) {
#pragma unroll
        for (int j = 0; j < NPAIR; ++j) {
            float2& a = v[3 * j + 0];
            float2& b = v[3 * j + 1];
            float2& c = v[3 * j + 2];
            if (CODE == CH_SWAP) { const float2 t = a; a = c; c = t; }
            else if (CODE == CH_SAT && BIASED) {
                a = make_float2(saturate_round_u8_biased(a.x), saturate_round_u8_biased(a.y));
                b = make_float2(saturate_round_u8_biased(b.x), saturate_round_u8_biased(b.y));
                c = make_float2(saturate_round_u8_biased(c.x), saturate_round_u8_biased(c.y));
            } else if (CODE == CH_SAT) {
                a = make_float2(saturate_round_u8(a.x), saturate_round_u8(a.y));
                b = make_float2(saturate_round_u8(b.x), saturate_round_u8(b.y));
                c = make_float2(saturate_round_u8(c.x), saturate_round_u8(c.y));
            } else {
                constexpr int KIND = CODE == CH_YUV ? PRE_YUV_BT709 : CODE == CH_YUV601 ? PRE_YUV_BT601 : PRE_YUV_BT2020;
                yuv_to_rgb(KIND, a.x, b.x, c.x);
                yuv_to_rgb(KIND, a.y, b.y, c.y);
            }
        }
        return;
    }
    const float2 p0 = s[0].p[0], p1 = UNIFORM ? p0 : s[0].p[1], p2 = UNIFORM ? p0 : s[0].p[2]; /* UNIFORM: one parameter for the three channels */
#pragma unroll
    for (int j = 0; j < NPAIR; ++j) {
        float2& a = v[3 * j + 0];
        float2& b = v[3 * j + 1];
        float2& c = v[3 * j + 2];
        if (CODE == CH_MUL) { a = mul2(a, p0); b = mul2(b, p1); c = mul2(c, p2); }
        else if (CODE == CH_DIV) {
            a = make_float2(__fdiv_rn(a.x, p0.x), __fdiv_rn(a.y, p0.x));
            b = make_float2(__fdiv_rn(b.x, p1.x), __fdiv_rn(b.y, p1.x));
            c = make_float2(__fdiv_rn(c.x, p2.x), __fdiv_rn(c.y, p2.x));
        } else if (CODE == CH_ADD || CODE == CH_SUB) { a = add2(a, p0, one); b = add2(b, p1, one); c = add2(c, p2, one); }
        else if (CODE == CH_DIVC) { /* div_by_constant on both halves: p holds -divisor, r its reciprocal */
            const float2 r0 = s[1].p[0], r1 = UNIFORM ? r0 : s[1].p[1], r2 = UNIFORM ? r0 : s[1].p[2];
            const float2 qa = mul2(a, r0), qb = mul2(b, r1), qc = mul2(c, r2);
            a = fma2(fma2(p0, qa, a), r0, qa); b = fma2(fma2(p1, qb, b), r1, qb); c = fma2(fma2(p2, qc, c), r2, qc);
        }
    }
}

/* `count` rounds of one or two operations out of Mul and Add (Sub is stored as an addition of the
 * negated parameter), with the parameters held in registers across the loop. */
template <int NPAIR>
__device__ __forceinline__ void repeat_ops(float2 (&v)[NPAIR * 3], const OpSlot* __restrict__ body, int count, int period,
                                           const float2 one) {
    const bool mul0 = body[0].opcode == FKB_OP_MUL;
    const float2 a0 = body[0].p[0], a1 = body[0].p[1], a2 = body[0].p[2];
    if (period == 1) {
        if (mul0) {
#pragma unroll 1
            for (int r = 0; r < count; ++r)
#pragma unroll
                for (int j = 0; j < NPAIR; ++j) { v[3 * j] = mul2(v[3 * j], a0); v[3 * j + 1] = mul2(v[3 * j + 1], a1); v[3 * j + 2] = mul2(v[3 * j + 2], a2); }
        } else {
#pragma unroll 1
            for (int r = 0; r < count; ++r)
#pragma unroll
                for (int j = 0; j < NPAIR; ++j) { v[3 * j] = add2(v[3 * j], a0, one); v[3 * j + 1] = add2(v[3 * j + 1], a1, one); v[3 * j + 2] = add2(v[3 * j + 2], a2, one); }
        }
        return;
    }
    const bool mul1 = body[1].opcode == FKB_OP_MUL;
    const float2 b0 = body[1].p[0], b1 = body[1].p[1], b2 = body[1].p[2];
#define FKB_REPEAT_PAIR(OP0, OP1)                                                                      \
    _Pragma("unroll 1") for (int r = 0; r < count; ++r) {                                              \
        _Pragma("unroll") for (int j = 0; j < NPAIR; ++j) {                                            \
            v[3 * j] = OP0(v[3 * j], a0); v[3 * j + 1] = OP0(v[3 * j + 1], a1); v[3 * j + 2] = OP0(v[3 * j + 2], a2); \
            v[3 * j] = OP1(v[3 * j], b0); v[3 * j + 1] = OP1(v[3 * j + 1], b1); v[3 * j + 2] = OP1(v[3 * j + 2], b2); \
        }                                                                                              \
    }
    auto MUL = [&](float2 x, float2 p) { return mul2(x, p); };
    auto ADD = [&](float2 x, float2 p) { return add2(x, p, one); };
    if (mul0 && mul1) { FKB_REPEAT_PAIR(MUL, MUL) }
    else if (mul0) { FKB_REPEAT_PAIR(MUL, ADD) }
    else if (mul1) { FKB_REPEAT_PAIR(ADD, MUL) }
    else { FKB_REPEAT_PAIR(ADD, ADD) }
#undef FKB_REPEAT_PAIR
}

/* Interpreter: runs ops [begin, end) of a sequence cached in shared memory.  The opcode is
 * uniform across the block, so the switch never diverges. */
template <int NPAIR>
__device__ __forceinline__ void interpret_ops(float2 (&v)[NPAIR * 3], const OpSlot* __restrict__ sops, int begin, int end,
                                              const float2 one) {
    for (int k = begin; k < end; ++k) {
        switch (sops[k].opcode) {
            case FKB_OP_MUL: apply_one<CH_MUL, NPAIR>(v, sops + k, one); break;
            case FKB_OP_SUB: apply_one<CH_SUB, NPAIR>(v, sops + k, one); break;
            case FKB_OP_DIV: apply_one<CH_DIV, NPAIR>(v, sops + k, one); break;
            case FKB_OP_ADD: apply_one<CH_ADD, NPAIR>(v, sops + k, one); break;
            case DEV_OP_DIV_BY_CONSTANT: /* two slots: {-p}, {1/p} */
                apply_one<CH_DIVC, NPAIR>(v, sops + k, one);
                ++k;
                break;
            case DEV_OP_REPEAT: {
                /* header: p[0] = (count, count), p[1] = (period, period) as integer bit patterns; the
                   body's opcodes are dispatched once, outside the counted loop */
                const int count = __float_as_int(sops[k].p[0].x), period = __float_as_int(sops[k].p[1].x);
                repeat_ops<NPAIR>(v, sops + k + 1, count, period, one);
                k += period;
                break;
            }
            case FKB_OP_SWAP_RB: apply_one<CH_SWAP, NPAIR>(v, sops + k, one); break;
            case FKB_OP_SATURATE_CAST_U8: apply_one<CH_SAT, NPAIR>(v, sops + k, one); break;
            case FKB_OP_YUV_TO_RGB_BT709_FULL: apply_one<CH_YUV, NPAIR>(v, sops + k, one); break;
            case FKB_OP_YUV_TO_RGB_BT601_FULL: apply_one<CH_YUV601, NPAIR>(v, sops + k, one); break;
            case FKB_OP_YUV_TO_RGB_BT2020_FULL: apply_one<CH_YUV2020, NPAIR>(v, sops + k, one); break;
            case FKB_OP_CAST_I32: apply_one<CH_CASTI, NPAIR>(v, sops + k, one); break;
            case FKB_OP_CAST_U32: apply_one<CH_CASTU, NPAIR>(v, sops + k, one); break;
            default: break;
        }
    }
}

/* A chain fixed at compile time: operation codes in the nibbles of CHAIN, parameters taken
   from consecutive slots of the cached operation table starting at `slot`. */
/* BIASED_LAST: a SaturateCast that ends the chain leaves its results under the exponent of 2^23 (chain_ends_biased). */
template <uint32_t CHAIN, int NPAIR, bool BIASED_LAST = false, bool UNIFORM = false>
__device__ __forceinline__ void apply_chain(float2 (&v)[NPAIR * 3], const OpSlot* __restrict__ sops, int slot, const float2 one) {
    constexpr uint32_t CODE = CHAIN & 0xFu;
    if constexpr (CODE != 0) {
        apply_one<CODE, NPAIR, (BIASED_LAST && CODE == CH_SAT && (CHAIN >> 4) == 0u), UNIFORM>(v, sops + slot, one);
        apply_chain<(CHAIN >> 4), NPAIR, BIASED_LAST, UNIFORM>(v, sops, slot + (CODE == CH_DIVC ? 2 : 1), one);
    }
}

/* Whether a compiled chain ends in SaturateCast: a receiver that packs bytes then takes them from under the exponent. */
__host__ __device__ constexpr bool chain_ends_biased(uint32_t chain) {
    if (chain == CHAIN_INTERPRET || chain == 0u) return false;
    chain &= ~CHAIN_UNIFORM;
    while ((chain >> 4) != 0u) chain >>= 4;
    return chain == CH_SAT;
}

template <uint32_t CHAIN, int NPAIR, bool BIASED_LAST = false>
__device__ __forceinline__ void run_ops(float2 (&v)[NPAIR * 3], const OpSlot* __restrict__ sops, int begin, int end,
                                        const float2 one) {
    if constexpr (CHAIN == CHAIN_INTERPRET) interpret_ops<NPAIR>(v, sops, begin, end, one);
    else apply_chain<(CHAIN & ~CHAIN_UNIFORM), NPAIR, BIASED_LAST, (CHAIN & CHAIN_UNIFORM) != 0u>(v, sops, begin, one);
}

/* The same on one pixel (both halves of a pair carry it). */
template <uint32_t CHAIN>
__device__ __forceinline__ void run_ops_1(float (&v)[3], const OpSlot* __restrict__ sops, int begin, int end, const float2 one) {
    float2 p[3] = {dup2(v[0]), dup2(v[1]), dup2(v[2])};
    run_ops<CHAIN, 1>(p, sops, begin, end, one);
    v[0] = p[0].x; v[1] = p[1].x; v[2] = p[2].x;
}

/* ------------------------------------------------------------------------------------ */
/* checked accesses                                                                     */
/* ------------------------------------------------------------------------------------ */
/* Every load from a source image goes through gld(), every store to a destination through gst(), every shared-memory
 * access of the staged bodies through the lds helpers.  In the ordinary build they are the plain instruction.  Built
 * with -DFKB_CHECK_BOUNDS (libfkb200_check.so, the stand-in for a memory checker) each access is first compared with
 * what the block's plane allows - the source image's rows, the destination's rows (row by row: padding between rows
 * counts as outside), the block's shared memory - and an access outside is NOT made: the plan's status word receives
 * STATUS_BOUNDS_* and the access is skipped (a load gives zero), so that nothing faults and the host reads the
 * status like that of a wait that ran out. */
#ifdef FKB_CHECK_BOUNDS
struct CheckCtx {
    const uint8_t* src_lo; const uint8_t* src_hi;   /* all rows of the source image (luma and chroma for NV12) */
    uint8_t* dst;                                   /* first byte of the destination plane (or column tile) */
    uint32_t dst_pitch, dst_rows, dst_row_bytes, dst_cstride, dst_channels;
    uint32_t smem_lo, smem_hi;                      /* the block's dynamic shared memory, as shared-window addresses */
    uint32_t* status;
};
static __shared__ CheckCtx s_check;
__device__ __forceinline__ bool check_fail(uint32_t code) { atomicMax(s_check.status, code); return false; }
__device__ __forceinline__ bool check_src(const void* p, uint32_t n) {
    const uint8_t* b = static_cast<const uint8_t*>(p);
    return (b >= s_check.src_lo && b + n <= s_check.src_hi) ? true : check_fail(STATUS_BOUNDS_SOURCE);
}
__device__ __forceinline__ bool check_dst(const void* p, uint32_t n) {
    const uint8_t* b = static_cast<const uint8_t*>(p);
    if (b < s_check.dst) return check_fail(STATUS_BOUNDS_DESTINATION);
    size_t off = (size_t)(b - s_check.dst);
    if (s_check.dst_channels > 1) { /* planar: channel planes dst_cstride apart */
        const size_t ch = off / s_check.dst_cstride;
        if (ch >= s_check.dst_channels) return check_fail(STATUS_BOUNDS_DESTINATION);
        off -= ch * s_check.dst_cstride;
    }
    if (s_check.dst_pitch == s_check.dst_row_bytes) /* dense rows: one run of bytes, a 16-byte word may straddle two rows */
        return off + n <= (size_t)s_check.dst_rows * s_check.dst_pitch ? true : check_fail(STATUS_BOUNDS_DESTINATION);
    const size_t row = off / s_check.dst_pitch, in_row = off - row * s_check.dst_pitch;
    return (row < s_check.dst_rows && in_row + n <= s_check.dst_row_bytes) ? true : check_fail(STATUS_BOUNDS_DESTINATION);
}
__device__ __forceinline__ bool check_smem(uint32_t addr, uint32_t n) {
    return (addr >= s_check.smem_lo && addr + n <= s_check.smem_hi) ? true : check_fail(STATUS_BOUNDS_SHARED);
}
template <typename T> __device__ __forceinline__ T gld(const T* p) { return check_src(p, (uint32_t)sizeof(T)) ? __ldg(p) : T{}; }
template <typename T> __device__ __forceinline__ void gst(T* p, const T& v) { if (check_dst(p, (uint32_t)sizeof(T))) *p = v; }
#else
template <typename T> __device__ __forceinline__ T gld(const T* p) { return __ldg(p); }
template <typename T> __device__ __forceinline__ void gst(T* p, const T& v) { *p = v; }
__device__ __forceinline__ bool check_src(const void*, uint32_t) { return true; }
__device__ __forceinline__ bool check_smem(uint32_t, uint32_t) { return true; }
#endif

/* ------------------------------------------------------------------------------------ */
/* reads                                                                                */
/* ------------------------------------------------------------------------------------ */

/* The read operation at crop-relative (a, b): Crop::exec adds the rect origin
 * (image_processing/crop.h:35-38); PerThreadRead loads base + y*pitch + x*sizeof(T)
 * (memory_operations.h:80-83, core/data/rawptr.h:205-207); ReadYUV<NV12> takes Y at (x,y)
 * and the U,V pair at (x>>1, y>>1) of the plane starting at base + pitch*height
 * (color_conversion.h:329-346). */
template <int SRC>
__device__ __forceinline__ void read_tap(const DevPlane& P, int a, int b, float& r0, float& r1, float& r2, bool swap_uv = false) {
    const int x = a + P.crop_x, y = b + P.crop_y;
    if (SRC == FKB_SRC_U8X3) {
        const uint8_t* p = P.src + (size_t)y * P.src_pitch + (size_t)x * 3;
        r0 = u8_to_float(gld(p)); r1 = u8_to_float(gld(p + 1)); r2 = u8_to_float(gld(p + 2));
    } else if (SRC == FKB_SRC_F32X3) {
        const float* p = reinterpret_cast<const float*>(P.src + (size_t)y * P.src_pitch + (size_t)x * 12);
        r0 = gld(p); r1 = gld(p + 1); r2 = gld(p + 2);
    } else {
        const uint8_t* luma = P.src + (size_t)y * P.src_pitch + (size_t)x;
        const uint8_t* chroma = P.src + (size_t)P.src_pitch * P.src_height + (size_t)(y >> 1) * P.src_pitch +
                                (size_t)(x >> 1) * 2;
        r0 = u8_to_float(gld(luma));
        r1 = u8_to_float(gld(chroma + (swap_uv ? 1 : 0))); /* NV21 stores the pair as V,U (color_conversion.h:357-359) */
        r2 = u8_to_float(gld(chroma + (swap_uv ? 0 : 1)));
    }
}

/* ConvertYUVToRGB<PF, Full, CP, false, float3> on a pixel of a 10-bit layout (color_conversion.h:284-309): the words were
 * shifted right by 6 when they were read (:292); the chroma offset is 512 and, for bt601, the luma offset 64 (:187-191);
 * the result is multiplied by 64 (NormalizeColorRangeDepth, :234-252).  The matrix rows are evaluated as in the 8-bit
 * functions above, whose reasoning about the dropped zero terms holds for any non-negative integer luma. */
__device__ __forceinline__ void yuv_to_rgb_10bit(int kind, float& a, float& b, float& c) {
    const float u = __fsub_rn(b, 512.0f), v = __fsub_rn(c, 512.0f);
    float r, g, bl;
    if (kind == PRE_YUV_BT601) {
        const float y = __fmul_rn(__fsub_rn(a, 64.0f), 1.164383562f);
        r = __fadd_rn(y, __fmul_rn(v, 1.596026786f));
        g = __fadd_rn(__fadd_rn(y, __fmul_rn(u, -0.39176229f)), __fmul_rn(v, -0.812967647f));
        bl = __fadd_rn(y, __fmul_rn(u, 2.017232143f));
    } else if (kind == PRE_YUV_BT709) {
        r = __fadd_rn(a, __fmul_rn(v, 1.5748f));
        g = __fadd_rn(__fadd_rn(a, __fmul_rn(u, -0.1873f)), __fmul_rn(v, -0.4681f));
        bl = __fadd_rn(a, __fmul_rn(u, 1.8556f));
    } else {
        r = __fadd_rn(a, __fmul_rn(v, 1.4746f));
        g = __fadd_rn(__fadd_rn(a, __fmul_rn(u, -0.16455312684366f)), __fmul_rn(v, -0.57135312684366f));
        bl = __fadd_rn(a, __fmul_rn(u, 1.8814f));
    }
    a = __fmul_rn(r, 64.0f); b = __fmul_rn(g, 64.0f); c = __fmul_rn(bl, 64.0f);
}

/* ReadYUV<P010 | P210 | Y210 | UYVY> at image (x, y) followed by the sequence's conversion (color_conversion.h:329-372). */
__device__ __forceinline__ void read_converted_yuv(const DevSeq& S, const DevPlane& P, int x, int y, float& r0, float& r1, float& r2) {
    const uint8_t* const row = P.src + (size_t)y * P.src_pitch;
    uint32_t Y, U, V;
    if (S.src_format == FKB_SRC_P010 || S.src_format == FKB_SRC_P210) {
        Y = gld(reinterpret_cast<const uint16_t*>(row) + x);
        const int cy = S.src_format == FKB_SRC_P010 ? (y >> 1) : y; /* 4:2:0 halves the chroma rows, 4:2:2 does not (:343-344) */
        const uint16_t* uv = reinterpret_cast<const uint16_t*>(P.src + (size_t)P.src_pitch * P.src_height + (size_t)cy * P.src_pitch) + 2 * (x >> 1);
        U = gld(uv); V = gld(uv + 1);
    } else if (S.src_format == FKB_SRC_Y210) {
        const uint16_t* q = reinterpret_cast<const uint16_t*>(row) + 4 * (x >> 1); /* Y0 U Y1 V */
        Y = gld(q + ((x & 1) ? 2 : 0)); U = gld(q + 1); V = gld(q + 3);
    } else { /* UYVY: U Y0 V Y1 */
        const uint8_t* q = row + 4 * (x >> 1);
        Y = gld(q + ((x & 1) ? 3 : 1)); U = gld(q); V = gld(q + 2);
    }
    r0 = (float)(Y >> S.yuv_shift); r1 = (float)(U >> S.yuv_shift); r2 = (float)(V >> S.yuv_shift);
    if (S.yuv_shift) yuv_to_rgb_10bit(S.yuv_kind, r0, r1, r2);
    else yuv_to_rgb(S.yuv_kind, r0, r1, r2);
}

__device__ __forceinline__ void read_tap_any(const DevSeq& S, const DevPlane& P, int a, int b, float& r0, float& r1,
                                             float& r2) {
    if (S.src_format == FKB_SRC_U8X3) read_tap<FKB_SRC_U8X3>(P, a, b, r0, r1, r2);
    else if (S.src_format == FKB_SRC_F32X3) read_tap<FKB_SRC_F32X3>(P, a, b, r0, r1, r2);
    else if (S.src_format >= FKB_SRC_P010) read_converted_yuv(S, P, a + P.crop_x, b + P.crop_y, r0, r1, r2);
    else read_tap<FKB_SRC_NV12>(P, a, b, r0, r1, r2, S.swap_uv != 0);
}

/* Bilinear geometry of one output coordinate: Resize::exec_resize (resize.h:183-194) and
 * Interpolate<INTER_LINEAR>::exec (interpolation.h:61-96, device branch :66-67). */
struct Axis {
    int i0, i1;   /* first tap, second tap clamped to the last source index (:76-77) */
    float w0, w1; /* (i0 + 1) - s and s - i0: weights use the UNCLAMPED second index (:92-95) */
};
__device__ __forceinline__ Axis make_axis(int r, float f, int src_extent) {
    Axis ax;
    const float s = __fmul_rn((float)r, f);
    ax.i0 = __float2int_rd(s);
    ax.i1 = min(ax.i0 + 1, src_extent - 1);
    ax.w0 = __fsub_rn((float)(ax.i0 + 1), s);
    ax.w1 = __fsub_rn(s, (float)ax.i0);
    return ax;
}

/* The first tap index alone: floor of the binary32 product (resize.h:183-194, interpolation.h:66-67). */
__device__ __forceinline__ int axis_first(int r, float f) { return __float2int_rd(__fmul_rn((float)r, f)); }

/* ((p00*w00 + p10*w10) + p01*w01) + p11*w11, products and sums rounded separately. */
__device__ __forceinline__ float blend(float p00, float p10, float p01, float p11, float w00, float w10, float w01,
                                       float w11) {
    return __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(p00, w00), __fmul_rn(p10, w10)), __fmul_rn(p01, w01)),
                     __fmul_rn(p11, w11));
}

/* ------------------------------------------------------------------------------------ */
/* body: generic, one output pixel per thread                                           */
/* ------------------------------------------------------------------------------------ */
/* BorderReader's index maps (border_reader.h:163-273): idx_low(idx_high(i)), for an axis of n elements. */
__device__ __forceinline__ int border_index(int mode, int i, int n) {
    const int last = n - 1;
    switch (mode) {
        case FKB_BORDER_REPLICATE: return max(min(i, last), 0);
        case FKB_BORDER_REFLECT: {
            const int v = last - abs(last - i) + (i > last ? 1 : 0);
            return (abs(v) - (v < 0 ? 1 : 0)) % n;
        }
        case FKB_BORDER_WRAP: {
            const int v = i < n ? i : i % n;
            return v >= 0 ? v : v - ((v - n + 1) / n) * n;
        }
        case FKB_BORDER_REFLECT_101: {
            const int v = abs(last - abs(last - i)) % n;
            return abs(v) % n;
        }
        default: return i;
    }
}

/* The source element at image coordinates (x, y), inside the image. */
__device__ __forceinline__ void read_image(const DevSeq& S, const DevPlane& P, int x, int y, float (&r)[3]) {
    if (S.src_format == FKB_SRC_U8X3) {
        const uint8_t* p = P.src + (size_t)y * P.src_pitch + (size_t)x * 3;
        r[0] = u8_to_float(gld(p)); r[1] = u8_to_float(gld(p + 1)); r[2] = u8_to_float(gld(p + 2));
    } else {
        const float* p = reinterpret_cast<const float*>(P.src + (size_t)y * P.src_pitch + (size_t)x * 12);
        r[0] = gld(p); r[1] = gld(p + 1); r[2] = gld(p + 2);
    }
}

/* The read chain of the one-pixel-per-thread body at crop-relative (a, b): PerThreadRead, then BorderReader or
 * Deinterlace if the sequence has one, then Crop (crop.h:35-38 adds the rect origin on the way down). */
__device__ __forceinline__ void fetch_generic(const DevSeq& S, const DevPlane& P, int a, int b, float (&r)[3]) {
    if (S.border_mode == FKB_BORDER_NONE && S.deinterlace == FKB_DEINTERLACE_NONE) {
        read_tap_any(S, P, a, b, r[0], r[1], r[2]);
        return;
    }
    const int x = a + P.crop_x, y = b + P.crop_y, w = (int)P.gw, h = (int)P.src_height;
    if (S.border_mode != FKB_BORDER_NONE) {
        if (S.border_mode == FKB_BORDER_CONSTANT) { /* border_reader.h:140-148 */
            if (x >= 0 && x < w && y >= 0 && y < h) read_image(S, P, x, y, r);
            else { r[0] = S.border_value[0]; r[1] = S.border_value[1]; r[2] = S.border_value[2]; }
        } else {
            read_image(S, P, border_index(S.border_mode, x, w), border_index(S.border_mode, y, h), r);
        }
        return;
    }
    /* Deinterlace (deinterlace.h:91-131): the row, or the mean of two rows with the reference's +1: for uchar3 the sum
       is an integer sum (exact in binary32), for float3 two rounded additions; then * 0.5f */
    const bool blend_mode = S.deinterlace == FKB_DEINTERLACE_BLEND;
    bool two;
    int ya, yb;
    if (blend_mode) { two = y > 0; ya = y; yb = y - 1; }
    else {
        const bool even = (y & 1) == 0;
        two = S.deinterlace == FKB_DEINTERLACE_LINEAR_EVEN ? (!even && y != h - 1) : (even && y != 0);
        ya = y - 1; yb = y + 1;
    }
    if (!two) { read_image(S, P, x, y, r); return; }
    float p[3], q[3];
    read_image(S, P, x, ya, p);
    read_image(S, P, x, yb, q);
#pragma unroll
    for (int c = 0; c < 3; ++c) r[c] = __fmul_rn(__fadd_rn(__fadd_rn(p[c], q[c]), 1.0f), 0.5f);
}

/* Bilinear geometry at a source coordinate that is already known (Warping, warping.h:89-92 -> interpolation.h:61-96). */
__device__ __forceinline__ Axis make_axis_at(float s, int src_extent) {
    Axis ax;
    ax.i0 = __float2int_rd(s);
    ax.i1 = min(ax.i0 + 1, src_extent - 1);
    ax.w0 = __fsub_rn((float)(ax.i0 + 1), s);
    ax.w1 = __fsub_rn(s, (float)ax.i0);
    return ax;
}

__device__ __forceinline__ void body_generic(const DevPlane& P, const DevSeq& S, const OpSlot* sops, uint32_t local) {
    const uint32_t idx = local * ITEM_PIXELS_GENERIC + threadIdx.x;
    if (idx >= P.dst_w * P.dst_h) return;
    const int y = idx / P.dst_w, x = idx - y * P.dst_w;
    const float2 one = dup2(S.one);
    float v[3];
    int first_post = 0;
    /* a plane whose region is empty (a default-value plane, batch_operations.h:236-241) has no geometry stage either way */
    if (S.resize_mode == FKB_RESIZE_NONE && P.x2 >= P.x1) {
        fetch_generic(S, P, x, y, v);
    } else {
        first_post = S.n_pre;
        const bool warp = S.resize_mode == FKB_GEOMETRY_WARP_AFFINE || S.resize_mode == FKB_GEOMETRY_WARP_PERSPECTIVE;
        bool inside;
        Axis ax, ay;
        if (warp) {
            /* WarpingCoords (warping.h:49-69): every product and sum rounded, int coordinates converted to float */
            const float* m = S.transform;
            const float fx = (float)x, fy = (float)y;
            float cx = __fadd_rn(__fadd_rn(__fmul_rn(m[0], fx), __fmul_rn(m[1], fy)), m[2]);
            float cy = __fadd_rn(__fadd_rn(__fmul_rn(m[3], fx), __fmul_rn(m[4], fy)), m[5]);
            if (S.resize_mode == FKB_GEOMETRY_WARP_PERSPECTIVE) {
                const float coeff = __fdiv_rn(1.0f, __fadd_rn(__fadd_rn(__fmul_rn(m[6], fx), __fmul_rn(m[7], fy)), m[8]));
                cx = __fmul_rn(coeff, cx);
                cy = __fmul_rn(coeff, cy);
            }
            inside = cx >= 0.0f && cx < (float)P.crop_w && cy >= 0.0f && cy < (float)P.crop_h; /* warping.h:89 */
            ax = make_axis_at(inside ? cx : 0.0f, P.crop_w);
            ay = make_axis_at(inside ? cy : 0.0f, P.crop_h);
        } else {
            /* Resize::exec (resize.h:75-87): outside the region of interest return the default */
            inside = x >= P.x1 && x <= P.x2 && y >= P.y1 && y <= P.y2;
            ax = make_axis(inside ? x - P.x1 : 0, P.fx, P.crop_w);
            ay = make_axis(inside ? y - P.y1 : 0, P.fy, P.crop_h);
        }
        if (!inside) {
            if (warp) { v[0] = 0.0f; v[1] = 0.0f; v[2] = 0.0f; } /* warping.h:92 */
            else { v[0] = S.bg[0]; v[1] = S.bg[1]; v[2] = S.bg[2]; }
        } else {
            float t[4][3];
            fetch_generic(S, P, ax.i0, ay.i0, t[0]);
            fetch_generic(S, P, ax.i1, ay.i0, t[1]);
            fetch_generic(S, P, ax.i0, ay.i1, t[2]);
            fetch_generic(S, P, ax.i1, ay.i1, t[3]);
            if (S.pre_kind != PRE_IDENTITY && S.n_pre > 0) {
#pragma unroll
                for (int k = 0; k < 4; ++k) run_ops_1<CHAIN_INTERPRET>(t[k], sops, 0, S.n_pre, one);
            }
            const float w00 = __fmul_rn(ax.w0, ay.w0), w10 = __fmul_rn(ax.w1, ay.w0);
            const float w01 = __fmul_rn(ax.w0, ay.w1), w11 = __fmul_rn(ax.w1, ay.w1);
#pragma unroll
            for (int c = 0; c < 3; ++c) v[c] = blend(t[0][c], t[1][c], t[2][c], t[3][c], w00, w10, w01, w11);
        }
    }
    run_ops_1<CHAIN_INTERPRET>(v, sops, first_post, S.n_ops, one);
    /* receivers: memory_operations.h:122-127 (PerThreadWrite), :181-184 (TensorWrite),
       :203-219 (TensorSplit) */
    if (S.dst_format == FKB_DST_F32X3_PACKED) {
        float* p = reinterpret_cast<float*>(P.dst + (size_t)y * P.dst_pitch + (size_t)x * 12);
        gst(p, v[0]); gst(p + 1, v[1]); gst(p + 2, v[2]);
    } else if (S.dst_format == FKB_DST_F32_PLANAR3) {
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            gst(reinterpret_cast<float*>(P.dst + (size_t)c * P.dst_cstride + (size_t)y * P.dst_pitch + (size_t)x * 4), v[c]);
        }
    } else {
        uint8_t* p = P.dst + (size_t)y * P.dst_pitch + (size_t)x * 3;
        gst(p, (uint8_t)v[0]); gst(p + 1, (uint8_t)v[1]); gst(p + 2, (uint8_t)v[2]);
    }
}

/* ------------------------------------------------------------------------------------ */
/* body: no geometry stage, four whole pixels per thread                                */
/* ------------------------------------------------------------------------------------ */
/* n / d for d > 0 and a quotient below 2^22 (row, slot and tile indices): the quotient of the two numbers as floats is off by
   at most one, which the remainder tells; ten instructions where the integer division takes three times as many, in a
   block's prologue that runs once per few thousand pixels. */
__device__ __forceinline__ uint32_t div_small(uint32_t n, uint32_t d) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(__uint2float_rn(d)));
    uint32_t q = __float2uint_rz(__fmul_rn(__uint2float_rn(n), r));
    const int32_t rem = (int32_t)(n - q * d);
    if (rem < 0) --q;
    else if ((uint32_t)rem >= d) ++q;
    return q;
}

template <uint32_t CHAIN, bool SRC_IS_U8, bool DST_IS_U8>
__device__ __forceinline__ void body_flat(const DevPlane& P, const DevSeq& S, const OpSlot* sops, uint32_t local,
                                          unsigned char* turn_mem, uint32_t prefetch_items = 0) {
    constexpr int SPX = SRC_IS_U8 ? 3 : 12;
    constexpr int DPX = DST_IS_U8 ? 3 : 12;
    constexpr int Q = flat_quads(SRC_IS_U8);
    constexpr int RAW = SRC_IS_U8 ? 3 : 12; /* words of a run of four pixels as it lies in memory */
    constexpr uint32_t ITEM = (uint32_t)flat_item_pixels(SRC_IS_U8);
    /* A work item is Q runs of 4 * blockDim pixels of one segment; a thread owns four consecutive
       pixels of each run, so that a warp reads and writes whole 128-byte lines.  The raw words of
       all runs are loaded before the first run is computed: the block's start-up (two dependent
       descriptor reads) is paid once for Q times the data, with Q loads in flight per thread. */
    const uint32_t items_per_seg = (P.seg_pixels + ITEM - 1) / ITEM;
    const uint32_t seg = local / items_per_seg;
    const uint32_t base = (local - seg * items_per_seg) * ITEM + threadIdx.x * PX_PER_THREAD;
    const uint8_t* const src_seg = P.src + (size_t)(P.crop_y + seg) * P.src_pitch + (size_t)P.crop_x * SPX;
    uint8_t* const dst_seg = P.dst + (size_t)seg * P.dst_pitch;

    /* A chain of tens of operations per value: a block computes far longer than it loads, and with one resident block in
       five loading at any time an SM has a few KB in flight where the memory needs tens (a 4K float3 image through 64
       operations took 68 us against 36 us for its bytes and 43 us for its arithmetic, nearly their sum).  The block
       therefore asks the L2 for the bytes of the work item `prefetch_items` ahead, one bulk prefetch by one thread:
       the memory then works at the rate at which blocks start, whatever they are doing, and a block's own loads
       find their lines in the L2.  Dense planes only (one segment). */
    if (!SRC_IS_U8 && prefetch_items != 0 && threadIdx.x == 0 && P.n_segs == 1u) {
        const uint64_t px_ahead = ((uint64_t)local + prefetch_items) * ITEM;
        if (px_ahead < P.seg_pixels) {
            const uint32_t bytes = (uint32_t)min((uint64_t)ITEM, P.seg_pixels - px_ahead) * SPX & ~15u;
            if (bytes != 0)
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_seg + px_ahead * SPX), "r"(bytes) : "memory");
        }
    }

    /* Output of one run, warp by warp: a thread's four pixels are 48 (12) bytes, so stores straight
       from the registers would write a third of every sector per instruction, and that pattern was
       measured at 5.0 TB/s against 6.4 TB/s for whole lines.  The warp therefore turns its 128
       pixels around in shared memory and every store instruction writes consecutive bytes. */
    using OutWord = typename std::conditional<DST_IS_U8, uint32_t, float4>::type;
    const uint32_t lane = threadIdx.x & 31u;
    OutWord* const my_turn = reinterpret_cast<OutWord*>(turn_mem) + (threadIdx.x >> 5) * 96u;

    uint32_t raw[Q][RAW];
    uint32_t n[Q];
    bool whole_warp[Q]; /* every thread of the warp has a full run: uniform across the warp */
#pragma unroll
    for (int r = 0; r < Q; ++r) {
        const uint32_t px0 = base + r * (BLOCK_THREADS * PX_PER_THREAD);
        n[r] = px0 < P.seg_pixels ? min((uint32_t)PX_PER_THREAD, P.seg_pixels - px0) : 0u;
        whole_warp[r] = px0 - lane * PX_PER_THREAD + 32u * PX_PER_THREAD <= P.seg_pixels;
        const uint8_t* src = src_seg + (size_t)px0 * SPX;
        if (n[r] == PX_PER_THREAD) {
            if constexpr (SRC_IS_U8) {
                const uint32_t* s4 = reinterpret_cast<const uint32_t*>(src);
#pragma unroll
                for (int k = 0; k < 3; ++k) raw[r][k] = gld(s4 + k);
            } else {
                const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    const uint4 w = gld(s4 + k);
                    raw[r][4 * k + 0] = w.x; raw[r][4 * k + 1] = w.y; raw[r][4 * k + 2] = w.z; raw[r][4 * k + 3] = w.w;
                }
            }
        } else {
            /* the ragged end of a segment, element by element into the same layout */
#pragma unroll
            for (int k = 0; k < RAW; ++k) raw[r][k] = 0u;
#pragma unroll
            for (int i = 0; i < 12; ++i) {
                if (i < (int)n[r] * 3) {
                    if constexpr (SRC_IS_U8) raw[r][i / 4] |= (uint32_t)gld(src + i) << (8 * (i % 4));
                    else raw[r][i] = gld(reinterpret_cast<const uint32_t*>(src) + i);
                }
            }
        }
    }

    const float2 one2 = dup2(S.one);
#pragma unroll
    for (int r = 0; r < Q; ++r) {
        if (n[r] == 0) break;
        float v[12];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            if constexpr (SRC_IS_U8) {
                v[4 * k + 0] = packed_u8_to_float<0>(raw[r][k]);
                v[4 * k + 1] = packed_u8_to_float<1>(raw[r][k]);
                v[4 * k + 2] = packed_u8_to_float<2>(raw[r][k]);
                v[4 * k + 3] = packed_u8_to_float<3>(raw[r][k]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[4 * k + j] = __uint_as_float(raw[r][4 * k + j]);
            }
        }
        /* pair pixels (0,1) and (2,3) channel by channel */
        float2 q[6];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < 3; ++c) q[3 * j + c] = make_float2(v[6 * j + c], v[6 * j + 3 + c]);
        constexpr bool BIASED = DST_IS_U8 && chain_ends_biased(CHAIN); /* v = 2^23 + byte from here on */
        run_ops<CHAIN, 2, BIASED>(q, sops, 0, S.n_ops, one2);
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < 3; ++c) { v[6 * j + c] = q[3 * j + c].x; v[6 * j + 3 + c] = q[3 * j + c].y; }

        const uint32_t px0 = base + r * (BLOCK_THREADS * PX_PER_THREAD);
        uint8_t* dst = dst_seg + (size_t)px0 * DPX;
        if (n[r] == PX_PER_THREAD) {
            OutWord w[3];
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                if constexpr (DST_IS_U8) {
                    /* The values are whole numbers 0..255 (bytes that were never touched, or SaturateCast's result):
                       2^23 + v is exact and carries v in its lowest byte, so four additions and three byte permutes
                       pack the word without four trips through the quarter-rate conversion unit. */
                    const float bias = BIASED ? 0.0f : 8388608.0f; /* a chain that ends in SaturateCast left its bytes there already */
                    const uint32_t b0 = __float_as_uint(BIASED ? v[4 * k + 0] : __fadd_rn(v[4 * k + 0], bias)), b1 = __float_as_uint(BIASED ? v[4 * k + 1] : __fadd_rn(v[4 * k + 1], bias));
                    const uint32_t b2 = __float_as_uint(BIASED ? v[4 * k + 2] : __fadd_rn(v[4 * k + 2], bias)), b3 = __float_as_uint(BIASED ? v[4 * k + 3] : __fadd_rn(v[4 * k + 3], bias));
                    w[k] = __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
                } else {
                    w[k] = make_float4(v[4 * k + 0], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
                }
            }
            if (whole_warp[r]) {
#pragma unroll
                for (int k = 0; k < 3; ++k) my_turn[lane * 3 + k] = w[k];
                __syncwarp();
                OutWord* const warp_dst = reinterpret_cast<OutWord*>(dst) - lane * 3;
#pragma unroll
                for (int k = 0; k < 3; ++k) gst(warp_dst + (k * 32 + lane), my_turn[k * 32 + lane]);
                __syncwarp();
            } else {
                OutWord* d4 = reinterpret_cast<OutWord*>(dst);
#pragma unroll
                for (int k = 0; k < 3; ++k) gst(d4 + k, w[k]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 12; ++i) {
                if (i < (int)n[r] * 3) {
                    if (DST_IS_U8) gst(dst + i, BIASED ? (uint8_t)(__float_as_uint(v[i]) & 0xFFu) : (uint8_t)v[i]);
                    else gst(reinterpret_cast<float*>(dst) + i, v[i]);
                }
            }
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* body: bilinear resize                                                                */
/* ------------------------------------------------------------------------------------ */

/* Position idx of a row-major walk over rows of `per_row` cells, advanced `step` cells at a time
   with one division at the start instead of one per step. */
struct CellWalk {
    uint32_t r, c, dr, dc, per_row;
    /* `more`: whether any walker will advance at all (uniform); the step's division is skipped if not */
    __device__ __forceinline__ CellWalk(uint32_t idx, uint32_t step, uint32_t per_row_, bool more = true) : per_row(per_row_) {
        r = div_small(idx, per_row); c = idx - r * per_row;
        dr = 0; dc = 0;
        if (more) { dr = div_small(step, per_row); dc = step - dr * per_row; }
    }
    __device__ __forceinline__ void advance() {
        r += dr; c += dc;
        if (c >= per_row) { c -= per_row; ++r; }
    }
};

/* Stores one group of four output pixels (v[3*i + channel]) at column x0 of row y. */
template <bool PLANAR>
__device__ __forceinline__ void store_group(uint8_t* dst, uint32_t pitch, uint32_t cstride, int x0, int y,
                                            const float (&v)[12]) {
    if (PLANAR) {
        uint8_t* d = dst + (size_t)y * pitch + (size_t)x0 * 4;
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            gst(reinterpret_cast<float4*>(d + (size_t)c * cstride), make_float4(v[c], v[3 + c], v[6 + c], v[9 + c]));
        }
    } else {
        float4* d = reinterpret_cast<float4*>(dst + (size_t)y * pitch + (size_t)x0 * 12);
#pragma unroll
        for (int k = 0; k < 3; ++k) gst(d + k, make_float4(v[4 * k + 0], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]));
    }
}

/* Stores one output pixel (three channels) at column x of row y. */
template <bool PLANAR>
__device__ __forceinline__ void store_pixel(uint8_t* dst, uint32_t pitch, uint32_t cstride, int x, int y, float a,
                                            float b, float c) {
    if (PLANAR) {
        uint8_t* d = dst + (size_t)y * pitch + (size_t)x * 4;
        gst(reinterpret_cast<float*>(d), a);
        gst(reinterpret_cast<float*>(d + (size_t)cstride), b);
        gst(reinterpret_cast<float*>(d + 2 * (size_t)cstride), c);
    } else {
        float* d = reinterpret_cast<float*>(dst + (size_t)y * pitch + (size_t)x * 12);
        gst(d, a); gst(d + 1, b); gst(d + 2, c);
    }
}

/* The same at an address already computed. */
template <bool PLANAR>
__device__ __forceinline__ void store_pixel_at(uint8_t* d, uint32_t cstride, float a, float b, float c) {
    if (PLANAR) {
        gst(reinterpret_cast<float*>(d), a);
        gst(reinterpret_cast<float*>(d + (size_t)cstride), b);
        gst(reinterpret_cast<float*>(d + 2 * (size_t)cstride), c);
    } else {
        float* f = reinterpret_cast<float*>(d);
        gst(f, a); gst(f + 1, b); gst(f + 2, c);
    }
}

/* Default value over cells of the output, a walk of `step` threads starting at cell `first`.  A planar cell is a group
 * of four pixels (one 16-byte word in each channel plane); a packed cell is one of the group's three 16-byte words, so
 * that the words a warp stores with one instruction lie side by side (a thread that stores the three words of its own
 * four pixels leaves every 32-byte sector to two instructions: 3.8 against 6.7 TB/s on a batch of nothing but default
 * planes).  Rows are `groups_per_row` groups long after `skip_groups` groups from group `skip_lo` on have been left
 * out (the region of interest); row_of(r) is the output row of the walk's r-th row.  `groups` bounds a thread's share,
 * counted in groups. */
template <bool PLANAR, typename RowOf>
__device__ __forceinline__ void fill_cells(uint8_t* dst, uint32_t pitch, uint32_t cstride, uint32_t first_group, uint32_t lane_in_walk,
                                           uint32_t step, uint32_t groups, uint32_t rows, uint32_t groups_per_row, uint32_t skip_lo,
                                           uint32_t skip_groups, const float (&bg)[3], RowOf row_of) {
    constexpr uint32_t UNITS = PLANAR ? 1u : 3u;
    const uint32_t per_row = groups_per_row * UNITS, total = rows * per_row, lo = skip_lo * UNITS, skip = skip_groups * UNITS;
    uint32_t idx = first_group * UNITS + lane_in_walk;
    const uint32_t iters = groups * UNITS;
    CellWalk w(idx, step, per_row, total > step);
#pragma unroll 1
    for (uint32_t k = 0; k < iters && idx < total; ++k, idx += step, w.advance()) {
        const uint32_t c = w.c < lo ? w.c : w.c + skip;
        uint8_t* const d = dst + (size_t)row_of(w.r) * pitch + (size_t)c * 16u;
        if (PLANAR) {
#pragma unroll
            for (int ch = 0; ch < 3; ++ch) gst(reinterpret_cast<float4*>(d + (size_t)ch * cstride), make_float4(bg[ch], bg[ch], bg[ch], bg[ch]));
        } else { /* word c of a row holds the channels (c, c+1, c+2, c) mod 3 */
            const uint32_t k3 = c % 3u;
            const float a = k3 == 0 ? bg[0] : k3 == 1 ? bg[1] : bg[2];
            const float b = k3 == 0 ? bg[1] : k3 == 1 ? bg[2] : bg[0];
            const float e = k3 == 0 ? bg[2] : k3 == 1 ? bg[0] : bg[1];
            gst(reinterpret_cast<float4*>(d), make_float4(a, b, e, a));
        }
    }
}

/* Default value over every row outside the region's rows, for a plane whose rows lie side by side in memory (pitch =
 * row bytes): the cells above and below the region are two runs of 16-byte words, walked by the whole block without any
 * row or column arithmetic.  A packed row is a multiple of three words long, so the channels of a word follow from its
 * index in the walk: (k, k+1, k+2, k) mod 3. */
template <bool PLANAR>
__device__ __forceinline__ void fill_outside_rows_dense(uint8_t* dst, uint32_t cstride, uint32_t words_per_row, uint32_t rows_above,
                                                        uint32_t region_rows, uint32_t rows_total, const float (&bg)[3]) {
    const uint32_t top = rows_above * words_per_row, skip = region_rows * words_per_row, total = (rows_total - region_rows) * words_per_row;
    if (PLANAR) {
        const uint32_t step = blockDim.x;
#pragma unroll 1
        for (uint32_t idx = threadIdx.x; idx < total; idx += step) {
            uint8_t* const d = dst + (size_t)(idx < top ? idx : idx + skip) * 16u;
#pragma unroll
            for (int ch = 0; ch < 3; ++ch) gst(reinterpret_cast<float4*>(d + (size_t)ch * cstride), make_float4(bg[ch], bg[ch], bg[ch], bg[ch]));
        }
    } else {
        /* The walk's step is the largest multiple of three threads (the one or two threads beyond it sit out), so that all
           words of a thread hold the same channels and the loop is a store and its address: with a few words per thread,
           what surrounds the loop counts as much as the loop. */
        const uint32_t step = blockDim.x - blockDim.x % 3u;
        if (threadIdx.x < step) {
            const uint32_t k3 = threadIdx.x % 3u;
            const float4 word = make_float4(k3 == 0 ? bg[0] : k3 == 1 ? bg[1] : bg[2], k3 == 0 ? bg[1] : k3 == 1 ? bg[2] : bg[0],
                                            k3 == 0 ? bg[2] : k3 == 1 ? bg[0] : bg[1], k3 == 0 ? bg[0] : k3 == 1 ? bg[1] : bg[2]);
#pragma unroll 1
            for (uint32_t idx = threadIdx.x; idx < total; idx += step)
                gst(reinterpret_cast<float4*>(dst + (size_t)(idx < top ? idx : idx + skip) * 16u), word);
        }
    }
}

template <uint32_t CHAIN, int SRC, bool PLANAR>
__device__ __forceinline__ void body_resize(const DevPlane& P, const DevSeq& S, const OpSlot* sops, uint32_t local) {
    /* plane fields used inside loops, copied out of shared memory once */
    uint8_t* const dst = P.dst;
    const uint32_t dst_pitch = P.dst_pitch, dst_cstride = P.dst_cstride, src_pitch = P.src_pitch;
    const uint32_t groups_per_row = P.dst_w / PX_PER_THREAD;
    const int x1 = P.x1, y1 = P.y1, x2 = P.x2, y2 = P.y2;
    const uint32_t g_lo = (uint32_t)x1 / PX_PER_THREAD;
    const uint32_t n_groups = (uint32_t)x2 / PX_PER_THREAD - g_lo + 1;
    const uint32_t n_rows = (uint32_t)(y2 - y1 + 1);
    const uint32_t nthreads = blockDim.x;

    /* The value every output element outside the region of interest ends up with: the
       default value run through the continuation (resize.h:84-86). */
    /* what every output element outside the region of interest ends up with: the default value
       after the continuation (resize.h:84-86), evaluated once when the plan was made */
    const float bgv[3] = {S.bg_out[0], S.bg_out[1], S.bg_out[2]};
    const float2 one = dup2(S.one);

    if (local >= P.roi_items) {
        /* store-only item: rows above and below the region of interest */
        fill_cells<PLANAR>(dst, dst_pitch, dst_cstride, (local - P.roi_items) * (nthreads * BG_GROUPS_PER_THREAD), threadIdx.x, nthreads,
                           BG_GROUPS_PER_THREAD, P.dst_h - n_rows, groups_per_row, 0u, 0u, bgv,
                           [&](uint32_t r) { return (int)r < y1 ? r : r + n_rows; });
        return;
    }

    const uint32_t tiles_x = P.tiles_x, gw = P.gw, rs = P.rs;
    const uint32_t tile_y = div_small(local, tiles_x), tile_x = local - tile_y * tiles_x;
    const uint32_t slot = div_small(threadIdx.x, gw), gi = threadIdx.x - slot * gw;
    const int row0 = y1 + (int)(tile_y * rs * RESIZE_ROWS_PER_THREAD); /* first row of this tile */

    if (slot < rs) {
        /* The thread's four columns are gw apart, so that neighbouring lanes read neighbouring
           source pixels and write neighbouring output elements: a warp-wide byte load then touches
           a few hundred contiguous bytes instead of a span four times as wide. */
        const int x0 = (int)(g_lo * PX_PER_THREAD + tile_x * gw * RESIZE_PX + gi);
        const int x_end = (int)(g_lo * PX_PER_THREAD + min(n_groups * PX_PER_THREAD, (tile_x + 1) * gw * RESIZE_PX));
        /* horizontal taps and weights of the thread's columns, once per thread; columns 2j and
           2j+1 travel as one pair */
        constexpr int NPAIR = RESIZE_PX / 2;
        uint32_t off0[RESIZE_PX], off1[RESIZE_PX]; /* U8X3: byte offsets in a source row; NV12: columns */
        float2 wx0[NPAIR], wx1[NPAIR];
        uint32_t inside = 0, valid = 0;
#pragma unroll
        for (int i = 0; i < RESIZE_PX; ++i) {
            const int x = x0 + i * (int)gw;
            const bool in = (x >= x1 && x <= x2);
            valid |= (x < x_end ? 1u : 0u) << i;
            const Axis ax = make_axis(in ? x - x1 : 0, P.fx, P.crop_w);
            if (SRC == FKB_SRC_NV12) { off0[i] = (uint32_t)(ax.i0 + P.crop_x); off1[i] = (uint32_t)(ax.i1 + P.crop_x); }
            else { off0[i] = (uint32_t)ax.i0 * 3u; off1[i] = (uint32_t)ax.i1 * 3u; }
            if (i & 1) { wx0[i / 2].y = ax.w0; wx1[i / 2].y = ax.w1; }
            else { wx0[i / 2].x = ax.w0; wx1[i / 2].x = ax.w1; }
            inside |= (in ? 1u : 0u) << i;
        }
        const float fy = P.fy;
        const int crop_h = P.crop_h, crop_y = P.crop_y;
        const uint8_t* const src0 = SRC == FKB_SRC_NV12 ? P.src : P.src + (size_t)crop_y * src_pitch + (size_t)P.crop_x * 3;
        const uint8_t* const chroma0 = P.src + (size_t)src_pitch * P.src_height;
        const int yuv = S.pre_kind; /* PRE_IDENTITY: no conversion */
        const uint32_t u_at = S.swap_uv ? 1u : 0u, v_at = 1u - u_at; /* NV21: the pair is V,U */

#pragma unroll 1
        for (int j = 0; j < RESIZE_ROWS_PER_THREAD; ++j) {
            const int y = row0 + (int)slot + j * (int)rs;
            if (y > y2) break;
            const Axis ay = make_axis(y - y1, fy, crop_h);
            float2 v[3 * NPAIR];
            if (SRC == FKB_SRC_U8X3) {
                const uint8_t* const r0 = src0 + (size_t)ay.i0 * src_pitch;
                const uint8_t* const r1 = src0 + (size_t)ay.i1 * src_pitch;
                const float2 wy0 = dup2(ay.w0), wy1 = dup2(ay.w1);
#pragma unroll
                for (int k = 0; k < NPAIR; ++k) {
                    const uint8_t* a00 = r0 + off0[2 * k]; const uint8_t* a10 = r0 + off1[2 * k];
                    const uint8_t* a01 = r1 + off0[2 * k]; const uint8_t* a11 = r1 + off1[2 * k];
                    const uint8_t* b00 = r0 + off0[2 * k + 1]; const uint8_t* b10 = r0 + off1[2 * k + 1];
                    const uint8_t* b01 = r1 + off0[2 * k + 1]; const uint8_t* b11 = r1 + off1[2 * k + 1];
                    const float2 w00 = mul2(wx0[k], wy0), w10 = mul2(wx1[k], wy0);
                    const float2 w01 = mul2(wx0[k], wy1), w11 = mul2(wx1[k], wy1);
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const float2 p00 = make_float2(u8_to_float(gld(a00 + c)), u8_to_float(gld(b00 + c)));
                        const float2 p10 = make_float2(u8_to_float(gld(a10 + c)), u8_to_float(gld(b10 + c)));
                        const float2 p01 = make_float2(u8_to_float(gld(a01 + c)), u8_to_float(gld(b01 + c)));
                        const float2 p11 = make_float2(u8_to_float(gld(a11 + c)), u8_to_float(gld(b11 + c)));
                        /* ((p00*w00 + p10*w10) + p01*w01) + p11*w11, every product and sum rounded */
                        v[3 * k + c] = add2(add2(add2(mul2(p00, w00), mul2(p10, w10), one), mul2(p01, w01), one), mul2(p11, w11), one);
                    }
                }
            } else {
                /* NV12: luma at (x, y), chroma pair at (x>>1, y>>1) (color_conversion.h:329-346).  A tap
                   whose weight is exactly zero contributes +-0 to the sum and is not fetched: the first
                   term is never -0 here, so the sum is unchanged bit for bit. */
                const int ya0 = ay.i0 + crop_y, ya1 = ay.i1 + crop_y;
                const uint8_t* const l0 = src0 + (size_t)ya0 * src_pitch;
                const uint8_t* const l1 = src0 + (size_t)ya1 * src_pitch;
                const uint8_t* const c0 = chroma0 + (size_t)(ya0 >> 1) * src_pitch;
                const uint8_t* const c1 = chroma0 + (size_t)(ya1 >> 1) * src_pitch;
                const bool need_row1 = ay.w1 != 0.0f;
#pragma unroll
                for (int i = 0; i < RESIZE_PX; ++i) {
                    const float wxa = (i & 1) ? wx0[i / 2].y : wx0[i / 2].x;
                    const float wxb = (i & 1) ? wx1[i / 2].y : wx1[i / 2].x;
                    const bool need_col1 = wxb != 0.0f;
                    const uint32_t xa = off0[i], xb = off1[i];
                    const uint32_t ca = (xa >> 1) * 2u, cb = (xb >> 1) * 2u;
                    float t[3];
                    t[0] = u8_to_float(gld(l0 + xa)); t[1] = u8_to_float(gld(c0 + ca + u_at)); t[2] = u8_to_float(gld(c0 + ca + v_at));
                    yuv_to_rgb(yuv, t[0], t[1], t[2]);
                    const float w00 = __fmul_rn(wxa, ay.w0);
                    float acc[3] = {__fmul_rn(t[0], w00), __fmul_rn(t[1], w00), __fmul_rn(t[2], w00)};
                    if (need_col1) {
                        t[0] = u8_to_float(gld(l0 + xb)); t[1] = u8_to_float(gld(c0 + cb + u_at)); t[2] = u8_to_float(gld(c0 + cb + v_at));
                        yuv_to_rgb(yuv, t[0], t[1], t[2]);
                        const float w10 = __fmul_rn(wxb, ay.w0);
#pragma unroll
                        for (int c = 0; c < 3; ++c) acc[c] = __fadd_rn(acc[c], __fmul_rn(t[c], w10));
                    }
                    if (need_row1) {
                        t[0] = u8_to_float(gld(l1 + xa)); t[1] = u8_to_float(gld(c1 + ca + u_at)); t[2] = u8_to_float(gld(c1 + ca + v_at));
                        yuv_to_rgb(yuv, t[0], t[1], t[2]);
                        const float w01 = __fmul_rn(wxa, ay.w1);
#pragma unroll
                        for (int c = 0; c < 3; ++c) acc[c] = __fadd_rn(acc[c], __fmul_rn(t[c], w01));
                        if (need_col1) {
                            t[0] = u8_to_float(gld(l1 + xb)); t[1] = u8_to_float(gld(c1 + cb + u_at)); t[2] = u8_to_float(gld(c1 + cb + v_at));
                            yuv_to_rgb(yuv, t[0], t[1], t[2]);
                            const float w11 = __fmul_rn(wxb, ay.w1);
#pragma unroll
                            for (int c = 0; c < 3; ++c) acc[c] = __fadd_rn(acc[c], __fmul_rn(t[c], w11));
                        }
                    }
#pragma unroll
                    for (int c = 0; c < 3; ++c) { if (i & 1) v[3 * (i / 2) + c].y = acc[c]; else v[3 * (i / 2) + c].x = acc[c]; }
                }
            }
            run_ops<CHAIN, NPAIR>(v, sops, S.n_pre, S.n_ops, one);
#pragma unroll
            for (int i = 0; i < RESIZE_PX; ++i) {
                if ((valid >> i) & 1u) {
                    const bool in = (inside >> i) & 1u; /* false: a column group straddling the edge of the region */
                    const float2 a = v[3 * (i / 2)], b = v[3 * (i / 2) + 1], c = v[3 * (i / 2) + 2];
                    store_pixel<PLANAR>(dst, dst_pitch, dst_cstride, x0 + i * (int)gw, y, in ? ((i & 1) ? a.y : a.x) : bgv[0],
                                        in ? ((i & 1) ? b.y : b.x) : bgv[1], in ? ((i & 1) ? c.y : c.x) : bgv[2]);
                }
            }
        }
    }

    /* background to the left and right of this tile's rows (first tile of a row band only) */
    const uint32_t n_band = groups_per_row - n_groups;
    if (tile_x == 0 && n_band != 0) {
        const uint32_t rows_here = min(rs * RESIZE_ROWS_PER_THREAD, (uint32_t)(y2 - row0 + 1));
        fill_cells<PLANAR>(dst, dst_pitch, dst_cstride, 0u, threadIdx.x, nthreads, 0xFFFFFFu, rows_here, n_band, g_lo, n_groups, bgv,
                           [&](uint32_t r) { return (uint32_t)row0 + r; });
    }
}

/* ------------------------------------------------------------------------------------ */
/* body: bilinear resize of uchar3 from a source footprint staged in shared memory      */
/* ------------------------------------------------------------------------------------ */

/* Asynchronous bulk copies (the copy engine that also serves tensor-map TMA) and the mbarrier
 * that counts their bytes.  Kernels are launched without clusters: every copy lands in the shared
 * memory of the block that issued it and nowhere else. */
/* Three consecutive aligned words of shared memory at a 32-bit shared-window address. */
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lds32x3(uint32_t addr, uint32_t& w0, uint32_t& w1, uint32_t& w2) {
    if (!check_smem(addr, 12u)) { w0 = w1 = w2 = 0u; return; }
    asm volatile("ld.shared.b32 %0, [%3];\n\tld.shared.b32 %1, [%3+4];\n\tld.shared.b32 %2, [%3+8];"
                 : "=r"(w0), "=r"(w1), "=r"(w2)
                 : "r"(addr));
}
__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t mbar) {
    /* checked build: a copy that would leave the image or the block's shared memory is not issued; its bytes then never
       arrive, the block's bounded wait runs out and the status word keeps the larger code */
    if (!check_src(src, bytes) || !check_smem(dst, bytes)) return;
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(mbar)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t mbar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(mbar), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
/* Waits for phase `parity` for at most `limit_us` microseconds of the GPU's global timer (each
   try_wait itself suspends the warp for a hardware-defined slice, far below a microsecond
   limit's resolution); false when the time ran out.  The clock is read only once a first
   attempt has failed. */
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity, uint32_t limit_us) {
    if (mbar_try_wait(mbar, parity)) return true;
    const uint64_t t0 = global_timer_ns(), limit = (uint64_t)limit_us * 1000ull;
    do {
        if (mbar_try_wait(mbar, parity)) return true;
    } while (global_timer_ns() - t0 < limit);
    return mbar_try_wait(mbar, parity);
}

/* What a body needs to bound its wait: the plan's status word, the limit, and the test-only
   surplus of expected bytes. */
struct WaitCtl {
    uint32_t* status;
    uint32_t limit_us;
    uint32_t test_extra_bytes;
    uint32_t prefetch_items = 0; /* float3 -> float3 element-wise planes: LaunchArgs::prefetch_items */
    uint32_t nv12_early = 0;     /* staged NV12: the kernel's first two warps have marked, packed and started the band's rows */
};

/* A work item is a band of STAGED rows of one plane's region of interest, all columns.  The rows
 * of the crop that the band's taps touch are copied into shared memory by bulk copies (one per
 * source row, started and sized on 16-byte boundaries), then every thread interpolates a pair
 * of columns `gw` apart down its row slots, reading its twelve tap bytes per pixel from shared
 * memory.  Vertical tap positions and weights are computed once per row of the band. */
template <uint32_t CHAIN, bool PLANAR>
__device__ __forceinline__ void body_resize_staged(const DevPlane& P, const DevSeq& S, const OpSlot* sops, uint32_t local,
                                                   unsigned char* staged_mem, const WaitCtl wc) {
    uint8_t* const dst = P.dst;
    const uint32_t dst_pitch = P.dst_pitch, dst_cstride = P.dst_cstride;
    const uint32_t groups_per_row = P.dst_w / PX_PER_THREAD;
    const int x1 = P.x1, y1 = P.y1, x2 = P.x2, y2 = P.y2;
    const uint32_t g_lo = (uint32_t)x1 / PX_PER_THREAD;
    const uint32_t n_groups = (uint32_t)x2 / PX_PER_THREAD - g_lo + 1;
    const uint32_t n_rows = (uint32_t)(y2 - y1 + 1);
    const uint32_t nthreads = blockDim.x;

    /* what every output element outside the region of interest ends up with: the default value
       after the continuation (resize.h:84-86), evaluated once when the plan was made */
    const float bgv[3] = {S.bg_out[0], S.bg_out[1], S.bg_out[2]};
    const float2 one = dup2(S.one);

    if (local >= P.roi_items) {
        /* store-only item: rows above and below the region of interest */
        fill_cells<PLANAR>(dst, dst_pitch, dst_cstride, (local - P.roi_items) * (nthreads * BG_GROUPS_PER_THREAD), threadIdx.x, nthreads,
                           BG_GROUPS_PER_THREAD, P.dst_h - n_rows, groups_per_row, 0u, 0u, bgv,
                           [&](uint32_t r) { return (int)r < y1 ? r : r + n_rows; });
        return;
    }

    /* shared memory: | mbarrier (16 B) | row table (32 B per row of the band) | staged source rows | */
    uint64_t* const mbar_ptr = reinterpret_cast<uint64_t*>(staged_mem);
    float4* const row_tab = reinterpret_cast<float4*>(staged_mem + 16);
    unsigned char* const stage = staged_mem + STAGED_U8_HEADER_BYTES;
    const uint32_t stage_addr = smem_addr(stage);
    const uint32_t mbar = smem_addr(mbar_ptr);

    const uint32_t band_rows = P.tiles_x, gw = P.gw, rs = P.rs; /* rows per band, threads across, row slots */
    const int ya = y1 + (int)(local * band_rows);
    const int yb = min(ya + (int)band_rows - 1, y2);
    const int crop_h = P.crop_h;
    const float fy = P.fy;

    /* source bytes of one crop row that this plane's region columns touch, widened to 16-byte
       boundaries; col0 > 0 when the plane is a column tile of a wider region */
    const uint32_t col0 = P.seg_pixels;
    const StagedSpan span = staged_span(P.crop_x, P.crop_w, col0, (uint32_t)(x2 - x1 + 1), P.fx);
    const uint32_t phase = span.phase, row_len = span.row_len;

    const int src_first = axis_first(ya - y1, fy);
    if (threadIdx.x <= (uint32_t)(yb - ya)) {
        /* vertical taps of one row of the band: shared-memory addresses of its two source rows, and
           its two weights already duplicated into pairs */
        const Axis ay = make_axis(ya + (int)threadIdx.x - y1, fy, crop_h);
        row_tab[2 * threadIdx.x] = make_float4(__uint_as_float(stage_addr + (uint32_t)(ay.i0 - src_first) * row_len),
                                               __uint_as_float(stage_addr + (uint32_t)(ay.i1 - src_first) * row_len), 0.0f, 0.0f);
        row_tab[2 * threadIdx.x + 1] = make_float4(ay.w0, ay.w0, ay.w1, ay.w1);
    }
    __syncthreads(); /* row table written (the band's copies were started when the block began) */

    /* The thread's two columns and their horizontal taps, while the copies are in flight.  The two
       taps of a column are six consecutive bytes of a staged row (three when the second tap is
       clamped onto the first, interpolation.h:76): they are fetched as the three aligned words
       that hold them, shifted down to byte 0, and each byte is turned into a float by one byte
       permute (2^23 + b) and half of a packed subtraction. */
    const uint32_t slot = div_small(threadIdx.x, gw), gi = threadIdx.x - slot * gw;
    const int xa = (int)(g_lo * PX_PER_THREAD + gi), xb = xa + (int)gw;
    const int x_end = (int)((g_lo + n_groups) * PX_PER_THREAD);
    const bool in_a = xa >= x1 && xa <= x2, in_b = xb >= x1 && xb <= x2;
    const bool valid_b = xb < x_end;
    const Axis axa = make_axis((in_a ? xa - x1 : 0) + (int)col0, P.fx, P.crop_w);
    const Axis axb = make_axis((in_b ? xb - x1 : 0) + (int)col0, P.fx, P.crop_w);
    const uint32_t oa = phase + (uint32_t)(axa.i0 - span.sx0) * 3u, ob = phase + (uint32_t)(axb.i0 - span.sx0) * 3u;
    const uint32_t word_a = oa & ~3u, word_b = ob & ~3u;
    const uint32_t shift_a = (oa & 3u) * 8u, shift_b = (ob & 3u) * 8u;
    const uint32_t second_a = axa.i1 == axa.i0 ? 0x3210u : 0x3543u; /* bytes of the second tap in (u0, u1) */
    const uint32_t second_b = axb.i1 == axb.i0 ? 0x3210u : 0x3543u;
    const float2 wx0 = make_float2(axa.w0, axb.w0), wx1 = make_float2(axa.w1, axb.w1);

    /* Stores that need no source byte: the default value to the left and right of this band's rows and, for a plane
       with few rows outside its region (no store-only items), those rows by its last band.  They go first, while the
       band's copies are in flight (1024 crops into planar 224x224: 158.4 -> 154.6 us; into packed receivers it pays
       since the cells are stored as side-by-side words: 8190 crops into packed 60x60 91.5 -> 90.7 us). */
    auto fill_background = [&]() {
        const uint32_t n_side = groups_per_row - n_groups;
        if (n_side != 0)
            fill_cells<PLANAR>(dst, dst_pitch, dst_cstride, 0u, threadIdx.x, nthreads, 0xFFFFFFu, (uint32_t)(yb - ya + 1), n_side, g_lo, n_groups, bgv,
                               [&](uint32_t r) { return (uint32_t)ya + r; });
        if (P.n_segs != 0 && local == P.roi_items - 1) {
            const uint32_t words_per_row = groups_per_row * (PLANAR ? 1u : 3u);
            if (dst_pitch == words_per_row * 16u)
                fill_outside_rows_dense<PLANAR>(dst, dst_cstride, words_per_row, (uint32_t)y1, n_rows, P.dst_h, bgv);
            else
                fill_cells<PLANAR>(dst, dst_pitch, dst_cstride, 0u, threadIdx.x, nthreads, 0xFFFFFFu, P.dst_h - n_rows, groups_per_row, 0u, 0u, bgv,
                                   [&](uint32_t r) { return (int)r < y1 ? r : r + n_rows; });
        }
    };
    fill_background();

    const bool arrived = mbar_wait_bounded(mbar, 0, wc.limit_us);
    if (!arrived) {
        /* never expected: record it and give the copies one more bounded chance to land before
           this block's shared memory is released */
        atomicExch(wc.status, STATUS_STAGED_WAIT_TIMEOUT);
        (void)mbar_wait_bounded(mbar, 0, wc.limit_us);
        return;
    }

    if (slot < rs) {
        const bool plain = in_a && in_b && valid_b;
        /* running output pointer of column a (channel 0), advanced one round of row slots at a time */
        const size_t px_bytes = PLANAR ? 4 : 12;
        uint8_t* out_a = dst + (size_t)(ya + (int)slot) * dst_pitch + (size_t)xa * px_bytes;
        const size_t b_off = (size_t)gw * px_bytes, row_step = (size_t)rs * dst_pitch;
        const float4* rt = row_tab + 2 * slot;

        /* interpolated value of the thread's two columns in the row described by t[0], t[1] */
        auto interpolate = [&](const float4* t, float2 (&v)[3]) {
            const float4 rows = t[0], wy = t[1];
            const uint32_t row_addr[2] = {__float_as_uint(rows.x), __float_as_uint(rows.y)};
            float2 tap[2][2][3]; /* [source row][first / second tap][channel] = (column a, column b) */
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                uint32_t wa0, wa1, wa2, wb0, wb1, wb2;
                lds32x3(row_addr[r] + word_a, wa0, wa1, wa2);
                lds32x3(row_addr[r] + word_b, wb0, wb1, wb2);
                const uint32_t ua0 = __funnelshift_r(wa0, wa1, shift_a), ua1 = __funnelshift_r(wa1, wa2, shift_a);
                const uint32_t ub0 = __funnelshift_r(wb0, wb1, shift_b), ub1 = __funnelshift_r(wb1, wb2, shift_b);
                const uint32_t ta = __byte_perm(ua0, ua1, second_a), tb = __byte_perm(ub0, ub1, second_b);
#pragma unroll
                for (int c = 0; c < 3; ++c) {
                    /* Two exact ways from a byte to its float.  The conversion instruction runs on the
                       quarter-rate unit, which was the busiest pipe of this body when it took all twelve
                       conversions of a row pair; placing the byte under the exponent of 2^23 and
                       subtracting 2^23 (one permute per value, one packed add per pair) runs on the
                       integer and FMA pipes.  One channel in three the second way measured fastest
                       (0.170 -> 0.164 ms on the 1024-crop batch; half and half 0.167). */
                    if (c == 2) {
                        tap[r][0][c] = bytes_to_float2_by_bias(ua0, ub0, c);
                        tap[r][1][c] = bytes_to_float2_by_bias(ta, tb, c);
                    } else {
                        tap[r][0][c] = make_float2(byte_to_float(ua0 >> (8 * c)), byte_to_float(ub0 >> (8 * c)));
                        tap[r][1][c] = make_float2(byte_to_float(ta >> (8 * c)), byte_to_float(tb >> (8 * c)));
                    }
                }
            }
            const float2 wy0 = make_float2(wy.x, wy.y), wy1 = make_float2(wy.z, wy.w);
            const float2 w00 = mul2(wx0, wy0), w10 = mul2(wx1, wy0), w01 = mul2(wx0, wy1), w11 = mul2(wx1, wy1);
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                /* ((p00*w00 + p10*w10) + p01*w01) + p11*w11, every product and sum rounded */
                v[c] = add2(add2(add2(mul2(tap[0][0][c], w00), mul2(tap[0][1][c], w10), one), mul2(tap[1][0][c], w01), one),
                            mul2(tap[1][1][c], w11), one);
            }
        };
        auto store_row = [&](uint8_t* oa, const float2& r, const float2& g, const float2& bl) {
            uint8_t* const ob = oa + b_off;
            if (plain) {
                store_pixel_at<PLANAR>(oa, dst_cstride, r.x, g.x, bl.x);
                store_pixel_at<PLANAR>(ob, dst_cstride, r.y, g.y, bl.y);
            } else { /* a column group straddling the edge of the region, or the last odd column */
                store_pixel_at<PLANAR>(oa, dst_cstride, in_a ? r.x : bgv[0], in_a ? g.x : bgv[1], in_a ? bl.x : bgv[2]);
                if (valid_b) store_pixel_at<PLANAR>(ob, dst_cstride, in_b ? r.y : bgv[0], in_b ? g.y : bgv[1], in_b ? bl.y : bgv[2]);
            }
        };

        int y = ya + (int)slot;
        /* two rows of the thread per round: the continuation's parameters are fetched once for both */
#pragma unroll 1
        for (; y + (int)rs <= yb; y += 2 * (int)rs, rt += 4 * rs, out_a += 2 * row_step) {
            float2 v[6], lo[3], hi[3];
            interpolate(rt, lo);
            interpolate(rt + 2 * rs, hi);
#pragma unroll
            for (int c = 0; c < 3; ++c) { v[c] = lo[c]; v[3 + c] = hi[c]; }
            run_ops<CHAIN, 2>(v, sops, S.n_pre, S.n_ops, one);
            store_row(out_a, v[0], v[1], v[2]);
            store_row(out_a + row_step, v[3], v[4], v[5]);
        }
        if (y <= yb) {
            float2 v[3];
            interpolate(rt, v);
            run_ops<CHAIN, 1>(v, sops, S.n_pre, S.n_ops, one);
            store_row(out_a, v[0], v[1], v[2]);
        }
    }

}

/* ------------------------------------------------------------------------------------ */
/* body: bilinear resize of NV12 from source rows staged in shared memory               */
/* ------------------------------------------------------------------------------------ */
__device__ __forceinline__ void mbar_expect_tx_only(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t mbar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr) {
    if (!check_smem(addr, 1u)) return 0u;
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    if (!check_smem(addr, 2u)) return 0u;
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

/* A work item is a band of rows of one plane's region of interest times a tile of its columns.
 * Only the luma and chroma rows that some tap of the band reads with a non-zero weight are
 * copied (an exact 3:1 reduction touches one luma row in three), each as one bulk copy of the
 * tile's byte range widened to 16-byte boundaries.  ReadYUV<NV12> takes Y at (x, y) and the U,V
 * pair at (x>>1, y>>1) (color_conversion.h:329-346); the conversion runs on every tap before
 * the interpolation, as in the reference's chain.  A tap whose weight is exactly zero adds +-0
 * to a sum whose first term is never -0, so it is skipped without changing a bit. */
template <uint32_t CHAIN>
__device__ __forceinline__ void body_nv12_staged(const DevPlane& P, const DevSeq& S, const OpSlot* sops, uint32_t local,
                                                 unsigned char* staged_mem, const WaitCtl wc) {
    constexpr bool PLANAR = false;
    uint8_t* const dst = P.dst;
    const uint32_t dst_pitch = P.dst_pitch, dst_cstride = P.dst_cstride;
    const uint32_t groups_per_row = P.dst_w / PX_PER_THREAD;
    const int x1 = P.x1, y1 = P.y1, x2 = P.x2, y2 = P.y2;
    const uint32_t g_lo = (uint32_t)x1 / PX_PER_THREAD;
    const uint32_t n_groups = (uint32_t)x2 / PX_PER_THREAD - g_lo + 1;
    const uint32_t n_rows = (uint32_t)(y2 - y1 + 1);
    const uint32_t nthreads = blockDim.x, tid = threadIdx.x;
    const float bgv[3] = {S.bg_out[0], S.bg_out[1], S.bg_out[2]};
    const float2 one = dup2(S.one);

    if (local >= P.roi_items) {
        /* store-only item: rows above and below the region of interest */
        fill_cells<PLANAR>(dst, dst_pitch, dst_cstride, (local - P.roi_items) * (nthreads * BG_GROUPS_PER_THREAD), tid, nthreads,
                           BG_GROUPS_PER_THREAD, P.dst_h - n_rows, groups_per_row, 0u, 0u, bgv,
                           [&](uint32_t r) { return (int)r < y1 ? r : r + n_rows; });
        return;
    }

    /* shared memory: | mbarrier (8 B) | row counts (8 B) | row table (32 B per row of the band) | luma flags |
       chroma flags | the luma rows that are read, packed | the chroma rows that are read, packed | */
    uint64_t* const mbar_ptr = reinterpret_cast<uint64_t*>(staged_mem);
    float4* const row_tab = reinterpret_cast<float4*>(staged_mem + 16);
    unsigned char* const need_l = staged_mem + STAGED_HEADER_BYTES;
    unsigned char* const need_c = need_l + NV12_MAX_SPAN;
    unsigned char* const stage = need_c + NV12_MAX_SPAN;
    const uint32_t stage_addr = smem_addr(stage);
    const uint32_t mbar = smem_addr(mbar_ptr);

    const uint32_t tiles_x = P.tiles_x, band_rows = P.seg_pixels, gw = P.gw, rs = P.rs;
    const uint32_t band = div_small(local, tiles_x), tile_x = local - band * tiles_x;
    const int ya = y1 + (int)(band * band_rows);
    const int yb = min(ya + (int)band_rows - 1, y2);
    const int crop_h = P.crop_h, crop_w = P.crop_w, crop_x = P.crop_x, crop_y = P.crop_y;
    const float fx = P.fx, fy = P.fy;

    /* columns of this tile and the byte range of a source row that their taps touch */
    const int c_base = (int)(g_lo * PX_PER_THREAD + tile_x * 2 * gw);
    const int x_end = (int)min((g_lo + n_groups) * PX_PER_THREAD, (uint32_t)c_base + 2 * gw);
    const int rc0 = min(max(c_base, x1), x2), rc1 = max(min(x_end - 1, x2), rc0); /* region columns inside the tile */
    const int sx_first = crop_x + make_axis(max(rc0, x1) - x1, fx, crop_w).i0;
    const int sx_last = crop_x + make_axis(max(rc1, x1) - x1, fx, crop_w).i1;
    const uint32_t byte0 = (uint32_t)sx_first & ~15u;
    const uint32_t row_len = min(((uint32_t)sx_last + 2u + 15u) & ~15u, P.src_pitch) - byte0;

    /* source rows of the band */
    const int l_first = crop_y + make_axis(ya - y1, fy, crop_h).i0;
    const int l_last = crop_y + make_axis(yb - y1, fy, crop_h).i1;
    const uint32_t l_span = (uint32_t)(l_last - l_first + 1);
    const int c_first = l_first >> 1;
    const uint32_t c_span = (uint32_t)((l_last >> 1) - c_first + 1);

    const bool early = wc.nv12_early != 0u; /* rows marked, packed and on their way since the block began (uniform) */
    if (!early) {
    if (tid == 0) {
        mbar_init(mbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    /* flags over the band's span of source rows, in whole 8-byte words for the scan below */
    if (tid < NV12_MAX_SPAN / 8) {
        reinterpret_cast<uint2*>(need_l)[tid] = make_uint2(0u, 0u);
        reinterpret_cast<uint2*>(need_c)[tid] = make_uint2(0u, 0u);
    }
    __syncthreads();
    }
    const bool row_thread = tid <= (uint32_t)(yb - ya);
    Axis ay = {0, 0, 0.0f, 0.0f};
    if (row_thread) {
        ay = make_axis(ya + (int)tid - y1, fy, crop_h);
        if (!early) {
        const int r0 = crop_y + ay.i0, r1 = crop_y + ay.i1;
        need_l[r0 - l_first] = 1;
        need_c[(r0 >> 1) - c_first] = 1;
        if (ay.w1 != 0.0f) { need_l[r1 - l_first] = 1; need_c[(r1 >> 1) - c_first] = 1; }
        }
    }
    if (!early) __syncthreads();
    /* The rows that are read are packed in the stage: a flag becomes 1 + the row's slot (an exclusive prefix sum
       over the flags; warp 0 takes the luma span, warp 1 the chroma span, eight flags per lane). */
    uint32_t* const counts = reinterpret_cast<uint32_t*>(staged_mem + 8); /* needed luma rows, needed chroma rows */
    if (!early && tid < 64) {
        unsigned char* const flags = tid < 32 ? need_l : need_c;
        const uint32_t lane = tid & 31u;
        const uint2 w = reinterpret_cast<const uint2*>(flags)[lane];
        uint32_t f[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) { f[k] = (w.x >> (8 * k)) & 1u; f[4 + k] = (w.y >> (8 * k)) & 1u; }
        uint32_t mine = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) mine += f[k];
        uint32_t incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= (uint32_t)d) incl += up;
        }
        uint32_t slot = incl - mine; /* rows needed before this lane's eight */
        uint32_t o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) { o[k] = f[k] ? slot + 1u : 0u; slot += f[k]; }
        reinterpret_cast<uint2*>(flags)[lane] = make_uint2(o[0] | (o[1] << 8) | (o[2] << 16) | (o[3] << 24),
                                                           o[4] | (o[5] << 8) | (o[6] << 16) | (o[7] << 24));
        if (lane == 31) counts[tid >> 5] = incl;
    }
    if (!early) __syncthreads();
    const uint32_t n_luma = counts[0];
    const uint32_t chroma_addr = stage_addr + n_luma * row_len;
    if (row_thread) {
        const int r0 = crop_y + ay.i0, r1 = crop_y + ay.i1;
        /* shared-memory addresses of the luma and chroma rows of the two vertical taps; a second tap that is never
           read (weight zero) points at the first tap's rows */
        const bool two = ay.w1 != 0.0f;
        const uint32_t a0 = (uint32_t)(need_l[r0 - l_first] - 1u) * row_len;
        const uint32_t a1 = two ? (uint32_t)(need_l[r1 - l_first] - 1u) * row_len : a0;
        const uint32_t b0 = (uint32_t)(need_c[(r0 >> 1) - c_first] - 1u) * row_len;
        const uint32_t b1 = two ? (uint32_t)(need_c[(r1 >> 1) - c_first] - 1u) * row_len : b0;
        row_tab[2 * tid] = make_float4(__uint_as_float(stage_addr + a0), __uint_as_float(stage_addr + a1),
                                       __uint_as_float(chroma_addr + b0), __uint_as_float(chroma_addr + b1));
        row_tab[2 * tid + 1] = make_float4(ay.w0, ay.w0, ay.w1, ay.w1);
    }
    if (!early) {
        const uint8_t* luma = P.src + (size_t)l_first * P.src_pitch + byte0;
        const uint8_t* chroma = P.src + (size_t)P.src_pitch * P.src_height + (size_t)c_first * P.src_pitch + byte0;
        for (uint32_t r = tid; r < l_span; r += nthreads) {
            const uint32_t s1 = need_l[r];
            if (s1) {
                mbar_expect_tx_only(mbar, row_len);
                bulk_copy_g2s(stage_addr + (s1 - 1u) * row_len, luma + (size_t)r * P.src_pitch, row_len, mbar);
            }
        }
        for (uint32_t r = tid; r < c_span; r += nthreads) {
            const uint32_t s1 = need_c[r];
            if (s1) {
                mbar_expect_tx_only(mbar, row_len);
                bulk_copy_g2s(chroma_addr + (s1 - 1u) * row_len, chroma + (size_t)r * P.src_pitch, row_len, mbar);
            }
        }
    }
    __syncthreads(); /* every copy's bytes are expected before the one arrival */
    if (tid == 0) {
        if (wc.test_extra_bytes) mbar_expect_tx_only(mbar, wc.test_extra_bytes);
        mbar_arrive(mbar);
    }

    /* the thread's two columns */
    const uint32_t slot = div_small(tid, gw), gi = tid - slot * gw;
    const int xa = c_base + (int)gi, xb = xa + (int)gw;
    const bool in_a = xa >= x1 && xa <= x2, in_b = xb >= x1 && xb <= x2;
    const bool valid_a = xa < x_end, valid_b = xb < x_end;
    const Axis axa = make_axis(in_a ? xa - x1 : rc0 - x1, fx, crop_w);
    const Axis axb = make_axis(in_b ? xb - x1 : rc0 - x1, fx, crop_w);
    /* byte offsets of the taps in a staged luma row, and of their U,V pairs in a staged chroma row */
    const uint32_t la0 = (uint32_t)(crop_x + axa.i0) - byte0, la1 = (uint32_t)(crop_x + axa.i1) - byte0;
    const uint32_t lb0 = (uint32_t)(crop_x + axb.i0) - byte0, lb1 = (uint32_t)(crop_x + axb.i1) - byte0;
    const uint32_t ca0 = (((uint32_t)(crop_x + axa.i0) >> 1) << 1) - byte0, ca1 = (((uint32_t)(crop_x + axa.i1) >> 1) << 1) - byte0;
    const uint32_t cb0 = (((uint32_t)(crop_x + axb.i0) >> 1) << 1) - byte0, cb1 = (((uint32_t)(crop_x + axb.i1) >> 1) << 1) - byte0;
    const bool col1_a = axa.w1 != 0.0f, col1_b = axb.w1 != 0.0f;
    const int yuv = S.pre_kind; /* PRE_IDENTITY: no conversion */
    const uint32_t u_shift = S.swap_uv ? 8u : 0u, v_shift = 8u - u_shift; /* NV21: the pair is V,U */

    if (!mbar_wait_bounded(mbar, 0, wc.limit_us)) {
        atomicExch(wc.status, STATUS_STAGED_WAIT_TIMEOUT);
        (void)mbar_wait_bounded(mbar, 0, wc.limit_us);
        return;
    }

    /* One tap of the thread's two columns at once: (Y, U, V) pairs as floats, converted when the chain says so.  The
       two columns travel as the halves of packed values, so that every product and sum of the conversion and of the
       blend is one instruction for both (each half rounded like the scalar instruction). */
    const float2 m128 = dup2(-128.0f);
    auto tap2 = [&](uint32_t l_a, uint32_t c_a, uint32_t l_b, uint32_t c_b, float2 (&t)[3]) {
        const uint32_t uva = lds_u16(c_a), uvb = lds_u16(c_b);
        t[0] = make_float2(byte_to_float(lds_u8(l_a)), byte_to_float(lds_u8(l_b)));
        t[1] = make_float2(byte_to_float(uva >> u_shift), byte_to_float(uvb >> u_shift));
        t[2] = make_float2(byte_to_float(uva >> v_shift), byte_to_float(uvb >> v_shift));
        if (yuv == PRE_IDENTITY) return;
        /* the three full-range matrices as in yuv_to_rgb_*_full above, terms that cannot change a bit dropped */
        const float2 u = add2(t[1], m128, one), v = add2(t[2], m128, one);
        float2 y = t[0];
        float kr, kgu, kgv, kb;
        if (yuv == PRE_YUV_BT709) { kr = 1.5748f; kgu = -0.1873f; kgv = -0.4681f; kb = 1.8556f; }
        else if (yuv == PRE_YUV_BT601) {
            y = mul2(add2(y, dup2(-16.0f), one), dup2(1.164383562f));
            kr = 1.596026786f; kgu = -0.39176229f; kgv = -0.812967647f; kb = 2.017232143f;
        } else { kr = 1.4746f; kgu = -0.16455312684366f; kgv = -0.57135312684366f; kb = 1.8814f; }
        t[0] = add2(mul2(v, dup2(kr)), y, one);
        t[1] = add2(mul2(v, dup2(kgv)), add2(mul2(u, dup2(kgu)), y, one), one);
        t[2] = add2(mul2(u, dup2(kb)), y, one);
    };

    if (slot < rs && valid_a) {
        uint8_t* out_a = dst + (size_t)(ya + (int)slot) * dst_pitch + (size_t)xa * 12;
        const size_t b_off = (size_t)gw * 12, row_step = (size_t)rs * dst_pitch;
        const float4* rt = row_tab + 2 * slot;
        /* a second column tap is read for both columns when either has a weight for it: the other's weight is zero and its
           product a zero that changes no bit of the sum (the tap lies inside the staged row either way) */
        const bool col1 = col1_a || col1_b;
        const float2 wx0 = make_float2(axa.w0, axb.w0), wx1 = make_float2(axa.w1, axb.w1);
        const bool plain = in_a && in_b && valid_b;
#pragma unroll 2
        for (int y = ya + (int)slot; y <= yb; y += (int)rs, rt += 2 * rs, out_a += row_step) {
            const float4 rows = rt[0], wy = rt[1];
            const uint32_t lr0 = __float_as_uint(rows.x), lr1 = __float_as_uint(rows.y);
            const uint32_t cr0 = __float_as_uint(rows.z), cr1 = __float_as_uint(rows.w);
            float2 t[3], v[3];
            tap2(lr0 + la0, cr0 + ca0, lr0 + lb0, cr0 + cb0, t);
            const float2 w00 = mul2(wx0, dup2(wy.x));
#pragma unroll
            for (int c = 0; c < 3; ++c) v[c] = mul2(t[c], w00);
            if (col1) {
                tap2(lr0 + la1, cr0 + ca1, lr0 + lb1, cr0 + cb1, t);
                const float2 w10 = mul2(wx1, dup2(wy.x));
#pragma unroll
                for (int c = 0; c < 3; ++c) v[c] = add2(mul2(t[c], w10), v[c], one);
            }
            if (wy.z != 0.0f) {
                tap2(lr1 + la0, cr1 + ca0, lr1 + lb0, cr1 + cb0, t);
                const float2 w01 = mul2(wx0, dup2(wy.z));
#pragma unroll
                for (int c = 0; c < 3; ++c) v[c] = add2(mul2(t[c], w01), v[c], one);
                if (col1) {
                    tap2(lr1 + la1, cr1 + ca1, lr1 + lb1, cr1 + cb1, t);
                    const float2 w11 = mul2(wx1, dup2(wy.z));
#pragma unroll
                    for (int c = 0; c < 3; ++c) v[c] = add2(mul2(t[c], w11), v[c], one);
                }
            }
            run_ops<CHAIN, 1>(v, sops, S.n_pre, S.n_ops, one);
            if (plain) {
                store_pixel_at<PLANAR>(out_a, dst_cstride, v[0].x, v[1].x, v[2].x);
                store_pixel_at<PLANAR>(out_a + b_off, dst_cstride, v[0].y, v[1].y, v[2].y);
            } else {
                store_pixel_at<PLANAR>(out_a, dst_cstride, in_a ? v[0].x : bgv[0], in_a ? v[1].x : bgv[1], in_a ? v[2].x : bgv[2]);
                if (valid_b)
                    store_pixel_at<PLANAR>(out_a + b_off, dst_cstride, in_b ? v[0].y : bgv[0], in_b ? v[1].y : bgv[1], in_b ? v[2].y : bgv[2]);
            }
        }
    }

    /* background to the left and right of this band's rows (first column tile only) */
    const uint32_t n_side = groups_per_row - n_groups;
    if (tile_x == 0 && n_side != 0)
        fill_cells<PLANAR>(dst, dst_pitch, dst_cstride, 0u, tid, nthreads, 0xFFFFFFu, (uint32_t)(yb - ya + 1), n_side, g_lo, n_groups, bgv,
                           [&](uint32_t r) { return (uint32_t)ya + r; });
}

/* ------------------------------------------------------------------------------------ */
/* the kernel                                                                           */
/* ------------------------------------------------------------------------------------ */
/* Chains compiled into the kernels (codes of the operations after the geometry stage, in
 * order).  Casts never reach the device table.  Anything else is interpreted. */
#define FKB_CHAIN_MENU(X)                                                                                         \
    X(chain_of())                                 /* no continuation (copy, Cast -> Resize)                    */ \
    X(chain_of(CH_DIVC))                          /* Div                                                       */ \
    X(chain_of(CH_DIVC) | CHAIN_UNIFORM)          /* the same with one parameter for the three channels        */ \
    X(chain_of(CH_DIVC, CH_SUB, CH_DIVC))         /* Div, Sub, Div: normalise with mean and std                */ \
    X(chain_of(CH_MUL, CH_SUB, CH_DIVC, CH_SWAP)) /* Mul, Sub, Div, RGB2BGR                                    */ \
    X(chain_of(CH_MUL, CH_SUB, CH_DIVC, CH_SWAP) | CHAIN_UNIFORM) /* the same with one parameter for the three channels */ \
    X(chain_of(CH_MUL, CH_SUB, CH_DIVC))          /* Mul, Sub, Div                                             */ \
    X(chain_of(CH_MUL, CH_SUB))                   /* Mul, Sub                                                  */ \
    X(chain_of(CH_ADD, CH_DIVC))                  /* Add, Div                                                  */ \
    X(chain_of(CH_SWAP, CH_MUL, CH_SAT))          /* RGB2BGR, Mul, SaturateCast                                */

/* The bodies of one continuation (compiled chain or interpreter), selected by the plane's class. */
template <uint32_t CLASS, uint32_t CHAIN>
__device__ __forceinline__ void run_class(uint32_t cls, const DevPlane& P, const DevSeq& S, const OpSlot* sops,
                                          uint32_t local, unsigned char* staged_mem, unsigned char* turn_mem, const WaitCtl status) {
    if (CLASS != CLASS_MIXED) cls = CLASS;
    switch (cls) {
        case CLASS_FLAT_U8_F32: body_flat<CHAIN, true, false>(P, S, sops, local, turn_mem); break;
        case CLASS_FLAT_F32_F32: body_flat<CHAIN, false, false>(P, S, sops, local, turn_mem, status.prefetch_items); break;
        case CLASS_FLAT_U8_U8: body_flat<CHAIN, true, true>(P, S, sops, local, turn_mem); break;
        case CLASS_RESIZE_U8_PLANAR: body_resize<CHAIN, FKB_SRC_U8X3, true>(P, S, sops, local); break;
        case CLASS_RESIZE_U8_PACKED: body_resize<CHAIN, FKB_SRC_U8X3, false>(P, S, sops, local); break;
        case CLASS_RESIZE_NV12_PACKED: body_resize<CHAIN, FKB_SRC_NV12, false>(P, S, sops, local); break;
        case CLASS_RESIZE_U8_PLANAR_STAGED:
            body_resize_staged<CHAIN, true>(P, S, sops, local, staged_mem, status);
            break;
        case CLASS_RESIZE_U8_PACKED_STAGED:
            body_resize_staged<CHAIN, false>(P, S, sops, local, staged_mem, status);
            break;
        case CLASS_RESIZE_NV12_PACKED_STAGED:
            if constexpr (CLASS != CLASS_MIXED) body_nv12_staged<CHAIN>(P, S, sops, local, staged_mem, status);
            break;
        default: body_generic(P, S, sops, local); break;
    }
}

/* A plan of one class runs the body of that class with the plan's continuation.  A plan of several
 * classes (divergent horizontal fusion, data_parallel_patterns.h:315-323) selects per block: first
 * the continuation of the plane's sequence, if it is one of the compiled chains, then the class.
 * Each (class, continuation) body is a function of its own (not inlined into the kernel): the
 * register allocation of one body then does not see the others, which is what made the kernel
 * spill when all of them were inlined into one function. */
template <uint32_t CLS, uint32_t CHAIN>
__device__ __noinline__ void mixed_body(const DevPlane* P, const DevSeq* S, const OpSlot* sops, uint32_t local,
                                        unsigned char* staged_mem, unsigned char* turn_mem, const WaitCtl status) {
    run_class<CLS, CHAIN>(CLS, *P, *S, sops, local, staged_mem, turn_mem, status);
}
template <uint32_t CHAIN>
__device__ __forceinline__ void run_mixed_chain(uint32_t cls, const DevPlane* P, const DevSeq* S, const OpSlot* sops,
                                                uint32_t local, unsigned char* staged_mem, unsigned char* turn_mem, const WaitCtl status) {
    switch (cls) {
#define FKB_MIXED_BODY(C) case C: mixed_body<C, CHAIN>(P, S, sops, local, staged_mem, turn_mem, status); break;
        FKB_MIXED_BODY(CLASS_FLAT_U8_F32) FKB_MIXED_BODY(CLASS_FLAT_F32_F32) FKB_MIXED_BODY(CLASS_FLAT_U8_U8)
        FKB_MIXED_BODY(CLASS_RESIZE_U8_PLANAR) FKB_MIXED_BODY(CLASS_RESIZE_U8_PACKED) FKB_MIXED_BODY(CLASS_RESIZE_NV12_PACKED)
        FKB_MIXED_BODY(CLASS_RESIZE_U8_PLANAR_STAGED) FKB_MIXED_BODY(CLASS_RESIZE_U8_PACKED_STAGED)
#undef FKB_MIXED_BODY
        default: mixed_body<CLASS_GENERIC, CHAIN_INTERPRET>(P, S, sops, local, staged_mem, turn_mem, status); break;
    }
}

template <uint32_t CLASS, uint32_t CHAIN>
__device__ __forceinline__ void run_body(uint32_t cls, const DevPlane& P, const DevSeq& S, const OpSlot* sops,
                                         uint32_t local, unsigned char* staged_mem, unsigned char* turn_mem, const WaitCtl status) {
    if constexpr (CLASS != CLASS_MIXED) {
        run_class<CLASS, CHAIN>(cls, P, S, sops, local, staged_mem, turn_mem, status);
    } else {
        const uint32_t chain = S.chain;
#define FKB_MIXED_CASE(CH) \
    if (chain == (CH)) { run_mixed_chain<(CH)>(cls, &P, &S, sops, local, staged_mem, turn_mem, status); return; }
        FKB_CHAIN_MENU(FKB_MIXED_CASE)
#undef FKB_MIXED_CASE
        run_mixed_chain<CHAIN_INTERPRET>(cls, &P, &S, sops, local, staged_mem, turn_mem, status);
    }
}

/* Checked build: what this block's plane allows, written once the plane is known (the bulk copies of the staged uchar3
   classes, which the ordinary build starts before that, start after it). */
#ifdef FKB_CHECK_BOUNDS
__device__ __forceinline__ void check_begin(const DevPlane& P, const DevSeq& S, const LaunchArgs& a, const unsigned char* smem_raw) {
    if (threadIdx.x == 0) {
        const size_t src_rows = source_rows(S.src_format, P.src_height);
        s_check.src_lo = P.src;
        s_check.src_hi = P.src ? P.src + src_rows * P.src_pitch : P.src;
        s_check.dst = P.dst;
        s_check.dst_pitch = P.dst_pitch; s_check.dst_rows = P.dst_h;
        const bool planar = S.dst_format == FKB_DST_F32_PLANAR3;
        const uint32_t px = S.dst_format == FKB_DST_U8X3_PACKED ? 3u : planar ? 4u : 12u;
        s_check.dst_row_bytes = P.dst_w * px;
        s_check.dst_cstride = P.dst_cstride; s_check.dst_channels = planar ? 3u : 1u;
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        s_check.smem_lo = smem_addr(smem_raw); s_check.smem_hi = s_check.smem_lo + dyn;
        s_check.status = a.status;
        if (a.test_shrink_bounds) { /* TEST ONLY: pretend the destination has fewer rows, so that the checker has something to refuse */
            s_check.dst_rows = P.dst_h > a.test_shrink_bounds ? P.dst_h - a.test_shrink_bounds : 0u;
        }
    }
    __syncthreads();
}
#else
__device__ __forceinline__ void check_begin(const DevPlane&, const DevSeq&, const LaunchArgs&, const unsigned char*) {}
#endif

/* Resident blocks per SM that the compiler must leave registers for.  Measured on B200: the staged
 * uchar3 resize runs five blocks (48 registers; four at 64 registers take the same time), the staged NV12
 * resize four (two rows of taps in flight per thread need 64 registers), plans
 * of several classes four as well (the flat bodies hold four runs per thread and the
 * interpolating body its taps: at six blocks and 40 registers both spilled; four groups of 16 images
 * 1920x1080 took 0.319 ms at six, 0.294 at five, 0.285 at four); the bodies that read taps straight
 * from global memory keep all their loads in flight in registers instead.  The flat bodies run
 * five blocks (48 registers, no spills in the compiled chains): a 4K float3 Add took 37.6 us
 * unconstrained (three to four blocks) and 35.9 us at five, 64 alternating Add/Mul 76.6 and 65.7. */
constexpr int min_blocks_of(uint32_t cls) {
    return (cls == CLASS_RESIZE_U8_PLANAR_STAGED || cls == CLASS_RESIZE_U8_PACKED_STAGED) ? 5
           : cls == CLASS_RESIZE_NV12_PACKED_STAGED ? 4
           : cls == CLASS_MIXED ? 4
           : (cls == CLASS_FLAT_U8_F32 || cls == CLASS_FLAT_U8_U8 || cls == CLASS_FLAT_F32_F32) ? 5 : 1;
}
template <uint32_t CLASS, uint32_t CHAIN>
__global__ void __launch_bounds__(BLOCK_THREADS, min_blocks_of(CLASS)) fused_plan_kernel(const __grid_constant__ LaunchArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    OpSlot* sops = reinterpret_cast<OpSlot*>(smem_raw);
    __shared__ DevPlane s_plane;
    __shared__ DevSeq s_seq;
    /* flat bodies: 96 sixteen-byte words per warp in which a run of output is turned around */
    constexpr bool HAS_FLAT = CLASS == CLASS_FLAT_U8_F32 || CLASS == CLASS_FLAT_F32_F32 || CLASS == CLASS_FLAT_U8_U8 || CLASS == CLASS_MIXED;
    __shared__ __align__(16) unsigned char s_turn[HAS_FLAT ? (BLOCK_THREADS / 32) * 96 * 16 : 16];

    if (a.inline_plane) {
        /* one plane: everything is in the kernel arguments; only the operation table is expanded */
        const uint32_t n_ops = (uint32_t)a.seq0.n_ops;
        if (threadIdx.x < n_ops) expand_op(*reinterpret_cast<const uint4*>(&a.ops0[threadIdx.x]), sops + threadIdx.x);
        __syncthreads();
        check_begin(a.plane0, a.seq0, a, smem_raw);
        run_body<CLASS, CHAIN>(a.plane0.plane_class, a.plane0, a.seq0, sops, blockIdx.x, nullptr, s_turn,
                               WaitCtl{a.status, a.wait_limit_us, a.test_extra_bytes, a.prefetch_items});
        return;
    }
    /* One 16-byte table entry tells the block its plane, its tile within the plane and where the
       plane's sequence and operations are, so that the three descriptors arrive in one round trip.
       The staged uchar3 classes have a second entry with the band's copy parameters: warp 0 starts
       the bulk copies of the source rows from it at once, before the plane's descriptor is known. */
    const bool EARLY_COPIES = CLASS == CLASS_RESIZE_U8_PLANAR_STAGED || CLASS == CLASS_RESIZE_U8_PACKED_STAGED ||
                              (CLASS == CLASS_MIXED && a.staged_bytes != 0); /* a plan of several classes with staged planes */
    const bool NV12_EARLY = CLASS == CLASS_RESIZE_NV12_PACKED_STAGED && a.nv12_early != 0u;
    const uint4 entry = __ldg(a.items + (EARLY_COPIES ? 2u * blockIdx.x : NV12_EARLY ? NV12_ITEM_WORDS * blockIdx.x : blockIdx.x));
    if (NV12_EARLY && threadIdx.x < 64) {
        /* The staged NV12 class: the work item's table words name the source rows that some tap of the band tile reads
           (one bit per row of the luma and of the chroma span, found by the host with the kernel's own arithmetic).
           Warp 0 takes the luma rows, warp 1 the chroma rows, eight per lane: a prefix sum over the bit counts gives every
           row its slot in the stage, the row's copy starts, and the slots (plus one; zero = not read) are left in shared
           memory for the row table.  The copies are on their way one round trip after the block began, instead of after
           the plane's descriptor, the marking of the rows and three block barriers. */
        const uint4* const words = a.items + NV12_ITEM_WORDS * blockIdx.x;
        const uint4 ptrs = __ldg(words + 1), geo = __ldg(words + 2); /* luma, chroma bases; pitch, row bytes, luma span, luma rows */
        const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
        const uint32_t bits = __ldg(reinterpret_cast<const unsigned char*>(words + 4 + 2u * warp) + lane);
        unsigned char* const staged = smem_raw + (((a.max_seq_ops > 0 ? a.max_seq_ops : 1u) * (uint32_t)sizeof(OpSlot) + 127u) & ~127u);
        const uint32_t mbar = smem_addr(staged);
        unsigned char* const flags = staged + STAGED_HEADER_BYTES + warp * NV12_MAX_SPAN;
        const uint32_t stage_addr = smem_addr(staged + STAGED_HEADER_BYTES + 2u * NV12_MAX_SPAN);
        if (threadIdx.x == 0) {
            mbar_init(mbar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        asm volatile("bar.sync 1, 64;" ::: "memory"); /* the barrier is initialised before warp 1 counts bytes on it */
        const uint32_t pitch = geo.x, row_len = geo.y;
        const uint32_t mine = __popc(bits);
        uint32_t incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= (uint32_t)d) incl += up;
        }
        uint32_t slot = incl - mine; /* rows read before this lane's eight */
        const uint8_t* const base = reinterpret_cast<const uint8_t*>(warp == 0 ? ((size_t)ptrs.x | ((size_t)ptrs.y << 32)) : ((size_t)ptrs.z | ((size_t)ptrs.w << 32)));
        const uint32_t dst0 = stage_addr + (warp == 0 ? 0u : geo.w * row_len);
        uint32_t o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const bool read = (bits >> k) & 1u;
            o[k] = read ? slot + 1u : 0u;
            if (read) {
                mbar_expect_tx_only(mbar, row_len);
                bulk_copy_g2s(dst0 + slot * row_len, base + (size_t)(lane * 8u + (uint32_t)k) * pitch, row_len, mbar);
                ++slot;
            }
        }
        reinterpret_cast<uint2*>(flags)[lane] = make_uint2(o[0] | (o[1] << 8) | (o[2] << 16) | (o[3] << 24), o[4] | (o[5] << 8) | (o[6] << 16) | (o[7] << 24));
        if (lane == 31) reinterpret_cast<uint32_t*>(staged + 8)[warp] = incl;
    }
    auto start_band_copies = [&]() {
        if (EARLY_COPIES && threadIdx.x < 32) {
            const uint4 cp = __ldg(a.items + 2u * blockIdx.x + 1u); /* source pointer, rows | row bytes << 16, pitch */
            unsigned char* const staged = smem_raw + (((a.max_seq_ops > 0 ? a.max_seq_ops : 1u) * (uint32_t)sizeof(OpSlot) + 127u) & ~127u);
            const uint32_t mbar = smem_addr(staged), stage_addr = smem_addr(staged + STAGED_U8_HEADER_BYTES);
            if (a.tiled_copies) {
                /* the whole footprint as one tile of the plane's tensor map: tensor map index, -, bytes of the box,
                   x | y << 16 (x in eight-byte elements, even, so that the copy starts on a 16-byte boundary) */
                if (threadIdx.x == 0 && cp.z != 0u) {
                    mbar_init(mbar, 1);
                    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                    mbar_expect_tx(mbar, cp.z + a.test_extra_bytes);
                    /* a tile lands on a 128-byte boundary and starts at an even element; anything else is never expected
                       and is not issued (the block's wait then runs out and reports it) */
                    if (((stage_addr & 127u) | (cp.w & 1u)) == 0u) {
                        /* the map lies in global memory, written by the host when the plan was made, at an address that an
                           earlier plan's map may have had: the copy engine's view of it is brought up to date first */
                        const unsigned char* const tmap = a.tmaps + (size_t)cp.x * TENSOR_MAP_BYTES;
                        asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(tmap) : "memory");
                        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                     ::"r"(stage_addr), "l"(tmap), "r"(cp.w & 0xFFFFu), "r"(cp.w >> 16), "r"(mbar)
                                     : "memory");
                    }
                }
                return;
            }
            const uint32_t n_src = cp.z & 0xFFFFu, row_len = cp.z >> 16;
            if (n_src != 0) {
                if (threadIdx.x == 0) {
                    mbar_init(mbar, 1);
                    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                    mbar_expect_tx(mbar, n_src * row_len + a.test_extra_bytes);
                }
                __syncwarp();
                const uint8_t* g = reinterpret_cast<const uint8_t*>((size_t)cp.x | ((size_t)cp.y << 32));
                for (uint32_t r = threadIdx.x; r < n_src; r += 32) bulk_copy_g2s(stage_addr + r * row_len, g + (size_t)r * cp.w, row_len, mbar);
            }
        }
    };
#ifndef FKB_CHECK_BOUNDS
    start_band_copies();
#endif
    const uint32_t plane_idx = entry.x, local = entry.y, seq = entry.z & 0xFFFFu, n_ops = entry.z >> 16, ops_begin = entry.w;
    /* the descriptors are fetched by the warps that do not issue copies (staged NV12: warps 2 and up of 8; staged uchar3:
       warps 1 and up of 4 or 8), so that they travel while the copies are issued */
    const uint32_t skip = NV12_EARLY ? 64u : EARLY_COPIES ? 32u : 0u;
    const uint32_t t = threadIdx.x - skip;
    if (t < sizeof(DevPlane) / 16) {
        reinterpret_cast<uint4*>(&s_plane)[t] = __ldg(reinterpret_cast<const uint4*>(a.planes + plane_idx) + t);
    } else if (t >= 32 && t < 32 + sizeof(DevSeq) / 16) {
        reinterpret_cast<uint4*>(&s_seq)[t - 32] = __ldg(reinterpret_cast<const uint4*>(a.seqs + seq) + (t - 32));
    } else if (t >= 64 && t < blockDim.x) {
        for (uint32_t k = t - 64; k < n_ops; k += blockDim.x - 64 - skip)
            expand_op(__ldg(reinterpret_cast<const uint4*>(a.ops + ops_begin + k)), sops + k);
    }
    __syncthreads();
    check_begin(s_plane, s_seq, a, smem_raw);
#ifdef FKB_CHECK_BOUNDS
    start_band_copies(); /* the checked build starts them once it knows what the plane allows */
#endif
    /* staged classes: the region after the operation cache, on a 128-byte boundary */
    unsigned char* staged_mem = smem_raw + (((a.max_seq_ops > 0 ? a.max_seq_ops : 1u) * (uint32_t)sizeof(OpSlot) + 127u) & ~127u);
    run_body<CLASS, CHAIN>(s_plane.plane_class, s_plane, s_seq, sops, local, staged_mem, s_turn,
                           WaitCtl{a.status, a.wait_limit_us, a.test_extra_bytes, 0u, NV12_EARLY ? 1u : 0u});
}

/* ------------------------------------------------------------------------------------ */
/* launching one instantiation                                                          */
/* ------------------------------------------------------------------------------------ */

/* Launches one instantiation; the first launch that needs more than the default 48 KB of
   shared memory raises the kernel's limit (once per instantiation and device). */
template <uint32_t CLASS, uint32_t CHAIN>
static cudaError_t launch_one(const LaunchArgs& a, size_t smem, cudaStream_t stream) {
    /* the kernel's static shared memory (descriptors, the flat bodies' turn-around buffer: under
       13 KB) counts against the same 48 KB */
    if (smem + 13 * 1024 > 48 * 1024) {
        static std::mutex mu; /* launches may come from several host threads */
        static size_t raised[64] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || raised[dev] < smem) {
            e = cudaFuncSetAttribute(fused_plan_kernel<CLASS, CHAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) raised[dev] = smem;
        }
    }
    fused_plan_kernel<CLASS, CHAIN><<<a.total_items, a.block_threads, smem, stream>>>(a);
    return cudaGetLastError();
}

template <uint32_t CLASS>
static cudaError_t launch_class(uint32_t chain, const LaunchArgs& a, size_t smem, cudaStream_t stream) {
#define FKB_LAUNCH_CASE(CH) \
    if (chain == (CH)) return launch_one<CLASS, (CH)>(a, smem, stream);
    FKB_CHAIN_MENU(FKB_LAUNCH_CASE)
#undef FKB_LAUNCH_CASE
    return launch_one<CLASS, CHAIN_INTERPRET>(a, smem, stream);
}

/* One function per translation unit (fkb_launch_*.cu). */
cudaError_t launch_flat(uint32_t cls, uint32_t chain, const LaunchArgs& a, size_t smem, cudaStream_t stream);
cudaError_t launch_resize(uint32_t cls, uint32_t chain, const LaunchArgs& a, size_t smem, cudaStream_t stream);
cudaError_t launch_staged(uint32_t cls, uint32_t chain, const LaunchArgs& a, size_t smem, cudaStream_t stream);
cudaError_t launch_nv12_staged(uint32_t chain, const LaunchArgs& a, size_t smem, cudaStream_t stream);
cudaError_t launch_mixed(const LaunchArgs& a, size_t smem, cudaStream_t stream);

}  // namespace fkb

#endif
