/* sm_100a kernels of the fused-execution path and their launcher.
 *
 * One grid serves a whole plan: thread block b looks up its work item (plane, tile) in a
 * device-resident table, copies that plane's descriptor and its operation sequence into
 * shared memory, and runs the body selected by the plane's class.  A plan whose planes all
 * share one class is launched with that body alone; a plan with several classes (divergent
 * horizontal fusion, data_parallel_patterns.h:315-323) is launched with a block-uniform
 * switch over the bodies.
 *
 * Arithmetic follows the reference's per-thread function exactly (execute_thread,
 * data_parallel_patterns.h:153-181): IEEE binary32, round to nearest even, no fused
 * multiply-add, true division; every operation is spelled with the __f*_rn intrinsics so
 * that compiler flags cannot change the rounding.
 */
#include <cuda_runtime.h>
#include <stdint.h>

#include "fkb200.h"
#include "fkb_device.h"

namespace fkb {

/* ------------------------------------------------------------------------------------ */
/* element-wise operations                                                              */
/* ------------------------------------------------------------------------------------ */

/* SaturateCast<float, uchar>: clamp, then cxp::round = (int)(x + 0.5f) for x > 0
 * (image_processing/saturate.h:27-50, constexpr_libs/constexpr_cmath.h:119-130). */
__device__ __forceinline__ float saturate_round_u8(float f) {
    if (f > 255.0f) return 255.0f;
    if (f < 0.0f) return 0.0f;
    return (float)__float2int_rz(__fadd_rn(f, 0.5f));
}

/* Exact uchar -> float without the conversion unit: 2^23 + b has b in its low mantissa bits. */
__device__ __forceinline__ float u8_to_float(uint32_t b) {
    return __fsub_rn(__uint_as_float(b | 0x4B000000u), 8388608.0f);
}

/* Byte LANE of a packed word, as float: one byte permute builds 2^23 + b, one add removes 2^23. */
template <int LANE>
__device__ __forceinline__ float packed_u8_to_float(uint32_t w) {
    return __fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440 | LANE)), 8388608.0f);
}

/* x / p for a divisor known when the plan was made: with r = RN(1/p),
 *     q0 = RN(x*r);  e = x - p*q0 (exact, one FMA);  q = RN(q0 + e*r)
 * The host emits this form only for divisors for which it has checked the sequence against
 * IEEE division on all 2^23 significands of x, and only where it has shown that x stays in
 * the range in which scaling by powers of two is exact (see prove_fast_division in
 * fkb_host.cu).  np is -p. */
__device__ __forceinline__ float div_by_constant(float x, float np, float r) {
    const float q0 = __fmul_rn(x, r);
    const float e = __fmaf_rn(np, q0, x);
    return __fmaf_rn(e, r, q0);
}

/* ConvertYUVToRGB<NV12, Full, bt709, false, float3> (color_conversion.h:265-308; matrix
 * :143-146; row reduction left to right, basic_ops/algebraic.h:58-64). */
__device__ __forceinline__ void yuv_to_rgb_bt709_full(float& a, float& b, float& c) {
    const float y = a, u = __fsub_rn(b, 128.0f), v = __fsub_rn(c, 128.0f);
    a = __fmul_rn(__fadd_rn(__fadd_rn(__fmul_rn(y, 1.0f), __fmul_rn(u, 0.0f)), __fmul_rn(v, 1.5748f)), 1.0f);
    b = __fmul_rn(__fadd_rn(__fadd_rn(__fmul_rn(y, 1.0f), __fmul_rn(u, -0.1873f)), __fmul_rn(v, -0.4681f)), 1.0f);
    c = __fmul_rn(__fadd_rn(__fadd_rn(__fmul_rn(y, 1.0f), __fmul_rn(u, 1.8556f)), __fmul_rn(v, 0.0f)), 1.0f);
}

/* Runs ops [begin, end) of a sequence (cached in shared memory) on NPX whole pixels held in
 * registers as v[3*i + channel].  The opcode is uniform across the block, so the switch
 * never diverges; its cost is shared by 3*NPX values. */
template <int NPX>
__device__ __forceinline__ void apply_ops(float (&v)[NPX * 3], const DevOp* __restrict__ sops, int begin, int end) {
    for (int k = begin; k < end; ++k) {
        const float4 o = *reinterpret_cast<const float4*>(&sops[k]);
        const int opcode = __float_as_int(o.x);
        switch (opcode) {
            case FKB_OP_MUL:
#pragma unroll
                for (int i = 0; i < NPX; ++i) {
                    v[3 * i + 0] = __fmul_rn(v[3 * i + 0], o.y);
                    v[3 * i + 1] = __fmul_rn(v[3 * i + 1], o.z);
                    v[3 * i + 2] = __fmul_rn(v[3 * i + 2], o.w);
                }
                break;
            case FKB_OP_SUB:
#pragma unroll
                for (int i = 0; i < NPX; ++i) {
                    v[3 * i + 0] = __fsub_rn(v[3 * i + 0], o.y);
                    v[3 * i + 1] = __fsub_rn(v[3 * i + 1], o.z);
                    v[3 * i + 2] = __fsub_rn(v[3 * i + 2], o.w);
                }
                break;
            case FKB_OP_DIV:
#pragma unroll
                for (int i = 0; i < NPX; ++i) {
                    v[3 * i + 0] = __fdiv_rn(v[3 * i + 0], o.y);
                    v[3 * i + 1] = __fdiv_rn(v[3 * i + 1], o.z);
                    v[3 * i + 2] = __fdiv_rn(v[3 * i + 2], o.w);
                }
                break;
            case FKB_OP_ADD:
#pragma unroll
                for (int i = 0; i < NPX; ++i) {
                    v[3 * i + 0] = __fadd_rn(v[3 * i + 0], o.y);
                    v[3 * i + 1] = __fadd_rn(v[3 * i + 1], o.z);
                    v[3 * i + 2] = __fadd_rn(v[3 * i + 2], o.w);
                }
                break;
            case DEV_OP_DIV_BY_CONSTANT: { /* two slots: {-p}, {1/p} */
                const float4 r = *reinterpret_cast<const float4*>(&sops[k + 1]);
                ++k;
#pragma unroll
                for (int i = 0; i < NPX; ++i) {
                    v[3 * i + 0] = div_by_constant(v[3 * i + 0], o.y, r.y);
                    v[3 * i + 1] = div_by_constant(v[3 * i + 1], o.z, r.z);
                    v[3 * i + 2] = div_by_constant(v[3 * i + 2], o.w, r.w);
                }
                break;
            }
            case FKB_OP_SWAP_RB:
#pragma unroll
                for (int i = 0; i < NPX; ++i) {
                    const float t = v[3 * i + 0];
                    v[3 * i + 0] = v[3 * i + 2];
                    v[3 * i + 2] = t;
                }
                break;
            case FKB_OP_SATURATE_CAST_U8:
#pragma unroll
                for (int i = 0; i < NPX * 3; ++i) v[i] = saturate_round_u8(v[i]);
                break;
            case FKB_OP_YUV_TO_RGB_BT709_FULL:
#pragma unroll
                for (int i = 0; i < NPX; ++i) yuv_to_rgb_bt709_full(v[3 * i + 0], v[3 * i + 1], v[3 * i + 2]);
                break;
            default: /* FKB_OP_CAST_F32: uchar -> float is exact, values are already float */
                break;
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* reads                                                                                */
/* ------------------------------------------------------------------------------------ */

/* The read operation at crop-relative (a, b): Crop::exec adds the rect origin
 * (image_processing/crop.h:35-38); PerThreadRead loads base + y*pitch + x*sizeof(T)
 * (memory_operations.h:80-83, core/data/rawptr.h:205-207); ReadYUV<NV12> takes Y at (x,y)
 * and the U,V pair at (x>>1, y>>1) of the plane starting at base + pitch*height
 * (color_conversion.h:329-346). */
template <int SRC>
__device__ __forceinline__ void read_tap(const DevPlane& P, int a, int b, float& r0, float& r1, float& r2) {
    const int x = a + P.crop_x, y = b + P.crop_y;
    if (SRC == FKB_SRC_U8X3) {
        const uint8_t* p = P.src + (size_t)y * P.src_pitch + (size_t)x * 3;
        r0 = u8_to_float(__ldg(p)); r1 = u8_to_float(__ldg(p + 1)); r2 = u8_to_float(__ldg(p + 2));
    } else if (SRC == FKB_SRC_F32X3) {
        const float* p = reinterpret_cast<const float*>(P.src + (size_t)y * P.src_pitch + (size_t)x * 12);
        r0 = __ldg(p); r1 = __ldg(p + 1); r2 = __ldg(p + 2);
    } else {
        const uint8_t* luma = P.src + (size_t)y * P.src_pitch + (size_t)x;
        const uint8_t* chroma = P.src + (size_t)P.src_pitch * P.src_height + (size_t)(y >> 1) * P.src_pitch +
                                (size_t)(x >> 1) * 2;
        r0 = u8_to_float(__ldg(luma)); r1 = u8_to_float(__ldg(chroma)); r2 = u8_to_float(__ldg(chroma + 1));
    }
}

__device__ __forceinline__ void read_tap_any(int src_format, const DevPlane& P, int a, int b, float& r0, float& r1,
                                             float& r2) {
    if (src_format == FKB_SRC_U8X3) read_tap<FKB_SRC_U8X3>(P, a, b, r0, r1, r2);
    else if (src_format == FKB_SRC_F32X3) read_tap<FKB_SRC_F32X3>(P, a, b, r0, r1, r2);
    else read_tap<FKB_SRC_NV12>(P, a, b, r0, r1, r2);
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

/* ((p00*w00 + p10*w10) + p01*w01) + p11*w11, products and sums rounded separately. */
__device__ __forceinline__ float blend(float p00, float p10, float p01, float p11, float w00, float w10, float w01,
                                       float w11) {
    return __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(p00, w00), __fmul_rn(p10, w10)), __fmul_rn(p01, w01)),
                     __fmul_rn(p11, w11));
}

/* ------------------------------------------------------------------------------------ */
/* body: generic, one output pixel per thread                                           */
/* ------------------------------------------------------------------------------------ */
__device__ __forceinline__ void body_generic(const DevPlane& P, const DevSeq& S, const DevOp* sops, uint32_t local) {
    const uint32_t idx = local * ITEM_PIXELS_GENERIC + threadIdx.x;
    if (idx >= P.dst_w * P.dst_h) return;
    const int y = idx / P.dst_w, x = idx - y * P.dst_w;
    float v[3];
    int first_post = 0;
    if (S.resize_mode == FKB_RESIZE_NONE) {
        read_tap_any(S.src_format, P, x, y, v[0], v[1], v[2]);
    } else {
        first_post = S.n_pre;
        /* Resize::exec (resize.h:75-87): outside the region of interest return the default */
        if (S.resize_mode == FKB_RESIZE_PRESERVE_AR && !(x >= P.x1 && x <= P.x2 && y >= P.y1 && y <= P.y2)) {
            v[0] = S.bg[0]; v[1] = S.bg[1]; v[2] = S.bg[2];
        } else {
            const Axis ax = make_axis(x - P.x1, P.fx, P.crop_w);
            const Axis ay = make_axis(y - P.y1, P.fy, P.crop_h);
            float t[4][3];
            read_tap_any(S.src_format, P, ax.i0, ay.i0, t[0][0], t[0][1], t[0][2]);
            read_tap_any(S.src_format, P, ax.i1, ay.i0, t[1][0], t[1][1], t[1][2]);
            read_tap_any(S.src_format, P, ax.i0, ay.i1, t[2][0], t[2][1], t[2][2]);
            read_tap_any(S.src_format, P, ax.i1, ay.i1, t[3][0], t[3][1], t[3][2]);
            if (S.pre_kind != PRE_IDENTITY) {
#pragma unroll
                for (int k = 0; k < 4; ++k) apply_ops<1>(t[k], sops, 0, S.n_pre);
            }
            const float w00 = __fmul_rn(ax.w0, ay.w0), w10 = __fmul_rn(ax.w1, ay.w0);
            const float w01 = __fmul_rn(ax.w0, ay.w1), w11 = __fmul_rn(ax.w1, ay.w1);
#pragma unroll
            for (int c = 0; c < 3; ++c) v[c] = blend(t[0][c], t[1][c], t[2][c], t[3][c], w00, w10, w01, w11);
        }
    }
    apply_ops<1>(v, sops, first_post, S.n_ops);
    /* receivers: memory_operations.h:122-127 (PerThreadWrite), :181-184 (TensorWrite),
       :203-219 (TensorSplit) */
    if (S.dst_format == FKB_DST_F32X3_PACKED) {
        float* p = reinterpret_cast<float*>(P.dst + (size_t)y * P.dst_pitch + (size_t)x * 12);
        p[0] = v[0]; p[1] = v[1]; p[2] = v[2];
    } else if (S.dst_format == FKB_DST_F32_PLANAR3) {
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            *reinterpret_cast<float*>(P.dst + (size_t)c * P.dst_cstride + (size_t)y * P.dst_pitch + (size_t)x * 4) =
                v[c];
        }
    } else {
        uint8_t* p = P.dst + (size_t)y * P.dst_pitch + (size_t)x * 3;
        p[0] = (uint8_t)v[0]; p[1] = (uint8_t)v[1]; p[2] = (uint8_t)v[2];
    }
}

/* ------------------------------------------------------------------------------------ */
/* body: no geometry stage, four whole pixels per thread                                */
/* ------------------------------------------------------------------------------------ */
template <bool SRC_IS_U8, bool DST_IS_U8>
__device__ __forceinline__ void body_flat(const DevPlane& P, const DevSeq& S, const DevOp* sops, uint32_t local) {
    constexpr int SPX = SRC_IS_U8 ? 3 : 12;
    constexpr int DPX = DST_IS_U8 ? 3 : 12;
    const uint32_t items_per_seg = (P.seg_pixels + ITEM_PIXELS_VEC - 1) / ITEM_PIXELS_VEC;
    const uint32_t seg = local / items_per_seg;
    const uint32_t px0 = (local - seg * items_per_seg) * ITEM_PIXELS_VEC + threadIdx.x * PX_PER_THREAD;
    if (px0 >= P.seg_pixels) return;
    const uint32_t n = min((uint32_t)PX_PER_THREAD, P.seg_pixels - px0);
    const uint8_t* src = P.src + (size_t)(P.crop_y + seg) * P.src_pitch + (size_t)P.crop_x * SPX + (size_t)px0 * SPX;
    uint8_t* dst = P.dst + (size_t)seg * P.dst_pitch + (size_t)px0 * DPX;

    float v[12];
    if (n == PX_PER_THREAD) {
        if (SRC_IS_U8) {
            const uint32_t* s4 = reinterpret_cast<const uint32_t*>(src);
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const uint32_t w = __ldg(s4 + k);
                v[4 * k + 0] = packed_u8_to_float<0>(w);
                v[4 * k + 1] = packed_u8_to_float<1>(w);
                v[4 * k + 2] = packed_u8_to_float<2>(w);
                v[4 * k + 3] = packed_u8_to_float<3>(w);
            }
        } else {
            const float4* s4 = reinterpret_cast<const float4*>(src);
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float4 w = __ldg(s4 + k);
                v[4 * k + 0] = w.x; v[4 * k + 1] = w.y; v[4 * k + 2] = w.z; v[4 * k + 3] = w.w;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 12; ++i) {
            v[i] = 0.0f;
            if (i < (int)n * 3) {
                v[i] = SRC_IS_U8 ? (float)__ldg(src + i) : __ldg(reinterpret_cast<const float*>(src) + i);
            }
        }
    }

    apply_ops<PX_PER_THREAD>(v, sops, 0, S.n_ops);

    if (n == PX_PER_THREAD) {
        if (DST_IS_U8) {
            uint32_t* d4 = reinterpret_cast<uint32_t*>(dst);
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                d4[k] = (uint32_t)(uint8_t)v[4 * k + 0] | ((uint32_t)(uint8_t)v[4 * k + 1] << 8) |
                        ((uint32_t)(uint8_t)v[4 * k + 2] << 16) | ((uint32_t)(uint8_t)v[4 * k + 3] << 24);
            }
        } else {
            float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
            for (int k = 0; k < 3; ++k) d4[k] = make_float4(v[4 * k + 0], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 12; ++i) {
            if (i < (int)n * 3) {
                if (DST_IS_U8) dst[i] = (uint8_t)v[i];
                else reinterpret_cast<float*>(dst)[i] = v[i];
            }
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* body: bilinear resize, a 4-column group walked down several rows per thread          */
/* ------------------------------------------------------------------------------------ */
template <int SRC, bool PLANAR>
__device__ __forceinline__ void body_resize(const DevPlane& P, const DevSeq& S, const DevOp* sops, uint32_t local) {
    const ResizeTiling T = resize_tiling(P.dst_w, P.dst_h);
    const uint32_t tile_y = local / T.tiles_x, tile_x = local - tile_y * T.tiles_x;
    const uint32_t slot = threadIdx.x / T.gw, gi = threadIdx.x - slot * T.gw;
    const uint32_t group = tile_x * T.gw + gi;
    if (slot >= T.rs || group >= P.dst_w / PX_PER_THREAD) return;
    const int x0 = group * PX_PER_THREAD;
    const bool preserve = S.resize_mode == FKB_RESIZE_PRESERVE_AR;

    /* The value every output element outside the region of interest ends up with: the
       default value run through the continuation (resize.h:84-86). */
    float bgv[3] = {S.bg[0], S.bg[1], S.bg[2]};
    if (preserve) apply_ops<1>(bgv, sops, S.n_pre, S.n_ops);

    /* horizontal taps and weights of the four columns, once per thread */
    int xa0[PX_PER_THREAD], xa1[PX_PER_THREAD];
    float wx0[PX_PER_THREAD], wx1[PX_PER_THREAD];
    uint32_t inside = 0;
#pragma unroll
    for (int i = 0; i < PX_PER_THREAD; ++i) {
        const int x = x0 + i;
        const bool in = !preserve || (x >= P.x1 && x <= P.x2);
        const Axis ax = make_axis(in ? x - P.x1 : 0, P.fx, P.crop_w);
        xa0[i] = ax.i0; xa1[i] = ax.i1; wx0[i] = ax.w0; wx1[i] = ax.w1;
        inside |= (in ? 1u : 0u) << i;
    }
    const uint8_t* const src0 =
        SRC == FKB_SRC_NV12 ? P.src : P.src + (size_t)P.crop_y * P.src_pitch + (size_t)P.crop_x * 3;

    const int y_first = tile_y * (T.rs * RESIZE_ROWS_PER_THREAD) + slot;
#pragma unroll 1
    for (int j = 0; j < RESIZE_ROWS_PER_THREAD; ++j) {
        const int y = y_first + j * (int)T.rs;
        if (y >= (int)P.dst_h) break;
        const bool row_inside = !preserve || (y >= P.y1 && y <= P.y2);
        float v[12];
        if (row_inside && inside != 0) {
            const Axis ay = make_axis(y - P.y1, P.fy, P.crop_h);
#pragma unroll
            for (int i = 0; i < PX_PER_THREAD; ++i) {
                float t[4][3];
                if (SRC == FKB_SRC_U8X3) {
                    const uint8_t* r0 = src0 + (size_t)ay.i0 * P.src_pitch;
                    const uint8_t* r1 = src0 + (size_t)ay.i1 * P.src_pitch;
                    const uint8_t* p00 = r0 + xa0[i] * 3; const uint8_t* p10 = r0 + xa1[i] * 3;
                    const uint8_t* p01 = r1 + xa0[i] * 3; const uint8_t* p11 = r1 + xa1[i] * 3;
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        t[0][c] = u8_to_float(__ldg(p00 + c)); t[1][c] = u8_to_float(__ldg(p10 + c));
                        t[2][c] = u8_to_float(__ldg(p01 + c)); t[3][c] = u8_to_float(__ldg(p11 + c));
                    }
                } else {
                    read_tap<SRC>(P, xa0[i], ay.i0, t[0][0], t[0][1], t[0][2]);
                    read_tap<SRC>(P, xa1[i], ay.i0, t[1][0], t[1][1], t[1][2]);
                    read_tap<SRC>(P, xa0[i], ay.i1, t[2][0], t[2][1], t[2][2]);
                    read_tap<SRC>(P, xa1[i], ay.i1, t[3][0], t[3][1], t[3][2]);
                    if (S.pre_kind == PRE_YUV_BT709) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) yuv_to_rgb_bt709_full(t[k][0], t[k][1], t[k][2]);
                    }
                }
                const float w00 = __fmul_rn(wx0[i], ay.w0), w10 = __fmul_rn(wx1[i], ay.w0);
                const float w01 = __fmul_rn(wx0[i], ay.w1), w11 = __fmul_rn(wx1[i], ay.w1);
#pragma unroll
                for (int c = 0; c < 3; ++c) v[3 * i + c] = blend(t[0][c], t[1][c], t[2][c], t[3][c], w00, w10, w01, w11);
            }
            apply_ops<PX_PER_THREAD>(v, sops, S.n_pre, S.n_ops);
            if (inside != 0xF) {
#pragma unroll
                for (int i = 0; i < PX_PER_THREAD; ++i) {
                    if (!((inside >> i) & 1u)) { v[3 * i + 0] = bgv[0]; v[3 * i + 1] = bgv[1]; v[3 * i + 2] = bgv[2]; }
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < PX_PER_THREAD; ++i) { v[3 * i + 0] = bgv[0]; v[3 * i + 1] = bgv[1]; v[3 * i + 2] = bgv[2]; }
        }

        if (PLANAR) {
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                float4* d = reinterpret_cast<float4*>(P.dst + (size_t)c * P.dst_cstride + (size_t)y * P.dst_pitch +
                                                      (size_t)x0 * 4);
                *d = make_float4(v[c], v[3 + c], v[6 + c], v[9 + c]);
            }
        } else {
            float4* d = reinterpret_cast<float4*>(P.dst + (size_t)y * P.dst_pitch + (size_t)x0 * 12);
#pragma unroll
            for (int k = 0; k < 3; ++k) d[k] = make_float4(v[4 * k + 0], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* the kernel                                                                           */
/* ------------------------------------------------------------------------------------ */
template <uint32_t CLASS>
__device__ __forceinline__ void run_body(uint32_t cls, const DevPlane& P, const DevSeq& S, const DevOp* sops,
                                         uint32_t local) {
    if (CLASS != CLASS_MIXED) cls = CLASS;
    switch (cls) {
        case CLASS_FLAT_U8_F32: body_flat<true, false>(P, S, sops, local); break;
        case CLASS_FLAT_F32_F32: body_flat<false, false>(P, S, sops, local); break;
        case CLASS_FLAT_U8_U8: body_flat<true, true>(P, S, sops, local); break;
        case CLASS_RESIZE_U8_PLANAR: body_resize<FKB_SRC_U8X3, true>(P, S, sops, local); break;
        case CLASS_RESIZE_U8_PACKED: body_resize<FKB_SRC_U8X3, false>(P, S, sops, local); break;
        case CLASS_RESIZE_NV12_PACKED: body_resize<FKB_SRC_NV12, false>(P, S, sops, local); break;
        default: body_generic(P, S, sops, local); break;
    }
}

template <uint32_t CLASS>
__global__ void __launch_bounds__(BLOCK_THREADS) fused_plan_kernel(const __grid_constant__ LaunchArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    DevOp* sops = reinterpret_cast<DevOp*>(smem_raw);
    __shared__ DevPlane s_plane;
    __shared__ DevSeq s_seq;

    const uint32_t item = blockIdx.x;
    uint32_t plane_idx, local;
    if (a.uniform_items) {
        plane_idx = item / a.uniform_items;
        local = item - plane_idx * a.uniform_items;
    } else {
        /* largest p with item_start[p] <= item */
        uint32_t lo = 0, hi = a.n_planes;
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (__ldg(a.item_start + mid) <= item) lo = mid; else hi = mid;
        }
        plane_idx = lo;
        local = item - __ldg(a.item_start + lo);
    }
    if (threadIdx.x < sizeof(DevPlane) / 16) {
        reinterpret_cast<uint4*>(&s_plane)[threadIdx.x] =
            __ldg(reinterpret_cast<const uint4*>(a.planes + plane_idx) + threadIdx.x);
    }
    __syncthreads();
    const uint32_t seq = s_plane.seq;
    if (threadIdx.x < sizeof(DevSeq) / 16) {
        reinterpret_cast<uint4*>(&s_seq)[threadIdx.x] = __ldg(reinterpret_cast<const uint4*>(a.seqs + seq) + threadIdx.x);
    }
    {
        const DevSeq* gs = a.seqs + seq;
        const int n_ops = __ldg(&gs->n_ops), begin = __ldg(&gs->ops_begin);
        for (int k = threadIdx.x; k < n_ops; k += BLOCK_THREADS) {
            reinterpret_cast<uint4*>(sops)[k] = __ldg(reinterpret_cast<const uint4*>(a.ops + begin + k));
        }
    }
    __syncthreads();
    run_body<CLASS>(s_plane.plane_class, s_plane, s_seq, sops, local);
}

/* ------------------------------------------------------------------------------------ */
/* launcher                                                                             */
/* ------------------------------------------------------------------------------------ */
template <uint32_t CLASS>
static cudaError_t launch_one(const LaunchArgs& a, size_t smem, cudaStream_t stream) {
    fused_plan_kernel<CLASS><<<a.total_items, BLOCK_THREADS, smem, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_plan_kernel(uint32_t launch_class, const LaunchArgs& a, cudaStream_t stream) {
    const size_t smem = (size_t)(a.max_seq_ops > 0 ? a.max_seq_ops : 1) * sizeof(DevOp);
    switch (launch_class) {
        case CLASS_GENERIC: return launch_one<CLASS_GENERIC>(a, smem, stream);
        case CLASS_FLAT_U8_F32: return launch_one<CLASS_FLAT_U8_F32>(a, smem, stream);
        case CLASS_FLAT_F32_F32: return launch_one<CLASS_FLAT_F32_F32>(a, smem, stream);
        case CLASS_FLAT_U8_U8: return launch_one<CLASS_FLAT_U8_U8>(a, smem, stream);
        case CLASS_RESIZE_U8_PLANAR: return launch_one<CLASS_RESIZE_U8_PLANAR>(a, smem, stream);
        case CLASS_RESIZE_U8_PACKED: return launch_one<CLASS_RESIZE_U8_PACKED>(a, smem, stream);
        case CLASS_RESIZE_NV12_PACKED: return launch_one<CLASS_RESIZE_NV12_PACKED>(a, smem, stream);
        default: return launch_one<CLASS_MIXED>(a, smem, stream);
    }
}

}  // namespace fkb
