/* CPU restatement of the reference's fused-execution path, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared with; it
 * is never linked into, imported by or called from the product library.  It consumes the
 * same plain-old-data plan description as the C ABI (include/fkb200.h) but with HOST
 * pointers, and walks it the way the reference's CPU backend does: three nested loops
 * over z, y, x calling the per-thread function (core/execution_model/
 * data_parallel_patterns.h:285-298, execute_thread :153-181).
 *
 * Parity status: PINNED.  Every function below is checked bit-for-bit against the
 * reference's own headers compiled here (oracle/ref/, built into oracle/_ref/) by
 * tests/test_oracle_golden.py, and against the golden vectors under tests/golden/
 * that were generated from that build.
 *
 * All arithmetic is IEEE-754 binary32, round-to-nearest-even, without contraction: build
 * with -ffp-contract=off (the reference's tests are built in ISO mode, which implies it:
 * cmake/tests/add_generated_test.cmake:30).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "fkb200.h"

/* cxp::round for positive/negative finite floats: core/constexpr_libs/constexpr_cmath.h:119-130 */
static float cxp_roundf(float x) {
    return (x > 0.0f) ? (float)(int)(x + 0.5f) : (float)(int)(x - 0.5f);
}

/* Resize::build + compute_target_size: algorithms/image_processing/resize.h:105-166,196-221 */
int fkl_oracle_derive_resize(int sw, int sh, int dw, int dh, int mode, fkb_resize_params* out) {
    int tw = dw, th = dh;
    if (sw <= 0 || sh <= 0 || dw <= 0 || dh <= 0 || !out) return 1;
    if (mode == FKB_RESIZE_PRESERVE_AR || mode == FKB_RESIZE_PRESERVE_AR_RN_EVEN || mode == FKB_RESIZE_PRESERVE_AR_LEFT) {
        const float scale = (float)dh / (float)sh;             /* resize.h:197 */
        th = dh;
        tw = (int)cxp_roundf(scale * (float)sw);               /* resize.h:199 */
        if (mode == FKB_RESIZE_PRESERVE_AR_RN_EVEN) tw -= tw % 2;  /* resize.h:200-202 */
        if (tw > dw) {                                         /* resize.h:203-207, 212-216 */
            const float scale2 = (float)dw / (float)sw;
            tw = dw;
            th = (int)cxp_roundf(scale2 * (float)sh);
            if (mode == FKB_RESIZE_PRESERVE_AR_RN_EVEN) th -= th % 2;
        }
        out->x1 = mode == FKB_RESIZE_PRESERVE_AR_LEFT ? 0 : (dw - tw) / 2;  /* resize.h:132-133, 150-151 */
        out->y1 = (dh - th) / 2;
        out->x2 = out->x1 + tw - 1;
        out->y2 = out->y1 + th - 1;
    } else if (mode == FKB_RESIZE_IGNORE_AR) {
        out->x1 = 0; out->y1 = 0; out->x2 = dw - 1; out->y2 = dh - 1;
    } else {
        return 1;
    }
    {
        const double cfx = (double)tw / (double)sw;            /* resize.h:108-109,127-128 */
        const double cfy = (double)th / (double)sh;
        out->fx = (float)(1.0 / cfx);
        out->fy = (float)(1.0 / cfy);
    }
    out->target_width = tw;
    out->target_height = th;
    return 0;
}

typedef struct { float v[3]; } px3;

/* The read operation at crop-relative coordinates (a, b):
 * Crop::exec adds the rect origin (image_processing/crop.h:35-38); PerThreadRead loads at
 * base + y*pitch + x*sizeof(T) (memory_operations.h:80-83, core/data/rawptr.h:205-207);
 * ReadYUV<NV12> loads Y at (x,y) and the U,V pair at (x>>1, y>>1) of the chroma plane that
 * starts at data + pitch*height (color_conversion.h:329-346). */
static px3 read_tap(const fkb_plane* pl, int src_format, int a, int b) {
    px3 r;
    const int x = a + pl->crop_x, y = b + pl->crop_y;
    const uint8_t* base = (const uint8_t*)pl->src;
    if (src_format == FKB_SRC_U8X3) {
        const uint8_t* p = base + (size_t)y * pl->src_pitch + (size_t)x * 3;
        r.v[0] = (float)p[0]; r.v[1] = (float)p[1]; r.v[2] = (float)p[2];
    } else if (src_format == FKB_SRC_F32X3) {
        const float* p = (const float*)(base + (size_t)y * pl->src_pitch + (size_t)x * 12);
        r.v[0] = p[0]; r.v[1] = p[1]; r.v[2] = p[2];
    } else if (src_format == FKB_SRC_P010 || src_format == FKB_SRC_P210) {
        /* 16-bit luma plane, interleaved 16-bit chroma at data + pitch*height; 4:2:0 halves the chroma row, 4:2:2 does not
           (color_conversion.h:329-346).  ConvertYUVToRGB first shifts the words right by 6 (:292, :177-180): done here. */
        const uint16_t* luma = (const uint16_t*)(base + (size_t)y * pl->src_pitch) + x;
        const int cy = src_format == FKB_SRC_P010 ? (y >> 1) : y;
        const uint16_t* chroma = (const uint16_t*)(base + (size_t)pl->src_pitch * pl->src_height + (size_t)cy * pl->src_pitch) + 2 * (x >> 1);
        r.v[0] = (float)(luma[0] >> 6); r.v[1] = (float)(chroma[0] >> 6); r.v[2] = (float)(chroma[1] >> 6);
    } else if (src_format == FKB_SRC_Y210) { /* Y0 U Y1 V per two pixels (:360-372) */
        const uint16_t* q = (const uint16_t*)(base + (size_t)y * pl->src_pitch) + 4 * (x >> 1);
        r.v[0] = (float)(q[(x & 1) ? 2 : 0] >> 6); r.v[1] = (float)(q[1] >> 6); r.v[2] = (float)(q[3] >> 6);
    } else if (src_format == FKB_SRC_UYVY) { /* U Y0 V Y1 per two pixels (:360-369) */
        const uint8_t* q = base + (size_t)y * pl->src_pitch + 4 * (size_t)(x >> 1);
        r.v[0] = (float)q[(x & 1) ? 3 : 1]; r.v[1] = (float)q[0]; r.v[2] = (float)q[2];
    } else { /* FKB_SRC_NV12, FKB_SRC_NV21 (the pair is stored V,U: color_conversion.h:357-359) */
        const uint8_t* luma = base + (size_t)y * pl->src_pitch + (size_t)x;
        const uint8_t* chroma = base + (size_t)pl->src_pitch * pl->src_height +
                                (size_t)(y >> 1) * pl->src_pitch + (size_t)(x >> 1) * 2;
        const int u_at = src_format == FKB_SRC_NV21 ? 1 : 0;
        r.v[0] = (float)luma[0]; r.v[1] = (float)chroma[u_at]; r.v[2] = (float)chroma[1 - u_at];
    }
    return r;
}

/* BorderReader's index maps: idx_low(idx_high(i)) for an axis of n elements (border_reader.h:163-273). */
static int border_index(int mode, int i, int n) {
    const int last = n - 1;
    int v;
    switch (mode) {
        case FKB_BORDER_REPLICATE: v = i < last ? i : last; return v > 0 ? v : 0;               /* :169-186 */
        case FKB_BORDER_REFLECT:                                                                /* :198-215 */
            v = last - abs(last - i) + (i > last);
            return (abs(v) - (v < 0)) % (last + 1);
        case FKB_BORDER_WRAP:                                                                   /* :232-249 */
            v = (i < n) ? i : (i % n);
            return (v >= 0) ? v : (v - ((v - n + 1) / n) * n);
        case FKB_BORDER_REFLECT_101:                                                            /* :261-272 */
            v = abs(last - abs(last - i)) % (last + 1);
            return abs(v) % (last + 1);
        default: return i;
    }
}

/* The read chain at crop-relative (a, b): PerThreadRead -> [BorderReader | Deinterlace] -> Crop. */
static px3 read_chain(const fkb_plane* pl, const fkb_sequence* sq, int a, int b) {
    px3 r, p, q;
    int c;
    if (sq->border_mode == FKB_BORDER_NONE && sq->deinterlace == FKB_DEINTERLACE_NONE) return read_tap(pl, sq->src_format, a, b);
    {
        /* image coordinates; read_tap adds the crop origin, so hand it coordinates relative to the crop */
        const int x = a + pl->crop_x, y = b + pl->crop_y, w = (int)pl->src_width, h = (int)pl->src_height;
        if (sq->border_mode == FKB_BORDER_CONSTANT) {                                           /* :140-148 */
            if (x >= 0 && x < w && y >= 0 && y < h) return read_tap(pl, sq->src_format, a, b);
            r.v[0] = sq->border_value[0]; r.v[1] = sq->border_value[1]; r.v[2] = sq->border_value[2];
            return r;
        }
        if (sq->border_mode != FKB_BORDER_NONE)
            return read_tap(pl, sq->src_format, border_index(sq->border_mode, x, w) - pl->crop_x, border_index(sq->border_mode, y, h) - pl->crop_y);
        /* Deinterlace, deinterlace.h:91-131 */
        if (sq->deinterlace == FKB_DEINTERLACE_BLEND) {
            if (y <= 0) return read_tap(pl, sq->src_format, a, b);
            p = read_tap(pl, sq->src_format, a, b);
            q = read_tap(pl, sq->src_format, a, b - 1);
        } else {
            const int even = (y % 2) == 0;
            const int interpolate = sq->deinterlace == FKB_DEINTERLACE_LINEAR_EVEN ? (!even && y != h - 1) : (even && y != 0);
            if (!interpolate) return read_tap(pl, sq->src_format, a, b);
            p = read_tap(pl, sq->src_format, a, b - 1);
            q = read_tap(pl, sq->src_format, a, b + 1);
        }
        /* (p + q + 1) * 0.5f: an integer sum for uchar3 (exact in binary32), two rounded additions for float3 */
        for (c = 0; c < 3; ++c) r.v[c] = ((p.v[c] + q.v[c]) + 1.0f) * 0.5f;
        return r;
    }
}

/* `src_format` matters to the YUV conversions only: the 10-bit layouts subtract 512 (and 64 from the luma for bt601)
   instead of 128 (16) and scale the result by 64 instead of 1 (color_conversion.h:187-191, 234-252). */
static px3 apply_op(px3 in, const fkb_op* op, int src_format) {
    px3 o = in;
    int c;
    const int ten = src_format == FKB_SRC_P010 || src_format == FKB_SRC_P210 || src_format == FKB_SRC_Y210;
    const float csub = ten ? 512.0f : 128.0f, ysub = ten ? 64.0f : 16.0f, scale = ten ? 64.0f : 1.0f;
    switch (op->opcode) {
        case FKB_OP_MUL: for (c = 0; c < 3; ++c) o.v[c] = in.v[c] * op->p[c]; break; /* arithmetic.h:71 */
        case FKB_OP_SUB: for (c = 0; c < 3; ++c) o.v[c] = in.v[c] - op->p[c]; break; /* arithmetic.h:58 */
        case FKB_OP_DIV: for (c = 0; c < 3; ++c) o.v[c] = in.v[c] / op->p[c]; break; /* arithmetic.h:84 */
        case FKB_OP_ADD: for (c = 0; c < 3; ++c) o.v[c] = in.v[c] + op->p[c]; break; /* arithmetic.h:33 */
        case FKB_OP_CAST_F32: break;                     /* uchar -> float is exact (cast_base.h:20-30) */
        case FKB_OP_SWAP_RB: o.v[0] = in.v[2]; o.v[2] = in.v[0]; break;  /* cuda_vector.h:57-61 */
        case FKB_OP_SATURATE_CAST_U8:                    /* saturate.h:27-50 */
            for (c = 0; c < 3; ++c) {
                const float f = in.v[c];
                if (f > 255.0f) o.v[c] = 255.0f;
                else if (f < 0.0f) o.v[c] = 0.0f;
                else o.v[c] = (float)(uint8_t)cxp_roundf(f);
            }
            break;
        case FKB_OP_CAST_I32:                            /* Cast<float3,int3>: static_cast per channel, cast_base.h:20-30 */
            for (c = 0; c < 3; ++c) { const int32_t i = (int32_t)in.v[c]; memcpy(&o.v[c], &i, 4); }  /* kept as bits */
            break;
        case FKB_OP_CAST_U32:                            /* Cast<float3,uint3> */
            for (c = 0; c < 3; ++c) { const uint32_t u = (uint32_t)in.v[c]; memcpy(&o.v[c], &u, 4); }
            break;
        case FKB_OP_YUV_TO_RGB_BT709_FULL: {             /* color_conversion.h:265-308, :143-146 */
            /* (Y, U-128, V-128) times the matrix rows, each row reduced left to right
               (algebraic.h:58-64, cuda_vector.h:113-126), then scaled by 1.0f (:241-243). */
            const float y = in.v[0], u = in.v[1] - csub, v = in.v[2] - csub;
            o.v[0] = ((y * 1.0f + u * 0.0f) + v * 1.5748f) * scale;
            o.v[1] = ((y * 1.0f + u * -0.1873f) + v * -0.4681f) * scale;
            o.v[2] = ((y * 1.0f + u * 1.8556f) + v * 0.0f) * scale;
            break;
        }
        case FKB_OP_YUV_TO_RGB_BT601_FULL: {             /* :137-140, luma offset :266-269 */
            const float y = in.v[0] - ysub, u = in.v[1] - csub, v = in.v[2] - csub;
            o.v[0] = ((y * 1.164383562f + u * 0.0f) + v * 1.596026786f) * scale;
            o.v[1] = ((y * 1.164383562f + u * -0.39176229f) + v * -0.812967647f) * scale;
            o.v[2] = ((y * 1.164383562f + u * 2.017232143f) + v * 0.0f) * scale;
            break;
        }
        case FKB_OP_YUV_TO_RGB_BT2020_FULL: {            /* :165-168 */
            const float y = in.v[0], u = in.v[1] - csub, v = in.v[2] - csub;
            o.v[0] = ((y * 1.0f + u * 0.0f) + v * 1.4746f) * scale;
            o.v[1] = ((y * 1.0f + u * -0.16455312684366f) + v * -0.57135312684366f) * scale;
            o.v[2] = ((y * 1.0f + u * 1.8814f) + v * 0.0f) * scale;
            break;
        }
        default: break;
    }
    return o;
}

static px3 read_pre(const fkb_plane* pl, const fkb_sequence* sq, int n_pre, int a, int b) {
    px3 t = read_chain(pl, sq, a, b);
    int k;
    for (k = 0; k < n_pre; ++k) t = apply_op(t, &sq->ops[k], sq->src_format);
    return t;
}

/* Interpolate<INTER_LINEAR>::exec: image_processing/interpolation.h:61-96.
 * host_branch != 0 reproduces the reference's host branch (:69-70), which takes the
 * vertical tap index from the horizontal coordinate; 0 follows the device branch (:66-67). */
static px3 interpolate(const fkb_plane* pl, const fkb_sequence* sq, int n_pre, float sx, float sy,
                       int host_branch) {
    const int x1 = (int)floorf(sx);
    const int y1 = host_branch ? (int)floorf(sx) : (int)floorf(sy);
    const int x2 = x1 + 1, y2 = y1 + 1;
    const int x2r = x2 < pl->crop_width - 1 ? x2 : pl->crop_width - 1;    /* :76 */
    const int y2r = y2 < pl->crop_height - 1 ? y2 : pl->crop_height - 1;  /* :77 */
    const px3 p00 = read_pre(pl, sq, n_pre, x1, y1);
    const px3 p10 = read_pre(pl, sq, n_pre, x2r, y1);
    const px3 p01 = read_pre(pl, sq, n_pre, x1, y2r);
    const px3 p11 = read_pre(pl, sq, n_pre, x2r, y2r);
    const float w00 = ((float)x2 - sx) * ((float)y2 - sy);               /* :92-95 */
    const float w10 = (sx - (float)x1) * ((float)y2 - sy);
    const float w01 = ((float)x2 - sx) * (sy - (float)y1);
    const float w11 = (sx - (float)x1) * (sy - (float)y1);
    px3 r;
    int c;
    for (c = 0; c < 3; ++c) {
        r.v[c] = ((p00.v[c] * w00 + p10.v[c] * w10) + p01.v[c] * w01) + p11.v[c] * w11;
    }
    return r;
}

/* Receivers: PerThreadWrite / TensorWrite at base + y*pitch + x*sizeof(T)
 * (memory_operations.h:122-127,181-184; rawptr.h:222-225 with the plane offset already in
 * fkb_plane.dst); TensorSplit writes channel c at +c*(width*height) elements
 * (memory_operations.h:203-219). */
static void write_px(const fkb_plane* pl, int dst_format, int x, int y, px3 v) {
    uint8_t* base = (uint8_t*)pl->dst;
    if (dst_format == FKB_DST_F32X3_PACKED || dst_format == FKB_DST_I32X3_PACKED || dst_format == FKB_DST_U32X3_PACKED) {
        /* int3 / uint3 values are carried as bit patterns (see FKB_OP_CAST_I32) */
        float* p = (float*)(base + (size_t)y * pl->dst_pitch + (size_t)x * 12);
        p[0] = v.v[0]; p[1] = v.v[1]; p[2] = v.v[2];
    } else if (dst_format == FKB_DST_F32_PLANAR3) {
        int c;
        for (c = 0; c < 3; ++c) {
            float* p = (float*)(base + (size_t)c * pl->dst_channel_stride + (size_t)y * pl->dst_pitch +
                                (size_t)x * 4);
            *p = v.v[c];
        }
    } else {
        uint8_t* p = base + (size_t)y * pl->dst_pitch + (size_t)x * 3;
        p[0] = (uint8_t)v.v[0]; p[1] = (uint8_t)v.v[1]; p[2] = (uint8_t)v.v[2];
    }
}

/* Runs planes [first, first+count) of a plan description whose image pointers are host
 * pointers.  host_branch: see interpolate().  Returns 0, or 1 for a malformed plan. */
int fkl_oracle_run_range(const fkb_plan_desc* d, int first, int count, int host_branch) {
    int z;
    if (!d || !d->planes || !d->sequences || first < 0 || count < 0 || first + count > d->n_planes) return 1;
    for (z = first; z < first + count; ++z) {
        const fkb_plane* pl = &d->planes[z];
        const fkb_sequence* sq;
        fkb_resize_params rp;
        int x, y, k;
        if (pl->sequence < 0 || pl->sequence >= d->n_sequences) return 1;
        sq = &d->sequences[pl->sequence];
        memset(&rp, 0, sizeof rp);
        const int is_default = (pl->flags & FKB_PLANE_DEFAULT_VALUE) != 0;  /* batch_operations.h:236-241 */
        const int warp = sq->resize_mode == FKB_GEOMETRY_WARP_AFFINE || sq->resize_mode == FKB_GEOMETRY_WARP_PERSPECTIVE;
        if (sq->resize_mode != FKB_RESIZE_NONE && !is_default && !warp) {
            if (fkl_oracle_derive_resize(pl->crop_width, pl->crop_height, (int)pl->dst_width,
                                         (int)pl->dst_height, sq->resize_mode, &rp)) return 1;
        }
        for (y = 0; y < (int)pl->dst_height; ++y) {
            for (x = 0; x < (int)pl->dst_width; ++x) {
                px3 v;
                int first_post = 0;
                if (is_default) {
                    first_post = sq->resize_mode == FKB_RESIZE_NONE ? 0 : sq->n_pre_ops;
                    v.v[0] = sq->background[0]; v.v[1] = sq->background[1]; v.v[2] = sq->background[2];
                } else if (sq->resize_mode == FKB_RESIZE_NONE) {
                    v = read_chain(pl, sq, x, y);
                } else if (warp) {
                    /* WarpingCoords + Warping::exec, warping.h:49-69, 86-94 */
                    const float* m = sq->transform;
                    float cx = (m[0] * (float)x + m[1] * (float)y) + m[2];
                    float cy = (m[3] * (float)x + m[4] * (float)y) + m[5];
                    first_post = sq->n_pre_ops;
                    if (sq->resize_mode == FKB_GEOMETRY_WARP_PERSPECTIVE) {
                        const float coeff = 1.0f / ((m[6] * (float)x + m[7] * (float)y) + m[8]);
                        cx = coeff * cx;
                        cy = coeff * cy;
                    }
                    if (cx >= 0.0f && cx < (float)pl->crop_width && cy >= 0.0f && cy < (float)pl->crop_height) {
                        v = interpolate(pl, sq, sq->n_pre_ops, cx, cy, 0);
                    } else {
                        v.v[0] = 0.0f; v.v[1] = 0.0f; v.v[2] = 0.0f;
                    }
                } else {
                    first_post = sq->n_pre_ops;
                    /* Resize::exec, resize.h:75-87 */
                    if (sq->resize_mode != FKB_RESIZE_IGNORE_AR &&
                        !(x >= rp.x1 && x <= rp.x2 && y >= rp.y1 && y <= rp.y2)) {
                        v.v[0] = sq->background[0]; v.v[1] = sq->background[1]; v.v[2] = sq->background[2];
                    } else {
                        const int rx = x - rp.x1, ry = y - rp.y1;
                        const float sx = (float)rx * rp.fx;      /* resize.h:186-187 */
                        const float sy = (float)ry * rp.fy;
                        v = interpolate(pl, sq, sq->n_pre_ops, sx, sy, host_branch);
                    }
                }
                for (k = first_post; k < sq->n_ops; ++k) v = apply_op(v, &sq->ops[k], sq->src_format);
                write_px(pl, sq->dst_format, x, y, v);
            }
        }
    }
    return 0;
}

int fkl_oracle_run(const fkb_plan_desc* d, int host_branch) {
    return fkl_oracle_run_range(d, 0, d ? d->n_planes : 0, host_branch);
}

/* getDefaultBlockSize / computeBestSolution: core/execution_model/executors.h:176-242.
 * Scan order (32,8) (32,6) (64,4) (64,3) (128,2) (128,3) (256,1) (256,2); keep the first
 * strict minimum of discarded threads; stop early at 0 or after a new minimum at (256,2)'s
 * predecessor column as the reference does. */
static unsigned discarded(unsigned w, unsigned h, unsigned bx, unsigned by) {
    const unsigned mx = w % bx, my = h % by;
    const unsigned dx = mx == 0 ? 0 : bx - mx;
    const unsigned dy = my == 0 ? 0 : by - my;
    return dx * (my == 0 ? h : (h + by)) + dy * w;
}

void fkl_oracle_block_size(unsigned w, unsigned h, unsigned* bx, unsigned* by) {
    static const unsigned BX[4] = {32, 64, 128, 256};
    static const unsigned BY[2][4] = {{8, 4, 2, 1}, {6, 3, 3, 2}};
    unsigned best = 0xFFFFFFFFu, bi = 0, bj = 0, i, j;
    for (i = 0; i < 4; ++i) {
        for (j = 0; j < 2; ++j) {
            const unsigned d = discarded(w, h, BX[i], BY[j][i]);
            if (best > d) {
                best = d; bi = i; bj = j;
                if (best == 0) goto done;            /* :201, :215 */
                if (i == 3 && j == 1) goto done;
            }
        }
    }
done:
    *bx = BX[bi];
    *by = BY[bj][bi];
}
