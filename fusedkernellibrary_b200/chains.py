"""Plan builders for the sender chains of the benchmark configurations.

Each helper lowers one reference-style chain (PerThreadRead -> Crop -> Resize -> ... ->
receiver) to an `abi.HostPlan`.  Pointers are plain integers: device pointers for the CUDA
path, host pointers (e.g. numpy `.ctypes.data`) when the same plan is handed to the checker.
"""
from __future__ import annotations

import numpy as np

from . import abi
from .abi import (DST_F32_PLANAR3, DST_F32X3_PACKED, DST_U8X3_PACKED, OP_ADD, OP_CAST_F32, OP_DIV,
                  OP_MUL, OP_SATURATE_CAST_U8, OP_SUB, OP_SWAP_RB, OP_YUV_TO_RGB_BT709_FULL,
                  RESIZE_IGNORE_AR, RESIZE_NONE, RESIZE_PRESERVE_AR, SRC_F32X3, SRC_NV12, SRC_U8X3, op)

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)
README_RECTS = np.array([(0, 0, 34, 25), (10, 10, 70, 15), (20, 20, 60, 59), (30, 30, 20, 23),
                         (40, 40, 12, 11)], np.int32)


def elementwise(ops, *, src, dst, width, height, src_format=SRC_U8X3, dst_format=DST_F32X3_PACKED,
                src_pitch=None, dst_pitch=None, plan=None, crop=None):
    """Read -> ops -> PerThreadWrite on one image (no geometry stage)."""
    spx = {SRC_U8X3: 3, SRC_F32X3: 12}[src_format]
    dpx = 3 if dst_format == DST_U8X3_PACKED else 12   # float3, int3 and uint3 pixels are twelve bytes
    plan = plan or abi.HostPlan()
    seq = plan.add_sequence(src_format, dst_format, RESIZE_NONE, list(ops))
    cw, ch = (crop[2], crop[3]) if crop is not None else (width, height)
    plan.add_plane(src=src, src_width=width, src_height=height, src_pitch=src_pitch or width * spx,
                   dst=dst, dst_width=cw, dst_height=ch, dst_pitch=dst_pitch or cw * dpx, crop=crop,
                   sequence=seq)
    return plan


def cast_mul_sub_div_ops(mul=1.4, sub=0.5, div=255.0):
    """Config 1: Cast<uchar3,float3> -> Mul -> Sub -> Div."""
    return [op(OP_CAST_F32), op(OP_MUL, mul), op(OP_SUB, sub), op(OP_DIV, div)]


def addmul_ops(n, add=0.001, mul=1.0001):
    """Config 5A: n alternating Add / Mul operations, Add first."""
    return [op(OP_ADD, add) if i % 2 == 0 else op(OP_MUL, mul) for i in range(n)]


def crop_resize_batch(*, frame_ptrs, frame_index, rects, src_width, src_height, src_pitch, dst, dst_width,
                      dst_height, post_ops, planar, mode=RESIZE_PRESERVE_AR, background=(0.0, 0.0, 0.0),
                      plan=None):
    """PerThreadRead[B] -> Crop[B] -> Resize -> post_ops -> TensorWrite (packed) or TensorSplit (planar).

    `dst` is the base of a dense tensor: B x dh x dw x 3 floats (packed) or B x 3 x dh x dw (planar)."""
    plan = plan or abi.HostPlan()
    seq = plan.add_sequence(SRC_U8X3, DST_F32_PLANAR3 if planar else DST_F32X3_PACKED, mode, list(post_ops),
                            n_pre_ops=0, background=background)
    plane_bytes = dst_width * dst_height * 12
    for i, (fi, r) in enumerate(zip(frame_index, rects)):
        plan.add_plane(src=frame_ptrs[fi], src_width=src_width, src_height=src_height, src_pitch=src_pitch,
                       crop=tuple(int(v) for v in r), dst=dst + i * plane_bytes, dst_width=dst_width,
                       dst_height=dst_height, dst_pitch=dst_width * (4 if planar else 12),
                       dst_channel_stride=dst_width * dst_height * 4 if planar else 0, sequence=seq)
    return plan


def readme_ops(mul=1.4, sub=0.5, div=255.0):
    """Config 2 continuation: Mul -> Sub -> Div -> COLOR_RGB2BGR."""
    return [op(OP_MUL, mul), op(OP_SUB, sub), op(OP_DIV, div), op(OP_SWAP_RB)]


def normalize_ops(mean=IMAGENET_MEAN, std=IMAGENET_STD):
    """Config 3 continuation: Div(255) -> Sub(mean) -> Div(std)."""
    return [op(OP_DIV, 255.0), op(OP_SUB, mean), op(OP_DIV, std)]


def nv12_resize_batch(*, frame_ptrs, width, height, pitch, dst, dst_width, dst_height, div=255.0, plan=None,
                      mode=RESIZE_IGNORE_AR, background=(0.0, 0.0, 0.0), crops=None, src_format=SRC_NV12,
                      conversion=OP_YUV_TO_RGB_BT709_FULL):
    """Config 4: ReadYUV<NV12>[B] -> ConvertYUVToRGB<bt709, Full, float3> -> Resize(IGNORE_AR) -> Div
    -> TensorWrite<float3>.  `crops` (one rect per frame), PRESERVE_AR, NV21 and the other matrices are variations."""
    plan = plan or abi.HostPlan()
    seq = plan.add_sequence(src_format, DST_F32X3_PACKED, mode,
                            [op(conversion), op(OP_DIV, div)], n_pre_ops=1, background=background)
    plane_bytes = dst_width * dst_height * 12
    for i, p in enumerate(frame_ptrs):
        plan.add_plane(src=p, src_width=width, src_height=height, src_pitch=pitch, dst=dst + i * plane_bytes,
                       dst_width=dst_width, dst_height=dst_height, dst_pitch=dst_width * 12, sequence=seq,
                       crop=None if crops is None else tuple(int(v) for v in crops[i]))
    return plan


def divergent_four_groups(*, src_ptrs, width, height, dst_ptrs, resize_to=(960, 540), per_group=16):
    """Config 5B: one plan, four different sequences on four groups of `per_group` uchar3 images.

    dst_ptrs[g] is the base of group g's dense output tensor.
    g0: Cast -> Mul(1.4) -> Sub(0.5)            -> float3
    g1: Cast -> Add(0.5) -> Div(255)            -> float3
    g2: RGB2BGR -> Cast -> Mul(1.4) -> Saturate -> uchar3
    g3: Cast -> Resize IGNORE_AR(resize_to)     -> float3"""
    plan = abi.HostPlan()
    rw, rh = resize_to
    seqs = [
        plan.add_sequence(SRC_U8X3, DST_F32X3_PACKED, RESIZE_NONE, [op(OP_CAST_F32), op(OP_MUL, 1.4), op(OP_SUB, 0.5)]),
        plan.add_sequence(SRC_U8X3, DST_F32X3_PACKED, RESIZE_NONE, [op(OP_CAST_F32), op(OP_ADD, 0.5), op(OP_DIV, 255.0)]),
        plan.add_sequence(SRC_U8X3, DST_U8X3_PACKED, RESIZE_NONE,
                          [op(OP_SWAP_RB), op(OP_CAST_F32), op(OP_MUL, 1.4), op(OP_SATURATE_CAST_U8)]),
        plan.add_sequence(SRC_U8X3, DST_F32X3_PACKED, RESIZE_IGNORE_AR, [op(OP_CAST_F32)], n_pre_ops=1),
    ]
    out_dims = [(width, height, 12), (width, height, 12), (width, height, 3), (rw, rh, 12)]
    for g in range(4):
        ow, oh, px = out_dims[g]
        for i in range(per_group):
            plan.add_plane(src=src_ptrs[g * per_group + i], src_width=width, src_height=height,
                           src_pitch=width * 3, dst=dst_ptrs[g] + i * ow * oh * px, dst_width=ow,
                           dst_height=oh, dst_pitch=ow * px, sequence=seqs[g])
    return plan


def random_rects(rng: np.random.Generator, n, src_width, src_height, lo=16, hi=512):
    """Config 3 crop rects: width and height uniform in [lo, hi], origin uniform within bounds."""
    w = rng.integers(lo, min(hi, src_width) + 1, n)
    h = rng.integers(lo, min(hi, src_height) + 1, n)
    x = (rng.random(n) * (src_width - w + 1)).astype(np.int64)
    y = (rng.random(n) * (src_height - h + 1)).astype(np.int64)
    return np.stack([x, y, w, h], 1).astype(np.int32)
