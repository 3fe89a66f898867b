"""Seeded parity cases shared by the CPU and GPU tests.

A case holds named host arrays (sources and zero-initialised outputs) and a function that
lowers its sender chain to a plan given a `ptr(name) -> int` lookup, so that the same chain
can be run by the checker on host pointers and by the CUDA path on device pointers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import numpy as np

from fusedkernellibrary_b200 import abi, chains
from fusedkernellibrary_b200.abi import op


@dataclass
class Case:
    name: str
    sources: dict
    outputs: dict
    build: Callable  # build(ptr) -> abi.HostPlan
    float_outputs: bool = True
    meta: dict = field(default_factory=dict)


def _u8(rng, *shape):
    return rng.integers(0, 256, shape, dtype=np.uint8)


def padded_u8_image(rng, h, w, pitch):
    """(h, w, 3) view with a row pitch of `pitch` bytes; the padding holds 0xEE."""
    buf = np.full((h, pitch), 0xEE, np.uint8)
    img = buf[:, :w * 3].reshape(h, w, 3)
    img[...] = _u8(rng, h, w, 3)
    return buf, img


def elementwise_case(name, seed, w, h, ops, src_fmt=abi.SRC_U8X3, dst_fmt=abi.DST_F32X3_PACKED, src_pitch=None,
                     dst_pitch=None, crop=None):
    rng = np.random.default_rng(seed)
    spx = 3 if src_fmt == abi.SRC_U8X3 else 12
    dpx = 3 if dst_fmt == abi.DST_U8X3_PACKED else 12   # float3, int3 and uint3 are twelve bytes
    sp = src_pitch or w * spx
    ow, oh = (crop[2], crop[3]) if crop else (w, h)
    dp = dst_pitch or ow * dpx
    src = np.full((h, sp), 0xEE, np.uint8)
    if src_fmt == abi.SRC_U8X3:
        src[:, :w * 3] = _u8(rng, h, w * 3)
    else:
        src[:, :w * 12] = rng.random((h, w * 3), dtype=np.float32).view(np.uint8)
    out = np.zeros((oh, dp), np.uint8)

    def build(ptr):
        return chains.elementwise(ops, src=ptr("src"), dst=ptr("out"), width=w, height=h, src_format=src_fmt,
                                  dst_format=dst_fmt, src_pitch=sp, dst_pitch=dp, crop=crop)

    return Case(name, {"src": src}, {"out": out}, build, float_outputs=dst_fmt != abi.DST_U8X3_PACKED,
                meta=dict(w=ow, h=oh, dpx=dpx, dst_pitch=dp))


def crop_resize_case(name, seed, n_frames, fw, fh, n_planes, dw, dh, planar, post_ops, rects=None, lo=4, hi=200,
                     mode=abi.RESIZE_PRESERVE_AR, background=(0.0, 0.0, 0.0), src_pitch=None):
    rng = np.random.default_rng(seed)
    sp = src_pitch or fw * 3
    sources = {}
    for i in range(n_frames):
        buf = np.full((fh, sp), 0xEE, np.uint8)
        buf[:, :fw * 3] = _u8(rng, fh, fw * 3)
        sources[f"frame{i}"] = buf
    if rects is None:
        rects = chains.random_rects(rng, n_planes, fw, fh, lo=lo, hi=hi)
    rects = np.asarray(rects, np.int32)
    frame_index = [i % n_frames for i in range(n_planes)]
    out = np.zeros((n_planes, 3, dh, dw) if planar else (n_planes, dh, dw, 3), np.float32)

    def build(ptr):
        return chains.crop_resize_batch(frame_ptrs=[ptr(f"frame{i}") for i in range(n_frames)], frame_index=frame_index,
                                        rects=rects, src_width=fw, src_height=fh, src_pitch=sp, dst=ptr("out"),
                                        dst_width=dw, dst_height=dh, post_ops=post_ops, planar=planar, mode=mode,
                                        background=background)

    return Case(name, sources, {"out": out}, build, meta=dict(rects=rects, frame_index=frame_index))


def nv12_case(name, seed, n_frames, w, h, dw, dh, pitch=None, mode=abi.RESIZE_IGNORE_AR, background=(0.0, 0.0, 0.0),
              crops=None, src_format=abi.SRC_NV12, conversion=abi.OP_YUV_TO_RGB_BT709_FULL):
    rng = np.random.default_rng(seed)
    pitch = pitch or w
    sources = {}
    for i in range(n_frames):
        buf = np.full((h + h // 2, pitch), 0xEE, np.uint8)
        buf[:, :w] = _u8(rng, h + h // 2, w)
        sources[f"frame{i}"] = buf
    out = np.zeros((n_frames, dh, dw, 3), np.float32)

    def build(ptr):
        return chains.nv12_resize_batch(frame_ptrs=[ptr(f"frame{i}") for i in range(n_frames)], width=w, height=h,
                                        pitch=pitch, dst=ptr("out"), dst_width=dw, dst_height=dh, mode=mode,
                                        background=background, crops=crops, src_format=src_format, conversion=conversion)

    return Case(name, sources, {"out": out}, build)


def default_planes_case(name, seed, w, h, mode, dst_fmt, n=5, used=3):
    """A partly filled batch: planes at or beyond `used` carry FKB_PLANE_DEFAULT_VALUE (and no image at all)."""
    rng = np.random.default_rng(seed)
    sources = {f"img{i}": _u8(rng, h, w * 3) for i in range(used)}
    dw, dh = (w, h) if mode == abi.RESIZE_NONE else (40, 28)
    dpx = 3 if dst_fmt == abi.DST_U8X3_PACKED else 12
    out = np.zeros((n, dh, dw * dpx), np.uint8)
    ops = [op(abi.OP_CAST_F32), op(abi.OP_MUL, (1.5, 0.25, 2.0))] + ([op(abi.OP_SATURATE_CAST_U8)] if dpx == 3 else [])

    def build(ptr):
        plan = abi.HostPlan()
        seq = plan.add_sequence(abi.SRC_U8X3, dst_fmt, mode, ops, n_pre_ops=1 if mode != abi.RESIZE_NONE else 0,
                                background=(7.0, 200.0, 33.0))
        for i in range(n):
            plan.add_plane(src=ptr(f"img{i}") if i < used else 0, src_width=w, src_height=h, src_pitch=w * 3,
                           dst=ptr("out") + i * dh * dw * dpx, dst_width=dw, dst_height=dh, dst_pitch=dw * dpx, sequence=seq,
                           flags=0 if i < used else abi.PLANE_DEFAULT_VALUE)
        return plan

    return Case(name, sources, {"out": out}, build, float_outputs=dpx == 12)


def yuv_layout_image(rng, fmt, w, h, pitch_pad=0):
    """A random image of one of the YUV layouts beyond NV12 / NV21 as a 2-D array of its words, rows one pitch apart
    (pitch a multiple of 8 bytes).  The 10-bit layouts carry their value in the top ten bits and noise in the low six,
    which the conversion must shift away."""
    pairs = (w + 1) // 2
    if fmt == abi.SRC_UYVY:
        row_words, rows, dtype = 4 * pairs, h, np.uint8
    elif fmt == abi.SRC_Y210:
        row_words, rows, dtype = 4 * pairs, h, np.uint16
    elif fmt == abi.SRC_P010:
        row_words, rows, dtype = 2 * pairs, h + (h + 1) // 2, np.uint16
    else:  # P210
        row_words, rows, dtype = 2 * pairs, 2 * h, np.uint16
    item = np.dtype(dtype).itemsize
    pitch_words = (-(-(row_words * item + pitch_pad) // 8) * 8) // item
    img = rng.integers(0, 256 if dtype == np.uint8 else 65536, (rows, pitch_words), dtype=dtype)
    return img


YUV_CONVERSIONS = (abi.OP_YUV_TO_RGB_BT709_FULL, abi.OP_YUV_TO_RGB_BT601_FULL, abi.OP_YUV_TO_RGB_BT2020_FULL)


def yuv_layout_case(name, seed, fmt, primitives, w, h, dw, dh, post_ops, mode=None, crop=None, pitch_pad=0, n=2):
    """ReadYUV<P010 | P210 | Y210 | UYVY> -> ConvertYUVToRGB -> [Resize] -> post_ops -> float3, a small batch."""
    rng = np.random.default_rng(seed)
    sources = {f"img{i}": yuv_layout_image(rng, fmt, w, h, pitch_pad) for i in range(n)}
    pitch = sources["img0"].strides[0]
    resize = (dw, dh) != ((crop[2], crop[3]) if crop else (w, h))
    mode = mode if mode is not None else (abi.RESIZE_IGNORE_AR if resize else abi.RESIZE_NONE)
    out = np.zeros((n, dh, dw * 12), np.uint8)

    def build(ptr):
        plan = abi.HostPlan()
        seq = plan.add_sequence(fmt, abi.DST_F32X3_PACKED, mode, [op(YUV_CONVERSIONS[primitives])] + list(post_ops), n_pre_ops=1,
                                background=(5.0, 6.0, 7.0))
        for i in range(n):
            plan.add_plane(src=ptr(f"img{i}"), src_width=w, src_height=h, src_pitch=pitch, crop=crop, dst=ptr("out") + i * dh * dw * 12,
                           dst_width=dw, dst_height=dh, dst_pitch=dw * 12, sequence=seq)
        return plan

    return Case(name, sources, {"out": out}, build, float_outputs=True)


def readback_case(name, seed, w, h, dw, dh, mode, dst_fmt=abi.DST_F32X3_PACKED, ops=(), n_pre=0, crop=None, border=0,
                  border_value=(0.0, 0.0, 0.0), deinterlace=0, transform=None, src_fmt=abi.SRC_U8X3, n=2):
    """BorderReader / Deinterlace / Warping chains on a small batch of images (the one-pixel-per-thread body)."""
    rng = np.random.default_rng(seed)
    if src_fmt == abi.SRC_U8X3:
        sources = {f"img{i}": _u8(rng, h, w * 3) for i in range(n)}
        spx = 3
    else:
        sources = {f"img{i}": (rng.random((h, w * 3), dtype=np.float32) * 255).astype(np.float32) for i in range(n)}
        spx = 12
    dpx = 3 if dst_fmt == abi.DST_U8X3_PACKED else 12
    out = np.zeros((n, dh, dw * dpx), np.uint8)

    def build(ptr):
        plan = abi.HostPlan()
        seq = plan.add_sequence(src_fmt, dst_fmt, mode, list(ops), n_pre_ops=n_pre, border_mode=border, border_value=border_value,
                                deinterlace=deinterlace, transform=transform, background=(5.0, 6.0, 7.0))
        for i in range(n):
            plan.add_plane(src=ptr(f"img{i}"), src_width=w, src_height=h, src_pitch=w * spx, crop=crop, dst=ptr("out") + i * dh * dw * dpx,
                           dst_width=dw, dst_height=dh, dst_pitch=dw * dpx, sequence=seq)
        return plan

    return Case(name, sources, {"out": out}, build, float_outputs=dpx == 12)


def resize_any_case(name, seed, src_fmt, dst_fmt, w, h, dw, dh, pre_ops, post_ops, mode=abi.RESIZE_IGNORE_AR):
    """One image -> pre_ops on every tap -> Resize -> post_ops -> receiver, any source / destination format."""
    rng = np.random.default_rng(seed)
    if src_fmt == abi.SRC_U8X3:
        src = _u8(rng, h, w * 3)
        sp = w * 3
    else:
        src = (rng.random((h, w * 3), dtype=np.float32) * 255).astype(np.float32)
        sp = w * 12
    planar = dst_fmt == abi.DST_F32_PLANAR3
    dpx = {abi.DST_F32X3_PACKED: 12, abi.DST_U8X3_PACKED: 3, abi.DST_F32_PLANAR3: 4, abi.DST_I32X3_PACKED: 12,
           abi.DST_U32X3_PACKED: 12}[dst_fmt]
    out = np.zeros((3 * dh if planar else dh, dw * dpx), np.uint8)

    def build(ptr):
        plan = abi.HostPlan()
        seq = plan.add_sequence(src_fmt, dst_fmt, mode, list(pre_ops) + list(post_ops), n_pre_ops=len(pre_ops))
        plan.add_plane(src=ptr("src"), src_width=w, src_height=h, src_pitch=sp, dst=ptr("out"), dst_width=dw, dst_height=dh,
                       dst_pitch=dw * dpx, dst_channel_stride=dh * dw * 4 if planar else 0, sequence=seq)
        return plan

    return Case(name, {"src": src}, {"out": out}, build, float_outputs=dst_fmt != abi.DST_U8X3_PACKED)


def divergent_case(name, seed, w, h, rw, rh, per_group):
    rng = np.random.default_rng(seed)
    sources = {f"img{i}": _u8(rng, h, w * 3) for i in range(4 * per_group)}
    outputs = {
        "g0": np.zeros((per_group, h, w, 3), np.float32),
        "g1": np.zeros((per_group, h, w, 3), np.float32),
        "g2": np.zeros((per_group, h, w, 3), np.uint8),
        "g3": np.zeros((per_group, rh, rw, 3), np.float32),
    }

    def build(ptr):
        return chains.divergent_four_groups(src_ptrs=[ptr(f"img{i}") for i in range(4 * per_group)], width=w, height=h,
                                            dst_ptrs=[ptr(f"g{g}") for g in range(4)], resize_to=(rw, rh),
                                            per_group=per_group)

    return Case(name, sources, outputs, build)


def small_cases():
    """Cases the checker finishes in well under a second each."""
    c1 = chains.cast_mul_sub_div_ops()
    g3 = [op(abi.OP_SWAP_RB), op(abi.OP_CAST_F32), op(abi.OP_MUL, 1.4), op(abi.OP_SATURATE_CAST_U8)]
    cases = [
        elementwise_case("c1_dense_aligned", 11, 64, 33, c1),
        elementwise_case("c1_odd_width", 12, 53, 37, c1),                      # rows not 4-byte multiples: generic
        elementwise_case("c1_1x1", 13, 1, 1, c1),
        elementwise_case("c1_1xN", 14, 1, 19, c1),
        elementwise_case("c1_Nx1", 15, 1023, 1, c1),
        elementwise_case("c1_pitched", 16, 100, 21, c1, src_pitch=304, dst_pitch=1216),  # row segments + tails
        elementwise_case("c1_pitched_unaligned", 17, 100, 21, c1, src_pitch=301),
        elementwise_case("c1_crop", 18, 96, 40, c1, crop=(8, 3, 64, 20)),
        elementwise_case("c1_crop_unaligned", 19, 96, 40, c1, crop=(7, 3, 61, 20)),
        elementwise_case("c1_tail", 20, 1027, 3, c1),                          # dense, pixel count not multiple of 4
        elementwise_case("c5a_n1", 21, 40, 30, chains.addmul_ops(1), src_fmt=abi.SRC_F32X3),
        elementwise_case("c5a_n16", 22, 40, 30, chains.addmul_ops(16), src_fmt=abi.SRC_F32X3),
        elementwise_case("c5a_n64", 23, 40, 30, chains.addmul_ops(64), src_fmt=abi.SRC_F32X3),
        elementwise_case("c5a_n256", 24, 41, 31, chains.addmul_ops(256), src_fmt=abi.SRC_F32X3),
        # repeated operations run as counted loops on the device (the reference's StaticLoop benchmark shape)
        elementwise_case("repeat_mul_then_sub", 29, 40, 30,
                         [op(abi.OP_MUL, (1.01, 0.99, 1.002))] * 21 + [op(abi.OP_SUB, (0.1, 0.2, 0.3))] * 7 +
                         [op(abi.OP_ADD, 0.001), op(abi.OP_MUL, 1.0001)] * 5 + [op(abi.OP_DIV, 3.0), op(abi.OP_MUL, 2.0)],
                         src_fmt=abi.SRC_F32X3),
        elementwise_case("repeat_after_cast_u8", 30, 53, 37,
                         [op(abi.OP_CAST_F32)] + [op(abi.OP_SUB, 1.5), op(abi.OP_ADD, 0.25)] * 9 + [op(abi.OP_MUL, 0.5)] * 6),
        elementwise_case("g3_saturate_u8", 25, 64, 32, g3, dst_fmt=abi.DST_U8X3_PACKED),
        elementwise_case("g3_saturate_u8_odd", 26, 53, 37, g3, dst_fmt=abi.DST_U8X3_PACKED),
        elementwise_case("copy_u8", 27, 300, 20, [], dst_fmt=abi.DST_U8X3_PACKED),
        elementwise_case("copy_f32", 28, 32, 20, [], src_fmt=abi.SRC_F32X3),
        crop_resize_case("c2_readme", 31, 1, 384, 216, 5, 60, 60, False, chains.readme_ops(), rects=chains.README_RECTS),
        crop_resize_case("c2_readme_ignore_ar", 32, 1, 384, 216, 5, 60, 60, False, chains.readme_ops(),
                         rects=chains.README_RECTS, mode=abi.RESIZE_IGNORE_AR),
        crop_resize_case("c2_background", 33, 2, 200, 120, 7, 40, 28, False, chains.readme_ops(),
                         background=(10.0, 20.0, 30.0)),
        crop_resize_case("c3_small", 34, 3, 480, 270, 37, 48, 32, True, chains.normalize_ops()),
        crop_resize_case("c3_odd_dst", 35, 2, 320, 200, 9, 45, 31, True, chains.normalize_ops()),  # generic path
        crop_resize_case("c3_edges", 36, 1, 64, 48, 6, 32, 32, True, chains.normalize_ops(),
                         rects=[(0, 0, 64, 48), (0, 0, 1, 1), (63, 47, 1, 1), (0, 47, 64, 1), (63, 0, 1, 48),
                                (10, 10, 2, 2)]),
        crop_resize_case("c3_upscale", 37, 1, 64, 48, 4, 224, 224, True, chains.normalize_ops(), lo=4, hi=24),
        crop_resize_case("c3_pitched_src", 38, 2, 100, 60, 5, 48, 32, True, chains.normalize_ops(), src_pitch=333),
        # frames whose pitch and base are 16-byte aligned take the shared-memory staged path
        crop_resize_case("c3_staged_borders", 61, 1, 512, 300, 6, 224, 224, True, chains.normalize_ops(),
                         rects=[(0, 0, 512, 300), (511, 299, 1, 1), (500, 0, 12, 300), (0, 290, 512, 10), (3, 5, 509, 295),
                                (255, 100, 2, 200)]),
        crop_resize_case("c3_staged_steep", 62, 2, 1024, 600, 5, 64, 64, True, chains.normalize_ops(),
                         rects=[(0, 0, 1024, 600), (1, 1, 1023, 599), (17, 33, 1000, 64), (100, 0, 64, 600), (0, 0, 1024, 8)]),
        crop_resize_case("c3_staged_upscale", 63, 1, 64, 64, 5, 224, 224, True, chains.normalize_ops(),
                         rects=[(0, 0, 3, 3), (61, 61, 3, 3), (5, 0, 7, 64), (0, 5, 64, 7), (31, 31, 2, 2)]),
        crop_resize_case("c2_staged_packed_bg", 64, 2, 208, 120, 9, 60, 44, False, chains.readme_ops(),
                         background=(10.0, 20.0, 30.0)),
        crop_resize_case("c2_staged_ignore_ar_odd_groups", 65, 1, 208, 120, 4, 36, 20, False, chains.readme_ops(),
                         mode=abi.RESIZE_IGNORE_AR),
        # regions wider than 512 columns: the staged body cuts them into column tiles
        crop_resize_case("wide_planar_preserve_ar_bg", 66, 1, 1600, 96, 4, 1320, 40, True, chains.normalize_ops(),
                         rects=[(0, 0, 1600, 40), (3, 1, 1597, 95), (37, 8, 901, 20), (800, 0, 640, 33)],
                         background=(7.0, 9.0, 11.0)),
        crop_resize_case("wide_packed_ignore_ar", 67, 2, 2048, 64, 3, 1024, 24, False, chains.readme_ops(),
                         rects=[(0, 0, 2048, 48), (5, 3, 2043, 61), (16, 0, 520, 10)], mode=abi.RESIZE_IGNORE_AR),
        crop_resize_case("wide_packed_upscale", 68, 1, 208, 32, 2, 2052, 12, False, chains.readme_ops(),
                         rects=[(1, 1, 203, 9), (0, 0, 208, 32)], mode=abi.RESIZE_IGNORE_AR),
        # PRESERVE_AR targets that round to zero columns or rows: the whole plane is background
        crop_resize_case("c3_empty_regions", 69, 1, 1024, 1024, 5, 32, 32, True, chains.normalize_ops(),
                         rects=[(0, 0, 2, 130), (0, 0, 1, 1000), (0, 0, 1000, 1), (10, 10, 100, 80), (5, 7, 3, 900)],
                         background=(3.0, 7.0, 11.0)),
        crop_resize_case("c3_all_empty_regions", 70, 1, 1024, 1024, 2, 224, 224, True, chains.normalize_ops(),
                         rects=[(0, 0, 2, 1000), (0, 0, 1000, 2)], background=(3.0, 7.0, 11.0)),
        crop_resize_case("c2_empty_regions_packed", 74, 2, 1024, 1024, 4, 60, 60, False, chains.readme_ops(),
                         rects=[(0, 0, 1, 1024), (0, 0, 34, 25), (0, 0, 1024, 1), (40, 40, 12, 11)], background=(1.0, 2.0, 3.0)),
        crop_resize_case("c3_empty_regions_odd_dst", 75, 1, 300, 700, 3, 45, 31, True, chains.normalize_ops(),
                         rects=[(0, 0, 1, 700), (0, 0, 300, 2), (3, 3, 100, 100)], background=(3.0, 7.0, 11.0)),
        nv12_case("c4_empty_regions", 48, 3, 1024, 256, 32, 32, mode=abi.RESIZE_PRESERVE_AR, background=(16.0, 128.0, 240.0),
                  crops=[(0, 0, 2, 130), (0, 0, 1000, 2), (0, 0, 64, 64)]),
        nv12_case("c4_exact3", 41, 3, 96, 54, 32, 18),
        nv12_case("c4_fractional", 42, 2, 96, 54, 40, 22),
        nv12_case("c4_pitched", 43, 2, 98, 54, 36, 20, pitch=128),
        nv12_case("c4_odd_dst", 44, 2, 96, 54, 37, 21),
        nv12_case("c4_preserve_ar_bg", 45, 2, 96, 54, 48, 48, mode=abi.RESIZE_PRESERVE_AR, background=(16.0, 128.0, 240.0)),
        nv12_case("c4_crops", 46, 3, 128, 64, 40, 24, crops=[(1, 1, 101, 33), (64, 31, 64, 33), (0, 0, 2, 2)]),
        nv12_case("c4_upscale_tiles", 47, 1, 32, 16, 1280, 40),                 # three column tiles, every tap fractional
        # chains that only the one-pixel-per-thread body takes
        resize_any_case("float_source_resize", 71, abi.SRC_F32X3, abi.DST_F32X3_PACKED, 40, 30, 24, 18,
                        [op(abi.OP_MUL, 2.0)], [op(abi.OP_ADD, 0.5)]),
        resize_any_case("resize_then_saturate_u8", 72, abi.SRC_U8X3, abi.DST_U8X3_PACKED, 64, 48, 32, 20,
                        [op(abi.OP_CAST_F32)], [op(abi.OP_MUL, 1.1), op(abi.OP_SATURATE_CAST_U8)]),
        resize_any_case("planar_ignore_ar", 73, abi.SRC_U8X3, abi.DST_F32_PLANAR3, 64, 48, 40, 28, [], chains.normalize_ops()),
        # the other aspect-ratio modes; NV21 and the bt601 / bt2020 matrices; planes of a partly filled batch
        crop_resize_case("ar_rn_even", 84, 2, 480, 270, 21, 48, 32, True, chains.normalize_ops(), mode=abi.RESIZE_PRESERVE_AR_RN_EVEN,
                         background=(3.0, 5.0, 7.0)),
        crop_resize_case("ar_left_packed", 85, 2, 480, 270, 21, 60, 44, False, chains.readme_ops(), mode=abi.RESIZE_PRESERVE_AR_LEFT,
                         background=(3.0, 5.0, 7.0)),
        crop_resize_case("ar_left_odd_dst", 86, 1, 300, 200, 7, 45, 31, True, chains.normalize_ops(), mode=abi.RESIZE_PRESERVE_AR_LEFT),
        nv12_case("nv21_bt709", 87, 2, 96, 54, 40, 22, src_format=abi.SRC_NV21),
        nv12_case("nv21_bt601_exact3", 88, 2, 96, 54, 32, 18, src_format=abi.SRC_NV21, conversion=abi.OP_YUV_TO_RGB_BT601_FULL),
        nv12_case("nv12_bt2020_odd_dst", 89, 2, 96, 54, 37, 21, conversion=abi.OP_YUV_TO_RGB_BT2020_FULL),
        nv12_case("nv12_bt601_pitched_preserve_ar", 90, 2, 98, 54, 48, 48, pitch=128, mode=abi.RESIZE_PRESERVE_AR_LEFT,
                  background=(16.0, 128.0, 240.0), conversion=abi.OP_YUV_TO_RGB_BT601_FULL),
        default_planes_case("default_planes_flat", 91, 64, 32, abi.RESIZE_NONE, abi.DST_F32X3_PACKED),
        default_planes_case("default_planes_flat_u8", 92, 53, 37, abi.RESIZE_NONE, abi.DST_U8X3_PACKED),
        default_planes_case("default_planes_resize", 93, 64, 48, abi.RESIZE_PRESERVE_AR, abi.DST_F32X3_PACKED),
        # YUV layouts beyond NV12 / NV21: read and converted by the one-pixel-per-thread body
        *[yuv_layout_case(f"yuv_layout{f}_primitives{p}", 130 + 3 * f + p, f, p, 38, 22, 38, 22, [op(abi.OP_MUL, (1.0, 0.5, 2.0))])
          for f in (abi.SRC_P010, abi.SRC_P210, abi.SRC_Y210, abi.SRC_UYVY) for p in (0, 1, 2)],
        *[yuv_layout_case(f"yuv_layout{f}_resize", 160 + f, f, f % 3, 64, 36, 28, 20, [op(abi.OP_DIV, 255.0)], pitch_pad=24)
          for f in (abi.SRC_P010, abi.SRC_P210, abi.SRC_Y210, abi.SRC_UYVY)],
        yuv_layout_case("yuv_p010_crop_preserve_ar_odd", 170, abi.SRC_P010, 0, 41, 27, 36, 24, [op(abi.OP_SUB, 3.0)], mode=abi.RESIZE_PRESERVE_AR,
                        crop=(3, 5, 31, 17)),
        yuv_layout_case("yuv_uyvy_crop_odd_origin", 171, abi.SRC_UYVY, 1, 40, 24, 21, 13, [], crop=(7, 3, 21, 13)),
        # BorderReader under a padded crop, Warping, Deinterlace
        *[readback_case(f"border{b}_padded_crop_u8", 100 + b, 40, 24, 60, 37, abi.RESIZE_NONE, dst_fmt=abi.DST_U8X3_PACKED,
                        crop=(-7, -5, 60, 37), border=b, border_value=(9.0, 99.0, 199.0)) for b in range(1, 6)],
        *[readback_case(f"border{b}_padded_crop_resize", 110 + b, 40, 24, 36, 28, abi.RESIZE_PRESERVE_AR, crop=(-45, -30, 130, 90),
                        border=b, border_value=(9.0, 99.0, 199.0), ops=[op(abi.OP_CAST_F32), op(abi.OP_MUL, 0.5)], n_pre=1)
          for b in range(1, 6)],
        readback_case("border_constant_float_source", 116, 33, 21, 50, 30, abi.RESIZE_NONE, crop=(-9, -4, 50, 30), border=1,
                      border_value=(0.5, 1.5, 2.5), src_fmt=abi.SRC_F32X3, ops=[op(abi.OP_ADD, 1.0)]),
        readback_case("warp_affine", 117, 40, 24, 48, 32, abi.GEOMETRY_WARP_AFFINE, ops=[op(abi.OP_MUL, (1.0, 0.5, 2.0))],
                      transform=(0.8, 0.25, -3.0, -0.2, 0.7, 2.5, 0, 0, 1)),
        readback_case("warp_perspective_crop", 118, 64, 48, 45, 31, abi.GEOMETRY_WARP_PERSPECTIVE, crop=(8, 6, 40, 30),
                      ops=[op(abi.OP_CAST_F32), op(abi.OP_SUB, 3.0)], n_pre=1, transform=(0.9, 0.1, -2.0, 0.05, 0.8, 1.0, 0.002, 0.001, 1.0)),
        *[readback_case(f"deinterlace{k}", 120 + k, 40, 24, 40, 24, abi.RESIZE_NONE, ops=[op(abi.OP_MUL, (1.0, 0.5, 2.0))],
                        deinterlace=k) for k in (1, 2, 3)],
        readback_case("deinterlace_blend_float_then_resize", 124, 40, 24, 28, 20, abi.RESIZE_IGNORE_AR, deinterlace=1,
                      src_fmt=abi.SRC_F32X3, ops=[op(abi.OP_MUL, 0.25)]),
        # Cast<float3,int3> / Cast<float3,uint3> closing a chain (truncation toward zero)
        elementwise_case("cast_int3_after_arithmetic", 81, 64, 33, [op(abi.OP_CAST_F32), op(abi.OP_MUL, (1.37, 0.5, 2.25)),
                                                                    op(abi.OP_SUB, (100.5, 3.25, 7.0)), op(abi.OP_CAST_I32)],
                         dst_fmt=abi.DST_I32X3_PACKED),
        elementwise_case("cast_uint3_odd_width", 82, 53, 37, [op(abi.OP_CAST_F32), op(abi.OP_MUL, (1.37, 300.5, 2.25)),
                                                              op(abi.OP_CAST_U32)], dst_fmt=abi.DST_U32X3_PACKED),
        resize_any_case("resize_then_cast_uint3", 83, abi.SRC_U8X3, abi.DST_U32X3_PACKED, 64, 48, 32, 20,
                        [op(abi.OP_CAST_F32)], [op(abi.OP_MUL, 3.7), op(abi.OP_CAST_U32)]),
        divergent_case("c5b_small", 51, 64, 36, 32, 18, 3),
        divergent_case("c5b_odd", 52, 50, 30, 25, 15, 2),
    ]
    return cases


def run_on_host(case: Case, port, host_branch=False):
    """Runs the checker in place on the case's host arrays; returns the outputs dict."""
    arrays = {**case.sources, **case.outputs}
    for a in case.outputs.values():
        a[...] = 0
    plan = case.build(lambda name: arrays[name].ctypes.data)
    port.run(plan, host_branch=host_branch)
    return case.outputs


def cuda_copy_to_host(host: np.ndarray, device_ptr: int) -> None:
    """Synchronous device-to-host copy from a raw device pointer (memory the library allocated)."""
    from cuda.bindings import runtime
    (err,) = runtime.cudaMemcpy(host.ctypes.data, int(device_ptr), host.nbytes, runtime.cudaMemcpyKind.cudaMemcpyDeviceToHost)
    assert int(err) == 0, err


def bits(a: np.ndarray) -> np.ndarray:
    return a.view(np.uint32) if a.dtype == np.float32 else a
