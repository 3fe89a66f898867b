"""Pins the plain-C checker against golden vectors produced by the reference's own headers
(tests/golden/make_golden.py) and, where oracle/_ref is present, against that build directly."""
from pathlib import Path

import numpy as np
import pytest

from fusedkernellibrary_b200 import abi, chains
from fusedkernellibrary_b200.abi import op
from oracle import reference as ref
from tests import cases as tc

GOLD = Path(__file__).resolve().parent / "golden"


def _same(a, b):
    return np.array_equal(tc.bits(np.ascontiguousarray(a)), tc.bits(np.ascontiguousarray(b)))


def _elementwise(port, src, ops, dst_fmt=abi.DST_F32X3_PACKED, src_fmt=abi.SRC_U8X3):
    h, w, _ = src.shape
    src = np.ascontiguousarray(src)
    out = np.zeros((h, w, 3), np.uint8 if dst_fmt == abi.DST_U8X3_PACKED else np.float32)   # int3 / uint3: same 12 bytes
    plan = chains.elementwise(ops, src=src.ctypes.data, dst=out.ctypes.data, width=w, height=h, src_format=src_fmt,
                              dst_format=dst_fmt)
    port.run(plan)
    return out


def test_elementwise_chains(oracle_port):
    g = np.load(GOLD / "elementwise_u8.npz")
    src = g["src"]
    assert _same(_elementwise(oracle_port, src, chains.cast_mul_sub_div_ops()), g["cast_mul_sub_div"])
    assert _same(_elementwise(oracle_port, src, [op(abi.OP_CAST_F32), op(abi.OP_MUL, 1.4), op(abi.OP_SUB, 0.5)]),
                 g["cast_mul_sub"])
    assert _same(_elementwise(oracle_port, src, [op(abi.OP_CAST_F32), op(abi.OP_ADD, 0.5), op(abi.OP_DIV, 255.0)]),
                 g["cast_add_div"])
    assert _same(_elementwise(oracle_port, src, [op(abi.OP_SWAP_RB), op(abi.OP_CAST_F32), op(abi.OP_MUL, 1.4),
                                                 op(abi.OP_SATURATE_CAST_U8)], dst_fmt=abi.DST_U8X3_PACKED),
                 g["bgr_cast_mul_saturate"])
    # known answer stated by hand: (56*1.4 - 0.5)/255 in binary32
    v = np.float32(np.float32(np.float32(56) * np.float32(1.4)) - np.float32(0.5)) / np.float32(255)
    one = np.full((1, 1, 3), 56, np.uint8)
    assert _elementwise(oracle_port, one, chains.cast_mul_sub_div_ops())[0, 0, 0] == v


def test_integer_casts_close_a_chain(oracle_port):
    """Cast<float3,int3> and Cast<float3,uint3> (cast_base.h:20-30): truncation toward zero, values stored as
    12-byte integer pixels."""
    g = np.load(GOLD / "int_casts.npz")
    src = np.ascontiguousarray(g["src"])
    got = _elementwise(oracle_port, src, [op(abi.OP_CAST_F32), op(abi.OP_MUL, (1.37, 0.5, 2.25)), op(abi.OP_SUB, (100.5, 3.25, 7.0)),
                                          op(abi.OP_CAST_I32)], dst_fmt=abi.DST_I32X3_PACKED)
    assert np.array_equal(got.view(np.int32), g["cast_mul_sub_cast_int3"])
    assert (g["cast_mul_sub_cast_int3"] < 0).any() and (g["cast_mul_sub_cast_int3"] > 0).any()
    h, w, _ = src.shape
    out = np.zeros((20, 30, 3), np.uint32)
    plan = abi.HostPlan()
    s = plan.add_sequence(abi.SRC_U8X3, abi.DST_U32X3_PACKED, abi.RESIZE_IGNORE_AR,
                          [op(abi.OP_CAST_F32), op(abi.OP_MUL, (3.7, 1.0, 0.01)), op(abi.OP_CAST_U32)], n_pre_ops=1)
    plan.add_plane(src=src.ctypes.data, src_width=w, src_height=h, src_pitch=w * 3, dst=out.ctypes.data, dst_width=30,
                   dst_height=20, dst_pitch=360, sequence=s)
    oracle_port.run(plan)
    assert np.array_equal(out, g["cast_resize_mul_cast_uint3_30x20"])


def _cast_resize(port, src, dw, dh, host_branch=False):
    h, w, _ = src.shape
    src = np.ascontiguousarray(src)
    out = np.zeros((dh, dw, 3), np.float32)
    plan = abi.HostPlan()
    s = plan.add_sequence(abi.SRC_U8X3, abi.DST_F32X3_PACKED, abi.RESIZE_IGNORE_AR, [op(abi.OP_CAST_F32)], n_pre_ops=1)
    plan.add_plane(src=src.ctypes.data, src_width=w, src_height=h, src_pitch=w * 3, dst=out.ctypes.data, dst_width=dw,
                   dst_height=dh, dst_pitch=dw * 12, sequence=s)
    port.run(plan, host_branch=host_branch)
    return out


def test_cast_then_resize(oracle_port):
    g = np.load(GOLD / "elementwise_u8.npz")
    assert _same(_cast_resize(oracle_port, g["src"], 30, 20), g["cast_resize_30x20"])


def test_addmul_chains(oracle_port):
    g = np.load(GOLD / "addmul_chain.npz")
    for n in (1, 2, 3, 16, 64, 256):
        got = _elementwise(oracle_port, g["src"], chains.addmul_ops(n), src_fmt=abi.SRC_F32X3)
        assert _same(got, g[f"n{n}"]), n


def _readme(port, frame, rects, mode=abi.RESIZE_PRESERVE_AR, host_branch=False):
    frame = np.ascontiguousarray(frame)
    h, w, _ = frame.shape
    out = np.zeros((len(rects), 60, 60, 3), np.float32)
    plan = chains.crop_resize_batch(frame_ptrs=[frame.ctypes.data], frame_index=[0] * len(rects), rects=rects,
                                    src_width=w, src_height=h, src_pitch=w * 3, dst=out.ctypes.data, dst_width=60,
                                    dst_height=60, post_ops=chains.readme_ops(), planar=False, mode=mode)
    port.run(plan, host_branch=host_branch)
    return out


def test_readme_chain(oracle_port):
    g = np.load(GOLD / "readme_crop_resize.npz")
    assert _same(_readme(oracle_port, g["frame"], g["rects"]), g["out"])
    assert _same(_readme(oracle_port, g["frame"], g["rects"], mode=abi.RESIZE_IGNORE_AR), g["out_ignore_ar"])


def test_literal_host_branch_is_reproduced_and_differs(oracle_port):
    """The reference's host branch takes the row tap from the column coordinate
    (interpolation.h:70).  The checker can reproduce it, and it is NOT the parity target."""
    g = np.load(GOLD / "readme_crop_resize.npz")
    lit = _readme(oracle_port, g["frame"], g["rects"], host_branch=True)
    assert _same(lit, g["literal_out"])
    assert np.abs(g["literal_out"] - g["out"]).max() > 1e-2


def test_batched_crop_resize_norm(oracle_port):
    g = np.load(GOLD / "batched_crop_resize_norm.npz")
    frames = [np.ascontiguousarray(f) for f in g["frames"]]
    n = len(g["rects"])
    out = np.zeros((n, 3, 32, 48), np.float32)
    plan = chains.crop_resize_batch(frame_ptrs=[f.ctypes.data for f in frames], frame_index=list(g["frame_index"]),
                                    rects=g["rects"], src_width=240, src_height=135, src_pitch=720,
                                    dst=out.ctypes.data, dst_width=48, dst_height=32,
                                    post_ops=chains.normalize_ops(), planar=True)
    oracle_port.run(plan)
    assert _same(out, g["out"])


def test_nv12_resize(oracle_port):
    g = np.load(GOLD / "nv12_resize.npz")
    frames = [np.ascontiguousarray(f) for f in g["frames"]]
    for (dw, dh) in ((32, 18), (40, 22)):
        out = np.zeros((len(frames), dh, dw, 3), np.float32)
        plan = chains.nv12_resize_batch(frame_ptrs=[f.ctypes.data for f in frames], width=96, height=54, pitch=96,
                                        dst=out.ctypes.data, dst_width=dw, dst_height=dh)
        oracle_port.run(plan)
        assert _same(out, g[f"out_{dw}x{dh}"])
    # no saturation on the float path: values leave [0, 1] (color_conversion.h:276-281)
    assert g["out_32x18"].min() < 0 and g["out_32x18"].max() > 1


def test_resize_params_table(oracle_port):
    g = np.load(GOLD / "resize_params.npz")
    for (sw, sh, dw, dh), res in zip(g["query"], g["result"]):
        for ar, mode in ((0, abi.RESIZE_IGNORE_AR), (1, abi.RESIZE_PRESERVE_AR)):
            rp = oracle_port.derive_resize(int(sw), int(sh), int(dw), int(dh), mode)
            got = [int(np.float32(rp.fx).view(np.uint32)), int(np.float32(rp.fy).view(np.uint32))]
            assert got == list(res[ar][:2])
            if ar:
                assert [rp.x1, rp.y1, rp.x2, rp.y2] == list(res[ar][2:])


def test_preserve_ar_geometry_worked_examples(oracle_port):
    """Crop 20x10 -> 8x8 PRESERVE_AR: target 8x4, factors 2.5, region [0,2]-[7,5]; 8x16 -> 8x8: target 4x8."""
    a = oracle_port.derive_resize(20, 10, 8, 8, abi.RESIZE_PRESERVE_AR)
    assert (a.target_width, a.target_height, a.fx, a.fy, a.x1, a.y1, a.x2, a.y2) == (8, 4, 2.5, 2.5, 0, 2, 7, 5)
    b = oracle_port.derive_resize(8, 16, 8, 8, abi.RESIZE_PRESERVE_AR)
    assert (b.target_width, b.target_height, b.fx, b.fy, b.x1, b.y1, b.x2, b.y2) == (4, 8, 2.0, 2.0, 2, 0, 5, 7)


@pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built (reference tree absent)")
def test_port_matches_reference_build_on_shared_cases(oracle_port):
    """Direct comparison with the compiled reference on fresh seeds (beyond the stored fixtures)."""
    rng = np.random.default_rng(5)
    for trial in range(4):
        fw, fh = int(rng.integers(40, 300)), int(rng.integers(40, 200))
        frames = [rng.integers(0, 256, (fh, fw, 3), dtype=np.uint8) for _ in range(2)]
        n = int(rng.integers(1, 20))
        rects = chains.random_rects(rng, n, fw, fh, lo=1, hi=min(fw, fh))
        fi = [i % 2 for i in range(n)]
        dw, dh = int(rng.integers(1, 80)), int(rng.integers(1, 80))
        out = np.zeros((n, 3, dh, dw), np.float32)
        plan = chains.crop_resize_batch(frame_ptrs=[f.ctypes.data for f in frames], frame_index=fi, rects=rects,
                                        src_width=fw, src_height=fh, src_pitch=fw * 3, dst=out.ctypes.data,
                                        dst_width=dw, dst_height=dh, post_ops=chains.normalize_ops(), planar=True,
                                        background=(3.0, 5.0, 7.0))
        oracle_port.run(plan)
        expect = ref.crop_resize_norm_planar(frames, fi, rects, dw, dh, (3.0, 5.0, 7.0), 255.0, chains.IMAGENET_MEAN,
                                             chains.IMAGENET_STD)
        assert _same(out, expect), trial


@pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built (reference tree absent)")
def test_port_matches_reference_build_on_empty_regions(oracle_port):
    """A PRESERVE_AR target of zero columns or rows (resize.h:196-221 rounds it down): the reference's
    factors are infinite, its region of interest is empty, every element is the default value after
    the continuation."""
    rng = np.random.default_rng(6)
    frame = rng.integers(0, 256, (1024, 1024, 3), dtype=np.uint8)
    rects = np.array([(0, 0, 2, 130), (0, 0, 1, 1000), (0, 0, 1000, 1), (5, 7, 3, 900), (10, 10, 100, 80)], np.int32)
    fi = [0] * len(rects)
    for dw, dh in ((32, 32), (224, 224), (45, 31)):
        out = np.zeros((len(rects), 3, dh, dw), np.float32)
        plan = chains.crop_resize_batch(frame_ptrs=[frame.ctypes.data], frame_index=fi, rects=rects, src_width=1024,
                                        src_height=1024, src_pitch=3072, dst=out.ctypes.data, dst_width=dw, dst_height=dh,
                                        post_ops=chains.normalize_ops(), planar=True, background=(3.0, 7.0, 11.0))
        oracle_port.run(plan)
        expect = ref.crop_resize_norm_planar([frame], fi, rects, dw, dh, (3.0, 7.0, 11.0), 255.0, chains.IMAGENET_MEAN,
                                             chains.IMAGENET_STD)
        assert _same(out, expect)
        n_empty = 0
        for i, r in enumerate(rects):
            rp = oracle_port.derive_resize(int(r[2]), int(r[3]), dw, dh, abi.RESIZE_PRESERVE_AR)
            if rp.target_width == 0 or rp.target_height == 0:   # background only
                n_empty += 1
                for c in range(3):
                    assert np.unique(expect[i, c]).size == 1
        assert n_empty >= 2


def test_other_aspect_ratio_modes(oracle_port):
    """PRESERVE_AR_RN_EVEN and PRESERVE_AR_LEFT (resize.h:42,132-147,200-210) against the reference build's output."""
    g = np.load(GOLD / "ar_modes.npz")
    frames = [np.ascontiguousarray(f) for f in g["frames"]]
    fi = [int(i) for i in g["frame_index"]]
    for key, mode in (("rn_even", abi.RESIZE_PRESERVE_AR_RN_EVEN), ("left", abi.RESIZE_PRESERVE_AR_LEFT)):
        out = np.zeros((len(fi), 3, 30, 44), np.float32)
        plan = chains.crop_resize_batch(frame_ptrs=[f.ctypes.data for f in frames], frame_index=fi, rects=g["rects"], src_width=200,
                                        src_height=120, src_pitch=600, dst=out.ctypes.data, dst_width=44, dst_height=30,
                                        post_ops=chains.normalize_ops(), planar=True, mode=mode, background=(3.0, 5.0, 7.0))
        oracle_port.run(plan)
        assert _same(out, g[key]), key
    assert not _same(g["rn_even"], g["left"])
    # worked examples: 10x7 -> 44x30: height fits (scale 30/7): width round(42.857) = 43 -> even 42, centred at 1; LEFT keeps 43 at 0
    a = oracle_port.derive_resize(10, 7, 44, 30, abi.RESIZE_PRESERVE_AR_RN_EVEN)
    b = oracle_port.derive_resize(10, 7, 44, 30, abi.RESIZE_PRESERVE_AR_LEFT)
    assert (a.target_width, a.x1, a.x2) == (42, 1, 42) and (b.target_width, b.x1, b.x2) == (43, 0, 42)


def test_nv21_and_the_other_matrices(oracle_port):
    g = np.load(GOLD / "nv_layouts.npz")
    frames = [np.ascontiguousarray(f) for f in g["frames"]]
    for key, fmt, conv, (dw, dh) in (("nv12_bt601", abi.SRC_NV12, abi.OP_YUV_TO_RGB_BT601_FULL, (40, 22)),
                                     ("nv12_bt2020", abi.SRC_NV12, abi.OP_YUV_TO_RGB_BT2020_FULL, (40, 22)),
                                     ("nv21_bt709", abi.SRC_NV21, abi.OP_YUV_TO_RGB_BT709_FULL, (40, 22)),
                                     ("nv21_bt601", abi.SRC_NV21, abi.OP_YUV_TO_RGB_BT601_FULL, (32, 18))):
        out = np.zeros((2, dh, dw, 3), np.float32)
        plan = chains.nv12_resize_batch(frame_ptrs=[f.ctypes.data for f in frames], width=96, height=54, pitch=96,
                                        dst=out.ctypes.data, dst_width=dw, dst_height=dh, src_format=fmt, conversion=conv)
        oracle_port.run(plan)
        assert _same(out, g[key]), key


def test_planes_of_a_partly_filled_batch_read_the_default_value(oracle_port):
    """BatchRead<4, CONDITIONAL_WITH_DEFAULT> (batch_operations.h:217-241) followed by Cast and Mul."""
    g = np.load(GOLD / "default_planes.npz")
    srcs = [np.ascontiguousarray(s) for s in g["srcs"]]
    for key, used in (("used2", 2), ("used0", 0)):
        out = np.zeros((4, 20, 36, 3), np.float32)
        plan = abi.HostPlan()
        seq = plan.add_sequence(abi.SRC_U8X3, abi.DST_F32X3_PACKED, abi.RESIZE_NONE, [op(abi.OP_CAST_F32), op(abi.OP_MUL, (1.5, 0.25, 2.0))],
                                background=(7.0, 200.0, 33.0))
        for i in range(4):
            plan.add_plane(src=srcs[i].ctypes.data if i < used else 0, src_width=36, src_height=20, src_pitch=108,
                           dst=out.ctypes.data + i * out[0].nbytes, dst_width=36, dst_height=20, dst_pitch=432, sequence=seq,
                           flags=0 if i < used else abi.PLANE_DEFAULT_VALUE)
        oracle_port.run(plan)
        assert _same(out, g[key]), key


def _readback_plan(src, out, *, dst_fmt, mode, dw, dh, ops, n_pre=0, crop=None, border=0, border_value=(0, 0, 0), deinterlace=0,
                   transform=None):
    h, w, _ = src.shape
    plan = abi.HostPlan()
    seq = plan.add_sequence(abi.SRC_U8X3, dst_fmt, mode, ops, n_pre_ops=n_pre, border_mode=border, border_value=border_value,
                            deinterlace=deinterlace, transform=transform)
    dpx = 3 if dst_fmt == abi.DST_U8X3_PACKED else 12
    plan.add_plane(src=src.ctypes.data, src_width=w, src_height=h, src_pitch=w * 3, crop=crop, dst=out.ctypes.data, dst_width=dw,
                   dst_height=dh, dst_pitch=dw * dpx, sequence=seq)
    return plan


def test_border_reader_warping_and_deinterlace(oracle_port):
    """BorderReader under a crop that reaches beyond the image (border_reader.h:136-279), Warping<Affine|Perspective>
    (warping.h:43-104) and Deinterlace<BLEND|INTER_LINEAR> (deinterlace.h:41-132) against the reference build's output."""
    g = np.load(GOLD / "readback_ops.npz")
    src = np.ascontiguousarray(g["src"])
    rect = tuple(int(v) for v in g["rect"])
    for b in range(1, 6):
        out = np.zeros((rect[3], rect[2], 3), np.uint8)
        oracle_port.run(_readback_plan(src, out, dst_fmt=abi.DST_U8X3_PACKED, mode=abi.RESIZE_NONE, dw=rect[2], dh=rect[3], ops=[],
                                       crop=rect, border=b, border_value=(9, 99, 199)))
        assert np.array_equal(out, g[f"border{b}_crop"]), f"border {b}"
        outf = np.zeros((28, 36, 3), np.float32)
        oracle_port.run(_readback_plan(src, outf, dst_fmt=abi.DST_F32X3_PACKED, mode=abi.RESIZE_IGNORE_AR, dw=36, dh=28, ops=[],
                                       crop=rect, border=b, border_value=(9, 99, 199)))
        assert _same(outf, g[f"border{b}_crop_resize"]), f"border {b} + resize"
    mul = [op(abi.OP_MUL, (1.0, 0.5, 2.0))]
    for key, mode in (("affine", abi.GEOMETRY_WARP_AFFINE), ("perspective", abi.GEOMETRY_WARP_PERSPECTIVE)):
        outf = np.zeros((32, 48, 3), np.float32)
        oracle_port.run(_readback_plan(src, outf, dst_fmt=abi.DST_F32X3_PACKED, mode=mode, dw=48, dh=32, ops=mul, transform=g[key]))
        assert _same(outf, g[f"warp_{key}"]), key
        assert (g[f"warp_{key}"] == 0).any() and (g[f"warp_{key}"] != 0).any()      # some of the output lies outside the source
    for k in (1, 2, 3):
        outf = np.zeros(src.shape, np.float32)
        oracle_port.run(_readback_plan(src, outf, dst_fmt=abi.DST_F32X3_PACKED, mode=abi.RESIZE_NONE, dw=src.shape[1], dh=src.shape[0],
                                       ops=mul, deinterlace=k))
        assert _same(outf, g[f"deinterlace{k}"]), f"deinterlace {k}"


def test_yuv_layouts_beyond_nv12(oracle_port):
    """ReadYUV<P010 | P210 | Y210 | UYVY> -> ConvertYUVToRGB<PF, Full, bt709 | bt601 | bt2020> (color_conversion.h:284-372):
    the 10-bit layouts shifted right by 6, offsets 512 / 64, result times 64; against the reference build's output."""
    g = np.load(GOLD / "yuv_layouts.npz")
    conv = (abi.OP_YUV_TO_RGB_BT709_FULL, abi.OP_YUV_TO_RGB_BT601_FULL, abi.OP_YUV_TO_RGB_BT2020_FULL)
    for fmt in (abi.SRC_P010, abi.SRC_P210, abi.SRC_Y210, abi.SRC_UYVY):
        img = np.ascontiguousarray(g[f"src{fmt}"])

        def run(prim, dw, dh):
            out = np.zeros((dh, dw, 3), np.float32)
            plan = abi.HostPlan()
            mode = abi.RESIZE_NONE if (dw, dh) == (38, 22) else abi.RESIZE_IGNORE_AR
            seq = plan.add_sequence(fmt, abi.DST_F32X3_PACKED, mode, [op(conv[prim]), op(abi.OP_MUL, (1.0, 0.5, 2.0))], n_pre_ops=1)
            plan.add_plane(src=img.ctypes.data, src_width=38, src_height=22, src_pitch=img.strides[0], dst=out.ctypes.data, dst_width=dw,
                           dst_height=dh, dst_pitch=dw * 12, sequence=seq)
            oracle_port.run(plan)
            return out

        for prim in (0, 1, 2):
            assert _same(run(prim, 38, 22), g[f"fmt{fmt}_prim{prim}"]), (fmt, prim)
        assert _same(run(fmt % 3, 27, 15), g[f"fmt{fmt}_resize"]), fmt
