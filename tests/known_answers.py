"""Known-answer cases taken from the reference's tests for this path (values read from the test
sources; nothing is executed from the reference tree).

* constant image (128x128 of 0) -> Cast<uchar3,float3> -> Resize 32x32 -> Add(3,1,32) -> Cast<float3,uint3>
  -> PerThreadWrite<uint3>: every pixel equals (3,1,32) as unsigned integers
  (tests/operation/test_instantiable_operations.h:236-264).
* constant 2 copied through PerThreadRead -> PerThreadWrite, full 1920x1080 image and a 300x200
  crop, for uchar3 and float3 (tests/data/basic_test.h:32-84).
* COLOR_BGR2RGB on uchar3 {100,150,200} -> {200,150,100} and {50,75,125} -> {125,75,50}
  (utests/algorithm/image_processing/utest_color_conversion.h:89-100).
* SaturateCast<float3,uchar3>: below range -> 0, above -> 255, halves round away from zero
  (utests/algorithm/image_processing/utest_saturate.h:43-84).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import numpy as np

from fusedkernellibrary_b200 import abi, chains
from fusedkernellibrary_b200.abi import op


@dataclass
class KnownAnswer:
    name: str
    make_arrays: Callable
    build: Callable
    expect: Callable  # expect(arrays) -> (got, wanted)


def _resize_constant():
    def make():
        return {"src": np.zeros((128, 128, 3), np.uint8), "out": np.zeros((32, 32, 3), np.uint32)}

    def build(ptr):
        plan = abi.HostPlan()
        s = plan.add_sequence(abi.SRC_U8X3, abi.DST_U32X3_PACKED, abi.RESIZE_IGNORE_AR,
                              [op(abi.OP_CAST_F32), op(abi.OP_ADD, (3.0, 1.0, 32.0)), op(abi.OP_CAST_U32)], n_pre_ops=1)
        plan.add_plane(src=ptr("src"), src_width=128, src_height=128, src_pitch=384, dst=ptr("out"), dst_width=32,
                       dst_height=32, dst_pitch=384, sequence=s)
        return plan

    def expect(a):
        want = np.empty((32, 32, 3), np.uint32)
        want[...] = (3, 1, 32)
        return a["out"], want

    return KnownAnswer("resize_constant_then_add_then_cast_uint3", make, build, expect)


def _copy(fmt, crop):
    is_u8 = fmt == abi.SRC_U8X3
    dt = np.uint8 if is_u8 else np.float32
    dfmt = abi.DST_U8X3_PACKED if is_u8 else abi.DST_F32X3_PACKED
    w, h = 1920, 1080
    ow, oh = (crop[2], crop[3]) if crop else (w, h)

    def make():
        return {"src": np.full((h, w, 3), 2, dt), "out": np.zeros((oh, ow, 3), dt)}

    def build(ptr):
        return chains.elementwise([], src=ptr("src"), dst=ptr("out"), width=w, height=h, src_format=fmt,
                                  dst_format=dfmt, crop=crop)

    def expect(a):
        return a["out"], np.full((oh, ow, 3), 2, dt)

    return KnownAnswer(f"copy_{'u8' if is_u8 else 'f32'}_{'crop' if crop else 'full'}", make, build, expect)


def _bgr2rgb():
    def make():
        return {"src": np.array([[[100, 150, 200], [50, 75, 125]]], np.uint8), "out": np.zeros((1, 2, 3), np.uint8)}

    def build(ptr):
        return chains.elementwise([op(abi.OP_SWAP_RB)], src=ptr("src"), dst=ptr("out"), width=2, height=1,
                                  dst_format=abi.DST_U8X3_PACKED)

    def expect(a):
        return a["out"], np.array([[[200, 150, 100], [125, 75, 50]]], np.uint8)

    return KnownAnswer("bgr2rgb_uchar3", make, build, expect)


def _saturate():
    vals = np.array([[-3.4e38, -1.0, -0.4], [0.0, 0.49, 0.5], [1.5, 2.5, 127.5], [254.4, 254.5, 255.0],
                     [255.4, 256.0, 3.4e38], [127.49, 128.0, 200.7]], np.float32).reshape(1, 6, 3)
    want = np.array([[0, 0, 0], [0, 0, 1], [2, 3, 128], [254, 255, 255], [255, 255, 255], [127, 128, 201]],
                    np.uint8).reshape(1, 6, 3)

    def make():
        return {"src": vals.copy(), "out": np.zeros((1, 6, 3), np.uint8)}

    def build(ptr):
        return chains.elementwise([op(abi.OP_SATURATE_CAST_U8)], src=ptr("src"), dst=ptr("out"), width=6, height=1,
                                  src_format=abi.SRC_F32X3, dst_format=abi.DST_U8X3_PACKED)

    def expect(a):
        return a["out"], want

    return KnownAnswer("saturate_cast_float3_uchar3", make, build, expect)


KNOWN_ANSWER_CASES = [
    _resize_constant(),
    _copy(abi.SRC_U8X3, None), _copy(abi.SRC_U8X3, (100, 50, 300, 200)),
    _copy(abi.SRC_F32X3, None), _copy(abi.SRC_F32X3, (100, 50, 300, 200)),
    _bgr2rgb(), _saturate(),
]


def check_known_answer(case: KnownAnswer, arrays) -> None:
    got, want = case.expect(arrays)
    assert np.array_equal(got, want), case.name
