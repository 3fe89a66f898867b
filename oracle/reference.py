"""ctypes binding of oracle/_ref/libfklref_*.so: the reference's own headers on the host.

TEST INFRASTRUCTURE ONLY.  Two flavours are built by oracle/Makefile:
  device_branch - with oracle/ref/device_branch_prelude.h force-included: the host runs the
                  device branch of interpolation.h:65-71.  This is the parity target.
  literal       - the unmodified CPU backend, whose bilinear taps take the row index from
                  the horizontal coordinate (interpolation.h:70); kept to document the
                  difference, and valid for chains without Resize.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
_libs: dict[str, C.CDLL] = {}

_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int)


def available(flavour: str = "device_branch") -> bool:
    return (REF_DIR / f"libfklref_{flavour}.so").exists()


def lib(flavour: str = "device_branch") -> C.CDLL:
    if flavour not in _libs:
        p = REF_DIR / f"libfklref_{flavour}.so"
        if not p.exists():
            raise FileNotFoundError(f"{p}: run `make -C oracle ref` where the reference tree is present")
        _libs[flavour] = C.CDLL(str(p))
    return _libs[flavour]


def _f3(v):
    if isinstance(v, (int, float)):
        v = (v, v, v)
    return (C.c_float * 3)(*[float(x) for x in v])


def _u8(a):
    return a.ctypes.data_as(_u8p)


def _f32(a):
    return a.ctypes.data_as(_f32p)


def cast_mul_sub_div(src, mul, sub, div, flavour="device_branch"):
    h, w, _ = src.shape
    out = np.empty((h, w, 3), np.float32)
    lib(flavour).fklref_cast_mul_sub_div(_u8(src), w, h, src.strides[0], _f3(mul), _f3(sub), _f3(div),
                                        _f32(out), out.strides[0])
    return out


def cast_mul_sub(src, mul, sub, flavour="device_branch"):
    h, w, _ = src.shape
    out = np.empty((h, w, 3), np.float32)
    lib(flavour).fklref_cast_mul_sub(_u8(src), w, h, src.strides[0], _f3(mul), _f3(sub), _f32(out),
                                    out.strides[0])
    return out


def cast_add_div(src, add, div, flavour="device_branch"):
    h, w, _ = src.shape
    out = np.empty((h, w, 3), np.float32)
    lib(flavour).fklref_cast_add_div(_u8(src), w, h, src.strides[0], _f3(add), _f3(div), _f32(out),
                                    out.strides[0])
    return out


def bgr_cast_mul_saturate(src, mul, flavour="device_branch"):
    h, w, _ = src.shape
    out = np.empty((h, w, 3), np.uint8)
    lib(flavour).fklref_bgr_cast_mul_saturate(_u8(src), w, h, src.strides[0], _f3(mul), _u8(out),
                                             out.strides[0])
    return out


def cast_mul_sub_cast_int3(src, mul, sub, flavour="device_branch"):
    h, w, _ = src.shape
    out = np.empty((h, w, 3), np.int32)
    lib(flavour).fklref_cast_mul_sub_cast_int3(_u8(src), w, h, src.strides[0], _f3(mul), _f3(sub),
                                              out.ctypes.data_as(C.POINTER(C.c_int32)), out.strides[0])
    return out


def cast_resize_mul_cast_uint3(src, dw, dh, mul, flavour="device_branch"):
    h, w, _ = src.shape
    out = np.empty((dh, dw, 3), np.uint32)
    lib(flavour).fklref_cast_resize_mul_cast_uint3(_u8(src), w, h, src.strides[0], dw, dh, _f3(mul),
                                                  out.ctypes.data_as(C.POINTER(C.c_uint32)), out.strides[0])
    return out


def cast_resize(src, dw, dh, flavour="device_branch"):
    h, w, _ = src.shape
    out = np.empty((dh, dw, 3), np.float32)
    lib(flavour).fklref_cast_resize(_u8(src), w, h, src.strides[0], dw, dh, _f32(out), out.strides[0])
    return out


def addmul_chain(src, n, add, mul, flavour="device_branch"):
    h, w, _ = src.shape
    out = np.empty((h, w, 3), np.float32)
    rc = lib(flavour).fklref_addmul_chain(_f32(src), w, h, src.strides[0], n, _f3(add), _f3(mul), _f32(out),
                                         out.strides[0])
    if rc != 0:
        raise ValueError(f"chain length {n} is not instantiated in the reference wrapper")
    return out


def _frames_arg(frames, frame_index):
    ptrs = (C.c_void_p * len(frame_index))(*[frames[i].ctypes.data for i in frame_index])
    return ptrs


def crop_resize_readme(frames, frame_index, rects, dw, dh, bg, mul, sub, div, preserve_ar=True,
                       flavour="device_branch"):
    """frames: list of (h,w,3) uint8 arrays of one size; frame_index[i] = source of plane i;
    rects: (B,4) int array of x,y,w,h.  Returns (B, dh, dw, 3) float32 (TensorWrite<float3>)."""
    h, w, _ = frames[0].shape
    rects = np.ascontiguousarray(rects, np.int32)
    b = len(frame_index)
    out = np.empty((b, dh, dw, 3), np.float32)
    ptrs = _frames_arg(frames, frame_index)
    if preserve_ar:
        lib(flavour).fklref_crop_resize_readme(ptrs, w, h, frames[0].strides[0], rects.ctypes.data_as(_i32p), b,
                                              dw, dh, _f3(bg), _f3(mul), _f3(sub), _f3(div), _f32(out))
    else:
        lib(flavour).fklref_crop_resize_readme_ignore_ar(ptrs, w, h, frames[0].strides[0],
                                                        rects.ctypes.data_as(_i32p), b, dw, dh, _f3(mul),
                                                        _f3(sub), _f3(div), _f32(out))
    return out


def crop_resize_norm_planar(frames, frame_index, rects, dw, dh, bg, d0, mean, std, flavour="device_branch",
                            out=None):
    """Returns (B, 3, dh, dw) float32 (TensorSplit<float3>)."""
    h, w, _ = frames[0].shape
    rects = np.ascontiguousarray(rects, np.int32)
    b = len(frame_index)
    if out is None:
        out = np.empty((b, 3, dh, dw), np.float32)
    ptrs = _frames_arg(frames, frame_index)
    lib(flavour).fklref_crop_resize_norm_planar(ptrs, w, h, frames[0].strides[0], rects.ctypes.data_as(_i32p), b,
                                               dw, dh, _f3(bg), _f3(d0), _f3(mean), _f3(std), _f32(out))
    return out


def nv12_resize(frames, w, h, dw, dh, div, flavour="device_branch", out=None):
    """frames: list of (h*3/2, pitch) uint8 arrays (luma rows then interleaved chroma rows).
    Returns (B, dh, dw, 3) float32."""
    b = len(frames)
    if out is None:
        out = np.empty((b, dh, dw, 3), np.float32)
    ptrs = (C.c_void_p * b)(*[f.ctypes.data for f in frames])
    lib(flavour).fklref_nv12_resize(ptrs, w, h, frames[0].strides[0], b, dw, dh, _f3(div), _f32(out))
    return out


def crop_resize_norm_planar_mode(frames, frame_index, rects, dw, dh, mode, bg, d0, mean, std, flavour="device_branch"):
    """mode: 3 = PRESERVE_AR_RN_EVEN, 4 = PRESERVE_AR_LEFT.  Returns (B, 3, dh, dw) float32."""
    h, w, _ = frames[0].shape
    rects = np.ascontiguousarray(rects, np.int32)
    b = len(frame_index)
    out = np.empty((b, 3, dh, dw), np.float32)
    rc = lib(flavour).fklref_crop_resize_norm_planar_mode(_frames_arg(frames, frame_index), w, h, frames[0].strides[0],
                                                         rects.ctypes.data_as(_i32p), b, dw, dh, mode, _f3(bg), _f3(d0), _f3(mean),
                                                         _f3(std), _f32(out))
    if rc != 0:
        raise ValueError(f"aspect-ratio mode {mode} is not instantiated in the reference wrapper")
    return out


def nv_resize_ex(frames, w, h, dw, dh, div, layout, primitives, flavour="device_branch"):
    """layout 0 = NV12, 1 = NV21; primitives 0 = bt709, 1 = bt601, 2 = bt2020.  Returns (B, dh, dw, 3) float32; B even."""
    b = len(frames)
    out = np.empty((b, dh, dw, 3), np.float32)
    ptrs = (C.c_void_p * b)(*[f.ctypes.data for f in frames])
    rc = lib(flavour).fklref_nv_resize_ex(ptrs, w, h, frames[0].strides[0], b, dw, dh, layout, primitives, _f3(div), _f32(out))
    if rc != 0:
        raise ValueError("this layout / matrix pair is not instantiated in the reference wrapper")
    return out


def batch4_default_cast_mul(srcs, used, default_value, mul, flavour="device_branch"):
    """Four (h,w,3) uint8 images, planes >= used read default_value (3 bytes).  Returns (4, h, w, 3) float32."""
    h, w, _ = srcs[0].shape
    out = np.empty((4, h, w, 3), np.float32)
    ptrs = (C.c_void_p * 4)(*[s.ctypes.data for s in srcs])
    dv = (C.c_uint8 * 3)(*[int(v) for v in default_value])
    lib(flavour).fklref_batch4_default_cast_mul(ptrs, w, h, srcs[0].strides[0], used, dv, _f3(mul), _f32(out))
    return out


def border_crop(src, border, value, rect, flavour="device_branch"):
    """PerThreadRead<uchar3> -> BorderReader<border> -> Crop(rect) -> PerThreadWrite<uchar3>; border 1..5 as fkb_border_mode."""
    h, w, _ = src.shape
    out = np.empty((rect[3], rect[2], 3), np.uint8)
    r = (C.c_int * 4)(*[int(v) for v in rect])
    v = (C.c_uint8 * 3)(*[int(x) for x in value])
    if lib(flavour).fklref_border_crop(_u8(src), w, h, src.strides[0], border, v, r, _u8(out)) != 0:
        raise ValueError("unknown border type")
    return out


def border_crop_resize(src, border, value, rect, dw, dh, flavour="device_branch"):
    """... -> Crop(rect) -> Resize<INTER_LINEAR>(dw, dh) -> PerThreadWrite<float3>."""
    h, w, _ = src.shape
    out = np.empty((dh, dw, 3), np.float32)
    r = (C.c_int * 4)(*[int(v) for v in rect])
    v = (C.c_uint8 * 3)(*[int(x) for x in value])
    if lib(flavour).fklref_border_crop_resize(_u8(src), w, h, src.strides[0], border, v, r, dw, dh, _f32(out)) != 0:
        raise ValueError("unknown border type")
    return out


def warp(src, perspective, matrix, dw, dh, mul, flavour="device_branch"):
    """PerThreadRead<uchar3> -> Warping<Affine|Perspective>(matrix, dw x dh) -> Mul -> PerThreadWrite<float3>."""
    h, w, _ = src.shape
    out = np.empty((dh, dw, 3), np.float32)
    m = (C.c_float * 9)(*[float(x) for x in matrix])
    lib(flavour).fklref_warp(_u8(src), w, h, src.strides[0], int(perspective), m, dw, dh, _f3(mul), _f32(out))
    return out


def deinterlace(src, kind, mul, flavour="device_branch"):
    """PerThreadRead<uchar3> -> Deinterlace -> Mul -> PerThreadWrite<float3>; kind 1 BLEND, 2 / 3 INTER_LINEAR even / odd."""
    h, w, _ = src.shape
    out = np.empty((h, w, 3), np.float32)
    if lib(flavour).fklref_deinterlace(_u8(src), w, h, src.strides[0], kind, _f3(mul), _f32(out)) != 0:
        raise ValueError("unknown deinterlace kind")
    return out


def yuv_format_chain(frame, fmt, primitives, w, h, dw, dh, mul, flavour="device_branch"):
    """ReadYUV<PF> -> ConvertYUVToRGB<PF, Full, CP, false, float3> [-> Resize(dw, dh)] -> Mul -> PerThreadWrite<float3>.
    frame: 2-D array of the layout's words (uint16 for P010 / P210 / Y210, uint8 for UYVY), rows one pitch apart; fmt as
    fkb_src_format (5 P010, 6 P210, 7 Y210, 8 UYVY); primitives 0 bt709, 1 bt601, 2 bt2020.  No resize when dw x dh = w x h."""
    out = np.empty((dh, dw, 3), np.float32)
    if lib(flavour).fklref_yuv_format_chain(fmt, primitives, C.c_void_p(frame.ctypes.data), w, h, frame.strides[0], dw, dh, _f3(mul), _f32(out)) != 0:
        raise ValueError("this layout / matrix pair is not instantiated in the reference wrapper")
    return out


def resize_params(sw, sh, dw, dh, preserve_ar, flavour="device_branch"):
    fxy = (C.c_float * 2)()
    roi = (C.c_int * 4)()
    lib(flavour).fklref_resize_params(sw, sh, dw, dh, int(preserve_ar), fxy, roi)
    return (fxy[0], fxy[1]), tuple(roi)
