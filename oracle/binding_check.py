"""ctypes access to oracle/_ref/libfklref_binding.so: chains built with the reference's real operation
types and handed to include/fkb200_executor.h, the reference-side binding of libfkb200.

TEST INFRASTRUCTURE ONLY (see oracle/ref/fklref_binding.cpp).  mode 0 executes on device pointers through
fk::executeOperations<fkb200::TransformDPP>; mode 1 lowers only and keeps the plan for inspection.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from fusedkernellibrary_b200 import abi

HERE = Path(__file__).resolve().parent
LIB = HERE / "_ref" / "libfklref_binding.so"
_lib = None

EXECUTE, DESCRIBE = 0, 1


def available() -> bool:
    return LIB.exists()


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB.exists():
            raise FileNotFoundError(f"{LIB}: run `make -C oracle binding` where the reference tree is present")
        abi.load_library()   # the binding links libfkb200.so: load the in-tree one first
        _lib = C.CDLL(str(LIB))
        _lib.fklbind_last_error.restype = C.c_char_p
    return _lib


def _f3(v):
    if isinstance(v, (int, float)):
        v = (v, v, v)
    return (C.c_float * 3)(*[float(x) for x in v])


def _p(x):
    return C.c_void_p(int(x) if x else 0)


def _check(rc):
    if rc != 0:
        raise RuntimeError(lib().fklbind_last_error().decode())


def readme5(mode, frame, w, h, pitch, rects, bg, mul, sub, div, out, stream=None):
    r = np.ascontiguousarray(rects, np.int32)
    _check(lib().fklbind_readme5(mode, _p(frame), w, h, pitch, r.ctypes.data_as(C.POINTER(C.c_int)), _f3(bg), _f3(mul), _f3(sub),
                                 _f3(div), _p(out), _p(stream)))


def norm_planar16(mode, frames16, w, h, pitch, rects, dw, dh, bg, d0, mean, std, out, stream=None):
    r = np.ascontiguousarray(rects, np.int32)
    ptrs = (C.c_void_p * 16)(*[int(p) for p in frames16])
    _check(lib().fklbind_norm_planar16(mode, ptrs, w, h, pitch, r.ctypes.data_as(C.POINTER(C.c_int)), dw, dh, _f3(bg), _f3(d0),
                                       _f3(mean), _f3(std), _p(out), _p(stream)))


def nv12_2(mode, frames2, w, h, pitch, dw, dh, div, out, stream=None):
    ptrs = (C.c_void_p * 2)(*[int(p) for p in frames2])
    _check(lib().fklbind_nv12_2(mode, ptrs, w, h, pitch, dw, dh, _f3(div), _p(out), _p(stream)))


def cast_mul_sub_div(mode, src, w, h, spitch, mul, sub, div, dst, dpitch, stream=None):
    _check(lib().fklbind_cast_mul_sub_div(mode, _p(src), w, h, spitch, _f3(mul), _f3(sub), _f3(div), _p(dst), dpitch, _p(stream)))


def cast_resize_add_cast_uint3(mode, src, w, h, spitch, dw, dh, add, dst, dpitch, stream=None):
    _check(lib().fklbind_cast_resize_add_cast_uint3(mode, _p(src), w, h, spitch, dw, dh, _f3(add), _p(dst), dpitch, _p(stream)))


def bgr_cast_mul_saturate(mode, src, w, h, spitch, mul, dst, dpitch, stream=None):
    _check(lib().fklbind_bgr_cast_mul_saturate(mode, _p(src), w, h, spitch, _f3(mul), _p(dst), dpitch, _p(stream)))


def nv21_bt601_2(mode, frames2, w, h, pitch, dw, dh, div, out, stream=None):
    ptrs = (C.c_void_p * 2)(*[int(p) for p in frames2])
    _check(lib().fklbind_nv21_bt601_2(mode, ptrs, w, h, pitch, dw, dh, _f3(div), _p(out), _p(stream)))


def left_tsplit4(mode, frames4, w, h, pitch, rects, dw, dh, bg, d0, mean, std, out, stream=None):
    r = np.ascontiguousarray(rects, np.int32)
    ptrs = (C.c_void_p * 4)(*[int(p) for p in frames4])
    _check(lib().fklbind_left_tsplit4(mode, ptrs, w, h, pitch, r.ctypes.data_as(C.POINTER(C.c_int)), dw, dh, _f3(bg), _f3(d0), _f3(mean),
                                      _f3(std), _p(out), _p(stream)))


def batch4_default_cast_mul(mode, srcs4, w, h, spitch, used, default_value, mul, dst, stream=None):
    ptrs = (C.c_void_p * 4)(*[int(p) for p in srcs4])
    dv = (C.c_uint8 * 3)(*[int(v) for v in default_value])
    _check(lib().fklbind_batch4_default_cast_mul(mode, ptrs, w, h, spitch, used, dv, _f3(mul), _p(dst), _p(stream)))


def border_crop_resize(mode, src, w, h, pitch, border, value, rect, dw, dh, out, stream=None):
    v = (C.c_uint8 * 3)(*[int(x) for x in value])
    r = (C.c_int * 4)(*[int(x) for x in rect])
    _check(lib().fklbind_border_crop_resize(mode, _p(src), w, h, pitch, border, v, r, dw, dh, _p(out), _p(stream)))


def warp(mode, src, w, h, pitch, perspective, matrix, dw, dh, mul, out, stream=None):
    m = (C.c_float * 9)(*[float(x) for x in np.asarray(matrix, np.float32).reshape(-1)])
    _check(lib().fklbind_warp(mode, _p(src), w, h, pitch, int(perspective), m, dw, dh, _f3(mul), _p(out), _p(stream)))


def deinterlace(mode, src, w, h, pitch, kind, mul, out, stream=None):
    _check(lib().fklbind_deinterlace(mode, _p(src), w, h, pitch, kind, _f3(mul), _p(out), _p(stream)))


def yuv_layout(mode, fmt, frame, w, h, pitch, dw, dh, mul, out, stream=None):
    _check(lib().fklbind_yuv_layout(mode, fmt, _p(frame), w, h, pitch, dw, dh, _f3(mul), _p(out), _p(stream)))


def circular_describe6(order, frame, w, h, pitch, rect, dw, dh, bg, d0, mean, std, visible, hidden, first):
    """Lowers the two sequences CircularTensor::update builds for a 6-plane planar tensor; the plan is kept for last_plan()."""
    r = (C.c_int * 4)(*[int(x) for x in rect])
    _check(lib().fklbind_circular_describe6(order, _p(frame), w, h, pitch, r, dw, dh, _f3(bg), _f3(d0), _f3(mean), _f3(std), _p(visible),
                                            _p(hidden), first))


class ReferenceCircularTensor:
    """fk::CircularTensor<float, 3, 6, order, ColorPlanes::Standard> itself (device memory it allocates); update() runs through
    the Executor<DivergentBatchTransformDPP> that include/fkb200_executor.h supplies."""

    def __init__(self, order, w, h):
        l = lib()
        l.fklbind_circular_create.restype = C.c_void_p
        l.fklbind_circular_data.restype = C.c_void_p
        l.fklbind_circular_data.argtypes = [C.c_void_p]
        l.fklbind_circular_destroy.argtypes = [C.c_void_p]
        self._h = l.fklbind_circular_create(order, w, h)
        if not self._h:
            raise RuntimeError(l.fklbind_last_error().decode())

    @property
    def data(self) -> int:
        return lib().fklbind_circular_data(self._h)

    def update(self, frame, w, h, pitch, rect, bg, d0, mean, std, stream=None):
        r = (C.c_int * 4)(*[int(x) for x in rect])
        _check(lib().fklbind_circular_update(C.c_void_p(self._h), _p(frame), w, h, pitch, r, _f3(bg), _f3(d0), _f3(mean), _f3(std), _p(stream)))

    def destroy(self):
        if self._h:
            lib().fklbind_circular_destroy(self._h)
            self._h = None


def last_plan():
    """(planes, sequences) of the last DESCRIBE call: planes as abi.Plane, sequences as (abi.Sequence, [abi.Op])."""
    n_p, n_s = C.c_int(), C.c_int()
    lib().fklbind_last_counts(C.byref(n_p), C.byref(n_s))
    planes = []
    for i in range(n_p.value):
        p = abi.Plane()
        assert lib().fklbind_last_plane(i, C.byref(p)) == 0
        planes.append(p)
    seqs = []
    for s in range(n_s.value):
        q = abi.Sequence()
        ops = (abi.Op * 64)()
        n = lib().fklbind_last_sequence(s, C.byref(q), ops, 64)
        seqs.append((q, [ops[k] for k in range(n)]))
    return planes, seqs


def last_reference_resize(i) -> abi.ResizeParams | None:
    rp = abi.ResizeParams()
    return rp if lib().fklbind_last_reference_resize(i, C.byref(rp)) == 0 else None
