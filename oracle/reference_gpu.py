"""ctypes binding of oracle/_ref/libfklref_gpu*.so: the reference's own CUDA backend on this GPU.

TEST INFRASTRUCTURE ONLY.  oracle/Makefile compiles the wrapper sources under oracle/ref/ a second
time with nvcc and -DFKLREF_GPU, so that every chain runs through
fk::executeOperations<TransformDPP<ParArch::GPU_NVIDIA>> (core/execution_model/executors.h:252-287,
executor_details/executor_kernels.h:25-29).  Two flavours:
  default - nvcc's default floating-point flags, as the reference's own build uses; up to 128 planes
            per launch (the per-plane parameters are kernel arguments, batch_operations.h:98-102).
            This is the GPU baseline that the benchmark times beside the kernels of this package.
  nofma   - the same with -fmad=false, so that products and sums round separately as in the
            reference's CPU backend: the flavour that must agree bit for bit with oracle/_ref's
            device-branch build and with this package's kernels.
All pointers are DEVICE pointers (plain integers); calls return after the launch, on the stream
given to set_stream(); nothing here synchronises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
_libs: dict[str, C.CDLL] = {}
_NAMES = {"default": "libfklref_gpu.so", "nofma": "libfklref_gpu_nofma.so"}


def available(flavour: str = "default") -> bool:
    return (REF_DIR / _NAMES[flavour]).exists()


def lib(flavour: str = "default") -> C.CDLL:
    if flavour not in _libs:
        p = REF_DIR / _NAMES[flavour]
        if not p.exists():
            raise FileNotFoundError(f"{p}: run `make -C oracle refgpu` where the reference tree is present")
        l = C.CDLL(str(p))
        l.fklref_gpu_launches.restype = C.c_long
        l.fklref_gpu_set_stream.argtypes = [C.c_void_p]
        _libs[flavour] = l
    return _libs[flavour]


def set_stream(stream: int | None, flavour: str = "default") -> None:
    lib(flavour).fklref_gpu_set_stream(C.c_void_p(stream or 0))


def launches(flavour: str = "default") -> int:
    return int(lib(flavour).fklref_gpu_launches())


def _f3(v):
    if isinstance(v, (int, float)):
        v = (v, v, v)
    return (C.c_float * 3)(*[float(x) for x in v])


def _p(x):
    return C.c_void_p(int(x))


def _ptrs(ptrs):
    return (C.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def cast_mul_sub_div(src, w, h, spitch, mul, sub, div, dst, dpitch, flavour="default"):
    lib(flavour).fklref_gpu_cast_mul_sub_div(_p(src), w, h, spitch, _f3(mul), _f3(sub), _f3(div), _p(dst), dpitch)


def cast_mul_sub_div_batch16(srcs, w, h, spitch, mul, sub, div, dst, flavour="default"):
    lib(flavour).fklref_gpu_cast_mul_sub_div_batch16(_ptrs(srcs), w, h, spitch, _f3(mul), _f3(sub), _f3(div), _p(dst))


def cast_mul_sub_batch16(srcs, w, h, spitch, mul, sub, dst, flavour="default"):
    lib(flavour).fklref_gpu_cast_mul_sub_batch16(_ptrs(srcs), w, h, spitch, _f3(mul), _f3(sub), _p(dst))


def cast_add_div_batch16(srcs, w, h, spitch, add, div, dst, flavour="default"):
    lib(flavour).fklref_gpu_cast_add_div_batch16(_ptrs(srcs), w, h, spitch, _f3(add), _f3(div), _p(dst))


def bgr_cast_mul_saturate_batch16(srcs, w, h, spitch, mul, dst, flavour="default"):
    lib(flavour).fklref_gpu_bgr_cast_mul_saturate_batch16(_ptrs(srcs), w, h, spitch, _f3(mul), _p(dst))


def cast_resize_batch16(srcs, w, h, spitch, dw, dh, dst, flavour="default"):
    lib(flavour).fklref_gpu_cast_resize_batch16(_ptrs(srcs), w, h, spitch, dw, dh, _p(dst))


def addmul_chain(src, w, h, spitch, n, add, mul, dst, dpitch, flavour="default") -> bool:
    """False when the chain length is not instantiated (256 does not compile under nvcc)."""
    return lib(flavour).fklref_gpu_addmul_chain(_p(src), w, h, spitch, n, _f3(add), _f3(mul), _p(dst), dpitch) == 0


def crop_resize_readme(frame_ptrs, frame_index, w, h, pitch, rects, dw, dh, bg, mul, sub, div, dst, preserve_ar=True,
                       flavour="default"):
    """dst: device tensor B x dh x dw x 3 float32 (TensorWrite<float3>); B >= 2."""
    rects = np.ascontiguousarray(rects, np.int32)
    ptrs = _ptrs([frame_ptrs[i] for i in frame_index])
    r = rects.ctypes.data_as(C.POINTER(C.c_int))
    if preserve_ar:
        lib(flavour).fklref_gpu_crop_resize_readme(ptrs, w, h, pitch, r, len(frame_index), dw, dh, _f3(bg), _f3(mul),
                                                   _f3(sub), _f3(div), _p(dst))
    else:
        lib(flavour).fklref_gpu_crop_resize_readme_ignore_ar(ptrs, w, h, pitch, r, len(frame_index), dw, dh, _f3(mul),
                                                             _f3(sub), _f3(div), _p(dst))


def crop_resize_norm_planar(frame_ptrs, frame_index, w, h, pitch, rects, dw, dh, bg, d0, mean, std, dst,
                            flavour="default"):
    """dst: device tensor B x 3 x dh x dw float32 (TensorSplit<float3>); B >= 2."""
    rects = np.ascontiguousarray(rects, np.int32)
    ptrs = _ptrs([frame_ptrs[i] for i in frame_index])
    lib(flavour).fklref_gpu_crop_resize_norm_planar(ptrs, w, h, pitch, rects.ctypes.data_as(C.POINTER(C.c_int)),
                                                    len(frame_index), dw, dh, _f3(bg), _f3(d0), _f3(mean), _f3(std),
                                                    _p(dst))


def nv12_resize(frame_ptrs, w, h, pitch, dw, dh, div, dst, flavour="default"):
    """dst: device tensor B x dh x dw x 3 float32; B >= 2."""
    lib(flavour).fklref_gpu_nv12_resize(_ptrs(frame_ptrs), w, h, pitch, len(frame_ptrs), dw, dh, _f3(div), _p(dst))


def circular_update6(frame, w, h, pitch, rect, dw, dh, bg, d0, mean, std, visible, hidden, first, order, planar=True, flavour="default"):
    """One update of a 6-plane circular tensor by the reference's divergent kernel (oracle/ref/fklref_circular.cpp): the
    sequences CircularTensor::update builds (core/data/circular_tensor.h:121-134), launched as its comment does (:136-142).
    `visible` / `hidden` are device tensors of 6 planes; `first` is the caller's m_nextUpdateIdx; order 0 newest first."""
    r = (C.c_int * 4)(*[int(v) for v in rect])
    fn = lib(flavour).fklref_gpu_circular_update_planar6 if planar else lib(flavour).fklref_gpu_circular_update_packed6
    if fn(_p(frame), w, h, pitch, r, dw, dh, _f3(bg), _f3(d0), _f3(mean), _f3(std), _p(visible), _p(hidden), int(first), int(order)) != 0:
        raise RuntimeError("the reference's divergent kernel did not launch")


def divergent_four_groups64(srcs, w, h, pitch, mul, sub, add, div, dw, dh, g0, g1, g2, g3, flavour="default"):
    """Configuration 5B as one launch of the reference's divergent kernel (oracle/ref/fklref_circular.cpp): 64 images, four
    chains on four groups of 16; g0..g3 are the groups' dense output tensors."""
    if lib(flavour).fklref_gpu_divergent_four_groups64(_ptrs(srcs), w, h, pitch, _f3(mul), _f3(sub), _f3(add), _f3(div), dw, dh,
                                                       _p(g0), _p(g1), _p(g2), _p(g3)) != 0:
        raise RuntimeError("the reference's divergent kernel did not launch")
