"""ctypes mirror of include/fkb200.h.

Python here is harness only (tests, benchmark, smoke check): the product is the C-ABI
shared library built from csrc/.  The structures below must match the header field for
field; tests/test_abi_layout.py checks their sizes against the compiled library.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CHECK_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfkb200_check.so"   # the bounds-checking build (tests only)
LIB_PATH = PKG_DIR / "lib" / "libfkb200.so"

# status codes -------------------------------------------------------------------------
OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_UNSUPPORTED = 2
ERR_CUDA = 3
ERR_TOO_LARGE = 4
ERR_NO_DEVICE = 5
ERR_DEVICE_WAIT = 6
ERR_DEVICE_BOUNDS = 7

# vocabulary ---------------------------------------------------------------------------
SRC_U8X3, SRC_F32X3, SRC_NV12, SRC_NV21, SRC_P010, SRC_P210, SRC_Y210, SRC_UYVY = 1, 2, 3, 4, 5, 6, 7, 8
DST_F32X3_PACKED, DST_F32_PLANAR3, DST_U8X3_PACKED, DST_I32X3_PACKED, DST_U32X3_PACKED = 1, 2, 3, 4, 5
RESIZE_NONE, RESIZE_IGNORE_AR, RESIZE_PRESERVE_AR, RESIZE_PRESERVE_AR_RN_EVEN, RESIZE_PRESERVE_AR_LEFT = 0, 1, 2, 3, 4
GEOMETRY_WARP_AFFINE, GEOMETRY_WARP_PERSPECTIVE = 5, 6
BORDER_NONE, BORDER_CONSTANT, BORDER_REPLICATE, BORDER_REFLECT, BORDER_WRAP, BORDER_REFLECT_101 = range(6)
DEINTERLACE_NONE, DEINTERLACE_BLEND, DEINTERLACE_LINEAR_EVEN, DEINTERLACE_LINEAR_ODD = range(4)
PLANE_DEFAULT_VALUE = 1
(OP_MUL, OP_SUB, OP_DIV, OP_ADD, OP_CAST_F32, OP_SWAP_RB, OP_SATURATE_CAST_U8,
 OP_YUV_TO_RGB_BT709_FULL, OP_CAST_I32, OP_CAST_U32) = range(1, 11)
OP_YUV_TO_RGB_BT601_FULL, OP_YUV_TO_RGB_BT2020_FULL = 11, 12
PLAN_WAIT_LIMIT_US, PLAN_TEST_EXPECT_EXTRA_BYTES, PLAN_TEST_SHRINK_BOUNDS = 1, 2, 3
DEFAULT_WAIT_LIMIT_US = 100000
ASYNC_ARENA_BYTES = 8 * 1024 * 1024


class Op(C.Structure):
    _fields_ = [("opcode", C.c_int32), ("p", C.c_float * 3)]


class Sequence(C.Structure):
    _fields_ = [
        ("src_format", C.c_int32),
        ("dst_format", C.c_int32),
        ("resize_mode", C.c_int32),
        ("n_ops", C.c_int32),
        ("n_pre_ops", C.c_int32),
        ("background", C.c_float * 3),
        ("ops", C.POINTER(Op)),
        ("border_mode", C.c_int32),
        ("border_value", C.c_float * 3),
        ("deinterlace", C.c_int32),
        ("transform", C.c_float * 9),
    ]


class Plane(C.Structure):
    _fields_ = [
        ("src", C.c_void_p),
        ("src_width", C.c_uint32),
        ("src_height", C.c_uint32),
        ("src_pitch", C.c_uint32),
        ("crop_x", C.c_int32),
        ("crop_y", C.c_int32),
        ("crop_width", C.c_int32),
        ("crop_height", C.c_int32),
        ("dst", C.c_void_p),
        ("dst_width", C.c_uint32),
        ("dst_height", C.c_uint32),
        ("dst_pitch", C.c_uint32),
        ("dst_channel_stride", C.c_uint32),
        ("sequence", C.c_int32),
        ("flags", C.c_int32),
    ]


class PlanDesc(C.Structure):
    _fields_ = [
        ("sequences", C.POINTER(Sequence)),
        ("n_sequences", C.c_int32),
        ("planes", C.POINTER(Plane)),
        ("n_planes", C.c_int32),
    ]


class ResizeParams(C.Structure):
    _fields_ = [
        ("fx", C.c_float), ("fy", C.c_float),
        ("x1", C.c_int32), ("y1", C.c_int32), ("x2", C.c_int32), ("y2", C.c_int32),
        ("target_width", C.c_int32), ("target_height", C.c_int32),
    ]


class PlanInfo(C.Structure):
    _fields_ = [
        ("n_planes", C.c_int32),
        ("n_sequences", C.c_int32),
        ("n_launches", C.c_int32),
        ("grid_x", C.c_uint32),
        ("block_x", C.c_uint32),
        ("output_pixels", C.c_uint64),
        ("algorithmic_bytes", C.c_uint64),
        ("device_bytes", C.c_uint64),
        ("n_constant_divisions", C.c_int32),
        ("n_ieee_divisions", C.c_int32),
        ("compiled_chain", C.c_int32),
        ("reserved", C.c_int32),
    ]


class DebugCounters(C.Structure):
    _fields_ = [("device_allocations", C.c_uint64), ("device_frees", C.c_uint64), ("host_pinned_allocations", C.c_uint64),
                ("plans_lowered", C.c_uint64), ("plans_reused", C.c_uint64)]


class MultiGpuShard(C.Structure):
    _fields_ = [("device", C.c_int32), ("available", C.c_int32), ("first_plane", C.c_int32), ("n_planes", C.c_int32),
                ("consolidated_output", C.c_void_p), ("consolidated_bytes", C.c_uint64), ("last_step_ms", C.c_float),
                ("reserved", C.c_int32)]


MULTI_GPU_DOWNLOAD, MULTI_GPU_GATHER = 1, 2


class CircularTensorDesc(C.Structure):
    _fields_ = [("width", C.c_uint32), ("height", C.c_uint32), ("batch", C.c_int32), ("order", C.c_int32),
                ("dst_format", C.c_int32), ("sliding", C.c_int32), ("tensor", C.c_void_p), ("ring", C.c_void_p)]


CIRCULAR_NEWEST_FIRST, CIRCULAR_OLDEST_FIRST = 0, 1


def op(opcode: int, p=(0.0, 0.0, 0.0)) -> Op:
    if isinstance(p, (int, float)):
        p = (p, p, p)
    o = Op()
    o.opcode = opcode
    o.p[0], o.p[1], o.p[2] = (float(v) for v in p)
    return o


class HostPlan:
    """Owns the ctypes arrays behind an fkb_plan_desc so they outlive the call."""

    def __init__(self):
        self._seqs: list[Sequence] = []
        self._op_arrays = []
        self._planes: list[Plane] = []
        self._desc = None

    def add_sequence(self, src_format, dst_format, resize_mode, ops, n_pre_ops=0,
                     background=(0.0, 0.0, 0.0), border_mode=0, border_value=(0.0, 0.0, 0.0), deinterlace=0,
                     transform=None) -> int:
        arr = (Op * max(len(ops), 1))(*ops)
        self._op_arrays.append(arr)
        s = Sequence()
        s.src_format, s.dst_format, s.resize_mode = src_format, dst_format, resize_mode
        s.n_ops, s.n_pre_ops = len(ops), n_pre_ops
        s.background[0], s.background[1], s.background[2] = (float(v) for v in background)
        s.ops = C.cast(arr, C.POINTER(Op))
        s.border_mode, s.deinterlace = border_mode, deinterlace
        s.border_value[0], s.border_value[1], s.border_value[2] = (float(v) for v in border_value)
        for k, v in enumerate(transform if transform is not None else [0.0] * 9):
            s.transform[k] = float(v)
        self._seqs.append(s)
        self._desc = None
        return len(self._seqs) - 1

    def add_plane(self, *, src, src_width, src_height, src_pitch, dst, dst_width, dst_height,
                  dst_pitch, dst_channel_stride=0, crop=None, sequence=0, flags=0) -> int:
        p = Plane()
        p.src, p.src_width, p.src_height, p.src_pitch = src, src_width, src_height, src_pitch
        cx, cy, cw, ch = crop if crop is not None else (0, 0, src_width, src_height)
        p.crop_x, p.crop_y, p.crop_width, p.crop_height = int(cx), int(cy), int(cw), int(ch)
        p.dst, p.dst_width, p.dst_height, p.dst_pitch = dst, dst_width, dst_height, dst_pitch
        p.dst_channel_stride, p.sequence, p.flags = dst_channel_stride, sequence, flags
        self._planes.append(p)
        self._desc = None
        return len(self._planes) - 1

    @property
    def n_planes(self) -> int:
        return len(self._planes)

    @property
    def planes(self) -> list:
        return self._planes

    def desc(self) -> PlanDesc:
        if self._desc is None:
            self._seq_arr = (Sequence * max(len(self._seqs), 1))(*self._seqs)
            self._plane_arr = (Plane * max(len(self._planes), 1))(*self._planes)
            d = PlanDesc()
            d.sequences = C.cast(self._seq_arr, C.POINTER(Sequence))
            d.n_sequences = len(self._seqs)
            d.planes = C.cast(self._plane_arr, C.POINTER(Plane))
            d.n_planes = len(self._planes)
            self._desc = d
        return self._desc


class FkbError(RuntimeError):
    """Non-zero status from the C ABI (the reference throws std::runtime_error,
    core/utils/utils.h:95-109)."""

    def __init__(self, status: int, where: str, message: str):
        super().__init__(f"{where}: status {status} ({message})")
        self.status = status


_lib = None

EXPORTS = [
    "fkb_version", "fkb_status_string", "fkb_last_error", "fkb_derive_resize",
    "fkb_reference_block_size", "fkb_plan_create", "fkb_plan_validate", "fkb_plan_launch", "fkb_plan_get_info",
    "fkb_plan_get_resize_params", "fkb_plan_destroy", "fkb_execute", "fkb_host_session_create",
    "fkb_host_session_run", "fkb_host_session_get_traffic", "fkb_host_session_destroy",
    "fkb_execute_host", "fkb_execute_static", "fkb_plan_check", "fkb_plan_set_option", "fkb_execute_async",
    "fkb_async_check", "fkb_debug_get_counters", "fkb_assign_planes", "fkb_multi_gpu_session_create",
    "fkb_multi_gpu_session_run", "fkb_multi_gpu_session_get_shard", "fkb_multi_gpu_session_destroy",
    "fkb_debug_set_device_unavailable", "fkb_circular_tensor_sizes", "fkb_circular_tensor_create", "fkb_circular_tensor_data",
    "fkb_circular_tensor_next_index", "fkb_debug_bounds_checked", "fkb_circular_tensor_plan_update", "fkb_circular_tensor_update", "fkb_circular_tensor_destroy",
]


def load_library(path: os.PathLike | None = None) -> C.CDLL:
    """Loads libfkb200.so.  There is no fallback: a missing library is an error."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = Path(path) if path else Path(os.environ.get("FKB200_LIBRARY", LIB_PATH))
    if not p.exists():
        raise FileNotFoundError(
            f"{p} not found: build it with `python -m fusedkernellibrary_b200.build` "
            "(there is no CPU or PyTorch fallback for this path)")
    lib = C.CDLL(str(p))
    lib.fkb_version.restype = C.c_int
    lib.fkb_status_string.restype = C.c_char_p
    lib.fkb_status_string.argtypes = [C.c_int]
    lib.fkb_last_error.restype = C.c_char_p
    lib.fkb_derive_resize.argtypes = [C.c_int32] * 5 + [C.POINTER(ResizeParams)]
    lib.fkb_reference_block_size.argtypes = [C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32),
                                             C.POINTER(C.c_uint32)]
    lib.fkb_plan_create.argtypes = [C.POINTER(PlanDesc), C.POINTER(C.c_void_p)]
    lib.fkb_plan_validate.argtypes = [C.POINTER(PlanDesc), C.POINTER(PlanInfo)]
    lib.fkb_plan_launch.argtypes = [C.c_void_p, C.c_void_p]
    lib.fkb_plan_get_info.argtypes = [C.c_void_p, C.POINTER(PlanInfo)]
    lib.fkb_plan_get_resize_params.argtypes = [C.c_void_p, C.c_int32, C.POINTER(ResizeParams)]
    lib.fkb_plan_destroy.argtypes = [C.c_void_p]
    lib.fkb_plan_check.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32)]
    lib.fkb_plan_set_option.argtypes = [C.c_void_p, C.c_int, C.c_uint32]
    lib.fkb_execute_async.argtypes = [C.POINTER(PlanDesc), C.c_void_p]
    lib.fkb_async_check.argtypes = [C.c_void_p, C.POINTER(C.c_uint32)]
    lib.fkb_debug_get_counters.argtypes = [C.POINTER(DebugCounters)]
    lib.fkb_assign_planes.argtypes = [C.c_int32, C.c_int32, C.POINTER(C.c_uint8), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.fkb_multi_gpu_session_create.argtypes = [C.POINTER(PlanDesc), C.c_int32, C.POINTER(C.c_int32), C.c_uint32, C.POINTER(C.c_void_p)]
    lib.fkb_multi_gpu_session_run.argtypes = [C.c_void_p]
    lib.fkb_multi_gpu_session_get_shard.argtypes = [C.c_void_p, C.c_int32, C.POINTER(MultiGpuShard)]
    lib.fkb_multi_gpu_session_destroy.argtypes = [C.c_void_p]
    lib.fkb_debug_set_device_unavailable.argtypes = [C.c_int32, C.c_int32]
    lib.fkb_execute.argtypes = [C.POINTER(PlanDesc), C.c_void_p]
    lib.fkb_execute_host.argtypes = [C.POINTER(PlanDesc), C.c_void_p]
    lib.fkb_execute_static.argtypes = [C.POINTER(PlanDesc), C.c_void_p]
    lib.fkb_host_session_create.argtypes = [C.POINTER(PlanDesc), C.POINTER(C.c_void_p)]
    lib.fkb_host_session_run.argtypes = [C.c_void_p, C.c_void_p]
    lib.fkb_host_session_get_traffic.argtypes = [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    lib.fkb_host_session_destroy.argtypes = [C.c_void_p]
    lib.fkb_circular_tensor_sizes.argtypes = [C.POINTER(CircularTensorDesc)] + [C.POINTER(C.c_size_t)] * 3
    lib.fkb_circular_tensor_create.argtypes = [C.POINTER(CircularTensorDesc), C.POINTER(C.c_void_p)]
    lib.fkb_circular_tensor_data.argtypes = [C.c_void_p]
    lib.fkb_circular_tensor_data.restype = C.c_void_p
    lib.fkb_circular_tensor_next_index.argtypes = [C.c_void_p]
    lib.fkb_circular_tensor_next_index.restype = C.c_int32
    lib.fkb_circular_tensor_plan_update.argtypes = [C.c_void_p, C.POINTER(Sequence), C.POINTER(Plane), C.POINTER(Sequence),
                                                    C.POINTER(C.c_int32), C.POINTER(Plane), C.POINTER(C.c_int32), C.c_int32]
    lib.fkb_circular_tensor_update.argtypes = [C.c_void_p, C.POINTER(Sequence), C.POINTER(Plane), C.c_void_p]
    lib.fkb_circular_tensor_destroy.argtypes = [C.c_void_p]
    if path is None:
        _lib = lib
    return lib


def check(status: int, where: str) -> None:
    if status != OK:
        lib = load_library()
        raise FkbError(status, where, (lib.fkb_last_error() or b"").decode() or
                       lib.fkb_status_string(status).decode())


class DevicePlan:
    """A plan resident on the current CUDA device (fkb_plan_create ... fkb_plan_destroy)."""

    def __init__(self, host_plan: HostPlan):
        self._lib = load_library()
        self._h = C.c_void_p()
        desc = host_plan.desc()
        check(self._lib.fkb_plan_create(C.byref(desc), C.byref(self._h)), "fkb_plan_create")

    def launch(self, stream: int | None = None) -> None:
        check(self._lib.fkb_plan_launch(self._h, C.c_void_p(stream or 0)), "fkb_plan_launch")

    def check(self, stream: int | None = None) -> int:
        """Synchronises `stream` and returns the device status word (0 = every block completed);
        raises FkbError(ERR_DEVICE_WAIT) otherwise."""
        st = C.c_uint32()
        check(self._lib.fkb_plan_check(self._h, C.c_void_p(stream or 0), C.byref(st)), "fkb_plan_check")
        return st.value

    def set_option(self, option: int, value: int) -> None:
        check(self._lib.fkb_plan_set_option(self._h, option, value), "fkb_plan_set_option")

    def info(self) -> PlanInfo:
        info = PlanInfo()
        check(self._lib.fkb_plan_get_info(self._h, C.byref(info)), "fkb_plan_get_info")
        return info

    def resize_params(self, index: int) -> ResizeParams:
        rp = ResizeParams()
        check(self._lib.fkb_plan_get_resize_params(self._h, index, C.byref(rp)),
              "fkb_plan_get_resize_params")
        return rp

    def destroy(self) -> None:
        if self._h:
            self._lib.fkb_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def validate(host_plan: HostPlan) -> PlanInfo:
    """Host-only validation and lowering of a plan description (no device needed)."""
    lib = load_library()
    info = PlanInfo()
    desc = host_plan.desc()
    check(lib.fkb_plan_validate(C.byref(desc), C.byref(info)), "fkb_plan_validate")
    return info


def execute(host_plan: HostPlan, stream: int | None = None) -> None:
    lib = load_library()
    desc = host_plan.desc()
    check(lib.fkb_execute(C.byref(desc), C.c_void_p(stream or 0)), "fkb_execute")


def execute_host(host_plan: HostPlan, stream: int | None = None) -> None:
    lib = load_library()
    desc = host_plan.desc()
    check(lib.fkb_execute_host(C.byref(desc), C.c_void_p(stream or 0)), "fkb_execute_host")


def execute_async(host_plan: HostPlan, stream: int | None = None) -> None:
    """fkb_execute_async: lower, one stream-ordered table copy from the library's pinned arena, launch; returns
    without synchronising."""
    lib = load_library()
    desc = host_plan.desc()
    check(lib.fkb_execute_async(C.byref(desc), C.c_void_p(stream or 0)), "fkb_execute_async")


def async_check(stream: int | None = None) -> int:
    """Synchronises `stream`; raises FkbError(ERR_DEVICE_WAIT) if an asynchronous launch gave up a wait."""
    lib = load_library()
    st = C.c_uint32()
    check(lib.fkb_async_check(C.c_void_p(stream or 0), C.byref(st)), "fkb_async_check")
    return st.value


def debug_counters() -> DebugCounters:
    c = DebugCounters()
    load_library().fkb_debug_get_counters(C.byref(c))
    return c


STATIC_TABLE_BYTES = 512 * 1024


def execute_static(host_plan: HostPlan, stream: int | None = None) -> None:
    """fkb_execute_static: the one-shot run that allocates no device memory (descriptor table in
    the library's fixed array; plans beyond STATIC_TABLE_BYTES raise FkbError with ERR_TOO_LARGE)."""
    lib = load_library()
    desc = host_plan.desc()
    check(lib.fkb_execute_static(C.byref(desc), C.c_void_p(stream or 0)), "fkb_execute_static")


class HostSession:
    """Device mirrors for a plan whose images are host buffers (fkb_host_session_*)."""

    def __init__(self, host_plan: HostPlan):
        self._lib = load_library()
        self._h = C.c_void_p()
        desc = host_plan.desc()
        check(self._lib.fkb_host_session_create(C.byref(desc), C.byref(self._h)), "fkb_host_session_create")

    def run(self, stream: int | None = None) -> None:
        check(self._lib.fkb_host_session_run(self._h, C.c_void_p(stream or 0)), "fkb_host_session_run")

    def traffic(self) -> tuple[int, int]:
        a, b = C.c_uint64(), C.c_uint64()
        check(self._lib.fkb_host_session_get_traffic(self._h, C.byref(a), C.byref(b)),
              "fkb_host_session_get_traffic")
        return a.value, b.value

    def destroy(self) -> None:
        if self._h:
            self._lib.fkb_host_session_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass



def assign_planes(n_planes: int, n_devices: int, available=None) -> list[tuple[int, int]]:
    """fkb_assign_planes: (first, count) per device; devices whose `available` entry is false get no planes."""
    lib = load_library()
    first, count = (C.c_int32 * n_devices)(), (C.c_int32 * n_devices)()
    avail = None if available is None else (C.c_uint8 * n_devices)(*[1 if a else 0 for a in available])
    check(lib.fkb_assign_planes(n_planes, n_devices, avail, first, count), "fkb_assign_planes")
    return [(first[d], count[d]) for d in range(n_devices)]


class MultiGpuSession:
    """One batch over several GPUs of one box (fkb_multi_gpu_session_*): host buffers in, shards by plane."""

    def __init__(self, host_plan: HostPlan, devices, flags: int = MULTI_GPU_DOWNLOAD):
        self._lib = load_library()
        self._h = C.c_void_p()
        self.devices = list(devices)
        desc = host_plan.desc()
        arr = (C.c_int32 * len(self.devices))(*self.devices)
        check(self._lib.fkb_multi_gpu_session_create(C.byref(desc), len(self.devices), arr, flags, C.byref(self._h)),
              "fkb_multi_gpu_session_create")

    def run(self) -> None:
        check(self._lib.fkb_multi_gpu_session_run(self._h), "fkb_multi_gpu_session_run")

    def shard(self, index: int) -> MultiGpuShard:
        sh = MultiGpuShard()
        check(self._lib.fkb_multi_gpu_session_get_shard(self._h, index, C.byref(sh)), "fkb_multi_gpu_session_get_shard")
        return sh

    def destroy(self) -> None:
        if self._h:
            self._lib.fkb_multi_gpu_session_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class CircularTensor:
    """fkb_circular_tensor_*: the newest `batch` results of a chain, kept in order (the reference's CircularTensor::update,
    core/data/circular_tensor.h:111-161).  `tensor` / `ring` are the caller's buffers (device pointers, or host pointers when
    only plans are wanted); None lets the library allocate on the current device."""

    def __init__(self, width, height, batch, dst_format, order=CIRCULAR_NEWEST_FIRST, sliding=False, tensor=None, ring=None):
        self._lib = load_library()
        self._h = C.c_void_p()
        d = CircularTensorDesc(width, height, batch, order, dst_format, 1 if sliding else 0, tensor, ring)
        self.desc = d
        pb, tb, rb = C.c_size_t(), C.c_size_t(), C.c_size_t()
        check(self._lib.fkb_circular_tensor_sizes(C.byref(d), C.byref(pb), C.byref(tb), C.byref(rb)), "fkb_circular_tensor_sizes")
        self.plane_bytes, self.tensor_bytes, self.ring_bytes = pb.value, tb.value, rb.value
        check(self._lib.fkb_circular_tensor_create(C.byref(d), C.byref(self._h)), "fkb_circular_tensor_create")

    @staticmethod
    def sizes(width, height, batch, dst_format, sliding=False) -> tuple[int, int, int]:
        """(plane, tensor buffer, ring buffer) in bytes."""
        lib = load_library()
        d = CircularTensorDesc(width, height, batch, CIRCULAR_NEWEST_FIRST, dst_format, 1 if sliding else 0, None, None)
        pb, tb, rb = C.c_size_t(), C.c_size_t(), C.c_size_t()
        check(lib.fkb_circular_tensor_sizes(C.byref(d), C.byref(pb), C.byref(tb), C.byref(rb)), "fkb_circular_tensor_sizes")
        return pb.value, tb.value, rb.value

    @property
    def data(self) -> int:
        return self._lib.fkb_circular_tensor_data(self._h)

    @property
    def next_index(self) -> int:
        return self._lib.fkb_circular_tensor_next_index(self._h)

    @staticmethod
    def _chain(host_plan: "HostPlan"):
        d = host_plan.desc()
        if d.n_sequences != 1 or d.n_planes != 1:
            raise ValueError("an update takes one sequence and one plane (the new image)")
        return d

    def plan_update(self, host_plan: "HostPlan", advance=True) -> "HostPlan":
        """The plan of the next update as a HostPlan; `host_plan` holds the chain and the plane of the new image."""
        d = self._chain(host_plan)
        seqs = (Sequence * 2)()
        planes = (Plane * (self.desc.batch + 1))()
        ns, np_ = C.c_int32(), C.c_int32()
        check(self._lib.fkb_circular_tensor_plan_update(self._h, d.sequences, d.planes, seqs, C.byref(ns), planes, C.byref(np_),
                                                        1 if advance else 0), "fkb_circular_tensor_plan_update")
        out = HostPlan()
        out._keep = (host_plan, seqs, planes)     # the chain's operation array lives in host_plan
        out._seqs = [seqs[i] for i in range(ns.value)]
        out._planes = [planes[i] for i in range(np_.value)]
        return out

    def update(self, host_plan: "HostPlan", stream: int | None = None) -> None:
        d = self._chain(host_plan)
        check(self._lib.fkb_circular_tensor_update(self._h, d.sequences, d.planes, stream), "fkb_circular_tensor_update")

    def destroy(self) -> None:
        if self._h:
            self._lib.fkb_circular_tensor_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass
