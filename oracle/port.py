"""ctypes binding of oracle/fkl_oracle.c (the plain-C restatement).

TEST INFRASTRUCTURE ONLY: the checker the CUDA path is compared with.  Parity status:
pinned against the reference's own headers (see fkl_oracle.c header).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

from fusedkernellibrary_b200 import abi

HERE = Path(__file__).resolve().parent
LIB = HERE / "libfkl_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    src = HERE / "fkl_oracle.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "port"], check=True, capture_output=True)
    return LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB.exists():
            build()
        _lib = C.CDLL(str(LIB))
        _lib.fkl_oracle_run.argtypes = [C.POINTER(abi.PlanDesc), C.c_int]
        _lib.fkl_oracle_run_range.argtypes = [C.POINTER(abi.PlanDesc), C.c_int, C.c_int, C.c_int]
        _lib.fkl_oracle_derive_resize.argtypes = [C.c_int] * 5 + [C.POINTER(abi.ResizeParams)]
        _lib.fkl_oracle_block_size.argtypes = [C.c_uint, C.c_uint, C.POINTER(C.c_uint), C.POINTER(C.c_uint)]
        _lib.fkl_oracle_block_size.restype = None
    return _lib


def run(host_plan: abi.HostPlan, host_branch: bool = False, first: int = 0, count: int | None = None) -> None:
    """Runs a plan whose src/dst pointers are HOST pointers (e.g. numpy buffers)."""
    d = host_plan.desc()
    n = host_plan.n_planes - first if count is None else count
    rc = lib().fkl_oracle_run_range(C.byref(d), first, n, int(host_branch))
    if rc != 0:
        raise ValueError("oracle: malformed plan")


def derive_resize(sw, sh, dw, dh, mode) -> abi.ResizeParams:
    rp = abi.ResizeParams()
    if lib().fkl_oracle_derive_resize(sw, sh, dw, dh, mode, C.byref(rp)) != 0:
        raise ValueError("oracle: bad resize arguments")
    return rp


def block_size(w, h) -> tuple[int, int]:
    bx, by = C.c_uint(), C.c_uint()
    lib().fkl_oracle_block_size(w, h, C.byref(bx), C.byref(by))
    return bx.value, by.value
