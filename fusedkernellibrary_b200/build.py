"""Builds libfkb200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m fusedkernellibrary_b200.build [--force] [--verbose] [--check]

Every translation unit under csrc/ is compiled to an object file on its own (in parallel; only
the stale ones) and the objects are linked into one shared library.  --check builds
libfkb200_check.so instead: the same sources with -DFKB_CHECK_BOUNDS, in which every access of a
kernel to an image or to shared memory is compared with what its plane allows before it is made
(tests only; see fkb_debug_bounds_checked in include/fkb200.h).
"""
from __future__ import annotations

import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "lib" / "obj"
OUT = PKG / "lib" / "libfkb200.so"
OBJ_CHECK = PKG / "lib" / "obj_check"
OUT_CHECK = PKG / "lib" / "libfkb200_check.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # every rounding on this path must match the reference's separate multiply and add
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC,-ffp-contract=off,-fvisibility=hidden,-Wall",
]
LINK_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static", "-ldl", "-lpthread"]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + [ROOT / "include" / "fkb200.h", Path(__file__)]


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def needs_build(check: bool = False) -> bool:
    return _stale(OUT_CHECK if check else OUT, sources() + _headers())


def build(force: bool = False, verbose: bool = False, check: bool = False) -> Path:
    out, obj_dir = (OUT_CHECK, OBJ_CHECK) if check else (OUT, OBJ)
    if not force and not needs_build(check):
        return out
    obj_dir.mkdir(parents=True, exist_ok=True)
    headers = _headers()

    def compile_one(src: Path):
        obj = obj_dir / (src.stem + ".o")
        if not force and not _stale(obj, [src] + headers):
            return obj, ""
        cmd = ["nvcc", *NVCC_FLAGS, f"-I{ROOT / 'include'}", f"-I{CSRC}"]
        if check:
            cmd += ["-DFKB_CHECK_BOUNDS"]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}{r.stderr}")
        return obj, r.stdout + r.stderr

    with ThreadPoolExecutor(max_workers=8) as pool:
        results = list(pool.map(compile_one, sources()))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    objs = [str(o) for o, _ in results]
    r = subprocess.run(["nvcc", *LINK_FLAGS, *objs, "-o", str(out)], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"linking {out.name} failed")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, check="--check" in sys.argv))
