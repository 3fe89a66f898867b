"""Builds libfkb200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m fusedkernellibrary_b200.build [--force] [--verbose]

Every translation unit under csrc/ is compiled to an object file on its own (in parallel; only
the stale ones) and the objects are linked into one shared library.
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


def needs_build() -> bool:
    return _stale(OUT, sources() + _headers())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return OUT
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = _headers()

    def compile_one(src: Path):
        obj = OBJ / (src.stem + ".o")
        if not force and not _stale(obj, [src] + headers):
            return obj, ""
        cmd = ["nvcc", *NVCC_FLAGS, f"-I{ROOT / 'include'}", f"-I{CSRC}"]
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
    r = subprocess.run(["nvcc", *LINK_FLAGS, *objs, "-o", str(OUT)], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("linking libfkb200.so failed")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
