"""Build the library: every CUDA/C++ source under csrc/ and host/ -> lib/libotter_b200.so (sm_100a only).

    python -m tensor_b200.build          # incremental
    python -m tensor_b200.build --force

nvcc cross-compiles without a GPU. The arch is given as an explicit -gencode: a plain -arch=sm_100a adds a
compute_100 pass on which the tcgen05 instructions do not assemble.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
HOST = PKG / "host"
LIBDIR = PKG / "lib"
OBJDIR = PKG / "lib" / "obj"
LIB = LIBDIR / "libotter_b200.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
    "-fmad=false",  # every FMA of the bit-exact epilogue is written explicitly; the compiler must not add any
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function", "-I", str(PKG.parent / "include"),
    "-DOTT_BUILDING_LIBRARY",
]


def sources():
    return sorted(list(CSRC.glob("*.cu")) + list(HOST.glob("*.cpp")))


def headers_mtime() -> float:
    hs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(HOST.glob("*.hpp")) + list((PKG.parent / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def compile_one(src: Path, force: bool, hdr_mtime: float, verbose: bool) -> Path:
    obj = OBJDIR / (src.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_mtime):
        return obj
    cmd = [NVCC, *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJDIR.mkdir(parents=True, exist_ok=True)
    hdr = headers_mtime()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: compile_one(s, force, hdr, verbose), srcs))
    if force or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [NVCC, "-shared", "-o", str(LIB), *map(str, objs), "-lpthread", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/spill/shared-memory usage")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
