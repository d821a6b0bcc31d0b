"""In-tree build of the native libraries (nvcc / g++, no build system needed).

    python -m kernelcodegen_b200.build            # build what is out of date
    python -m kernelcodegen_b200.build --force    # rebuild everything

Produces, inside the package directory:
    lib/libkcg_kernels.so   the sm_100a kernels behind the C ABI of include/kcg_kernels.h
    lib/libkcg_runtime.so   the C++ KernelCodeGen front end (graph builder + dispatch)
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
FRONT = PKG / "frontend"
LIB = PKG / "lib"
OBJ = PKG / "build"
INCLUDE = ROOT / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-I", str(INCLUDE), "-I", str(CSRC),
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return exe


def _newer(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))
    if proc.stderr.strip():
        sys.stderr.write(proc.stderr)


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile csrc/*.cu for sm_100a and link lib/libkcg_kernels.so."""
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", str(src), "-o", str(obj)]
            jobs.append(cmd)
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(_run, jobs))
    out = LIB / "libkcg_kernels.so"
    if jobs or not out.exists():
        _run([nvcc, "-shared", "-cudart", "static", "-o", str(out)] + [str(o) for o in objs] + ["-ldl"])
    return out


def build_frontend(force: bool = False) -> Path | None:
    """Compile the C++ front end (frontend/*.cc) into lib/libkcg_runtime.so."""
    sources = sorted(FRONT.glob("*.cc"))
    if not sources:
        return None
    LIB.mkdir(exist_ok=True)
    out = LIB / "libkcg_runtime.so"
    headers = list(INCLUDE.rglob("*.h"))
    if force or _newer(out, sources + headers):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-I", str(INCLUDE), "-o", str(out)]
             + [str(s) for s in sources]
             + ["-L", str(LIB), "-lkcg_kernels", "-Wl,-rpath,$ORIGIN"])
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_frontend(force=force)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / shared-memory usage")
    a = ap.parse_args()
    build_all(force=a.force, verbose=a.verbose)
    print("built:", ", ".join(str(p.relative_to(ROOT)) for p in sorted(LIB.glob("*.so"))))
