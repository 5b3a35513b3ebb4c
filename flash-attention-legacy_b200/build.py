"""Builds the C-ABI shared library `lib/libfal_b200.so` with plain nvcc for sm_100a.

Usage:  python build.py [--force] [--verbose] [--out PATH] [--define NAME[=VALUE] ...]

`--define` adds -D flags (the kernels' tuning switches and cycle counters, e.g.
`--define FAL_FWD_TIMING --out /tmp/libfal_timing.so`); `--out` keeps such a build away from
the product library.  A library built elsewhere is used through FAL_B200_LIB.

This replaces the reference's torch CUDAExtension build (setup.py:48-82 of
sirCamp/flash-attention-legacy): there are no torch headers on the native side,
and exactly one target architecture.
"""
import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(LIB_DIR, "libfal_b200.so")

SOURCES = ["fal_api.cu", "fal_fwd.cu", "fal_bwd.cu", "fal_decode.cu", "fal_ring.cu", "fal_selftest.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found; the library cannot be built")
    return path


def _newest_source_mtime():
    names = [n for n in os.listdir(CSRC) if n.endswith((".cu", ".cuh", ".h"))]
    paths = [os.path.join(CSRC, n) for n in names]
    paths.append(os.path.join(HERE, "..", "include", "fal_b200.h"))
    paths.append(os.path.abspath(__file__))
    return max(os.path.getmtime(p) for p in paths)


def up_to_date():
    return os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest_source_mtime()


def build(force=False, verbose=False, out=None, defines=()):
    """Compiles every source file and links the shared library. Returns its path."""
    variant = out is not None or bool(defines)
    lib_path = os.path.abspath(out) if out else LIB_PATH
    if variant and lib_path == LIB_PATH:
        raise RuntimeError("a build with --define needs --out: the product library takes no tuning flags")
    if not variant and not force and up_to_date():
        return LIB_PATH
    nvcc = _nvcc()
    obj_dir = OBJ_DIR if not variant else lib_path + ".obj"
    os.makedirs(os.path.dirname(lib_path), exist_ok=True)
    os.makedirs(obj_dir, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []
    extra += ["-D" + d for d in defines]

    def compile_one(src):
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    cmd = [nvcc, "-shared", "-o", lib_path, *objs, "-cudart", "static"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link failed")
    return lib_path


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--out", default=None, help="write the library here instead of lib/libfal_b200.so")
    ap.add_argument("--define", action="append", default=[], metavar="NAME[=VALUE]")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, out=a.out, defines=a.define))
