"""Builds libgptoss_b200.so: every .cu under csrc/ compiled for sm_100a and linked
into one shared library beside this file.

    python optimize_inference_gpt-oss_b200/build.py [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects are rebuilt only when a source or
header is newer.  The library links the CUDA runtime statically, so at run time
it needs nothing but the driver.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_build")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libgptoss_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden,-pthread",
          "-ccbin", "g++"]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".hpp"))]
    hs += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return hs


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src: str, verbose: bool, obj_dir: str = OBJ, defines=()) -> str:
    obj = os.path.join(obj_dir, src[:-3] + ".o")
    cmd = [NVCC, *ARCH, *CFLAGS, *defines, "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, lib: str = LIB, obj_dir: str = OBJ, defines=()) -> str:
    os.makedirs(obj_dir, exist_ok=True)
    hdrs = _headers()
    todo, objs = [], []
    for s in _sources():
        obj = os.path.join(obj_dir, s[:-3] + ".o")
        objs.append(obj)
        if force or _newer(obj, [os.path.join(CSRC, s), *hdrs]):
            todo.append(s)
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            list(ex.map(lambda s: _compile(s, verbose, obj_dir, defines), todo))
    if todo or not os.path.exists(lib):
        cmd = [NVCC, *ARCH, "-shared", "-Xcompiler", "-fPIC,-pthread", "-ccbin", "g++", "-o", lib, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


# The checked build: the same sources with -DGPTOSS_BOUNDS (every pointer argument held against
# the allocation it lies in, data-dependent row numbers held against their arrays; see
# csrc/common.cuh).  The GPU tests run their small cases through it as well.
BOUNDS_LIB = os.path.join(HERE, "libgptoss_b200_bounds.so")


def build_bounds(force: bool = False, verbose: bool = False) -> str:
    return build(force, verbose, BOUNDS_LIB, os.path.join(CSRC, "_build_bounds"), ("-DGPTOSS_BOUNDS",))


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--bounds" in sys.argv:
        print(build_bounds(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
