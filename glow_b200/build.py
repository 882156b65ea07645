"""Builds the CUDA library of this package in-tree: glow_b200/lib/libglow_b200.so.

Every .cu file under glow_b200/csrc is compiled for sm_100a only
(-gencode arch=compute_100a,code=sm_100a) and linked into one shared library that exports
the C ABI declared in include/glow_b200.h.  Run as `python -m glow_b200.build`.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libglow_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"), "-I", CSRC]


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(ROOT, "include", "glow_b200.h"))
    return hs


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, extra_flags=()):
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    srcs, hdrs = _sources(), _headers()
    jobs = []
    objs = []
    for src in srcs:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if _stale(obj, [src] + hdrs):
            jobs.append([NVCC] + NVCC_FLAGS + list(extra_flags) + ["-c", src, "-o", obj])

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n%s\n%s" % (" ".join(cmd), r.stderr))
        if verbose and r.stderr.strip():
            print(r.stderr, flush=True)
        return r.stderr

    with ThreadPoolExecutor(max(1, min(8, len(jobs)))) as ex:
        list(ex.map(run, jobs))
    if jobs or _stale(LIB, objs):
        run([NVCC, "-shared", "-o", LIB] + objs)
    return LIB


if __name__ == "__main__":
    flags = [a for a in sys.argv[1:] if a != "-v"]
    print(build(verbose="-v" in sys.argv[1:], extra_flags=flags))
