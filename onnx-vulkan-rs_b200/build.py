"""Builds libovk_cuda.so (every .cu under csrc/) for sm_100a with nvcc, then
libovk_host.so (host/*.cpp, the node-level layer above the C ABI) with g++.

Usage: python build.py [--force] [--verbose]
nvcc cross-compiles without a GPU; objects are cached under csrc/build/ by
source mtime.  -fmad=false keeps separate float multiplies and adds separately
rounded (the kernels spell out every fused multiply-add they want).
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libovk_cuda.so")
HOST_DIR = os.path.join(HERE, "host")
HOST_OUT = os.path.join(HERE, "libovk_host.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", os.path.join(ROOT, "include"),
    "-I", CSRC, "--expt-relaxed-constexpr", "-ccbin", "/usr/bin/g++",
]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h")) + [os.path.abspath(__file__)]
    objdir = os.path.join(CSRC, "build")
    os.makedirs(objdir, exist_ok=True)
    jobs = []
    objs = []
    for src in srcs:
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [NVCC, *FLAGS, "-c", src, "-o", obj] + (["-Xptxas", "-v"] if verbose else [])
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode:
                sys.stderr.write(" ".join(cmd[-4:]) + "\n" + r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {cmd[-3]}")
    if jobs or force or _stale(OUT, objs):
        link = [NVCC, "-shared", "-o", OUT, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
                "-ccbin", "/usr/bin/g++", "-lcudart"]
        r = subprocess.run(link, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    build_host(force)
    return OUT


def build_host(force: bool = False) -> str:
    """The C++ host layer: plain g++, linked against libovk_cuda.so beside it."""
    srcs = sorted(glob.glob(os.path.join(HOST_DIR, "*.cpp")))
    deps = srcs + glob.glob(os.path.join(HOST_DIR, "*.hpp")) + glob.glob(os.path.join(ROOT, "include", "*.h")) + [OUT]
    if force or _stale(HOST_OUT, deps):
        cmd = ["/usr/bin/g++", "-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra", "-shared",
               "-I", os.path.join(ROOT, "include"), *srcs, "-o", HOST_OUT, "-L", HERE, "-lovk_cuda",
               "-Wl,-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("host layer build failed")
    return HOST_OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
