"""Builds the CUDA library of this package in-tree for sm_100a.

    python cccc-lite_b200/build.py            # build if sources are newer than the library
    python cccc-lite_b200/build.py --force

The output is cccc-lite_b200/libcccc-cuda-b200.so, the drop-in for the reference's
`cccc-cuda` plug-in library on the quantized-weight linear path (see include/cccc_cuda_b200.h).
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcccc-cuda-b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--extended-lambda",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared", "-cudart", "shared",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


HOST_LIB = os.path.join(HERE, "libcccc-b200-host.so")
HOST_DIR = os.path.join(CSRC, "host")


def host_stale() -> bool:
    if not os.path.exists(HOST_LIB):
        return True
    t = os.path.getmtime(HOST_LIB)
    deps = glob.glob(os.path.join(HOST_DIR, "*")) + glob.glob(os.path.join(HERE, "..", "include", "*.h")) + [LIB]
    return any(os.path.getmtime(d) > t for d in deps)


def build_host(force: bool = False) -> str:
    """The C++ host layer (Matrix / Cublas / GpuControl mirror) on top of the CUDA library."""
    if force or host_stale():
        cuda = os.path.dirname(os.path.dirname(NVCC))
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-pthread", "-shared", "-fvisibility=hidden", f"-I{cuda}/include", "-o", HOST_LIB]
        cmd += sorted(glob.glob(os.path.join(HOST_DIR, "*.cpp")))
        cmd += [f"-L{HERE}", "-lcccc-cuda-b200", f"-L{cuda}/lib64", "-lcublas", "-lcudart", "-Wl,-rpath,$ORIGIN"]
        subprocess.check_call(cmd)
    return HOST_LIB


OBJ_DIR = os.path.join(HERE, "build")    # git-ignored object files: only changed translation units are recompiled


def _object_stale(src: str, obj: str) -> bool:
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    deps = [src] + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every translation unit of csrc/ for sm_100a (in parallel, only the stale ones) and links the library."""
    if force or stale():
        from concurrent.futures import ThreadPoolExecutor

        os.makedirs(OBJ_DIR, exist_ok=True)
        compile_flags = [f for f in FLAGS if f != "-shared"]
        extra = os.environ.get("B200_NVCC_EXTRA", "").split()
        jobs = []
        for src in sources():
            obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
            if force or extra or _object_stale(src, obj):
                jobs.append([NVCC] + compile_flags + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", obj, src])
        with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
            for rc in pool.map(subprocess.call, jobs):
                if rc != 0:
                    raise subprocess.CalledProcessError(rc, "nvcc")
        objs = [os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o") for src in sources()]
        subprocess.check_call([NVCC, "-shared", "-cudart", "shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs)
    build_host(force)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
