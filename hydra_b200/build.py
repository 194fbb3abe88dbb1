"""Builds libhydra_cuda.so from hydra_b200/csrc with nvcc for sm_100a.

The library is built in-tree (hydra_b200/lib/) so that it travels with the repository to a GPU
machine; nvcc cross-compiles without a GPU.  Each .cu file is compiled to an object of its own (in
parallel, only when it or a header changed) and the objects are linked with the CUDA runtime and
NCCL.  Usage: python -m hydra_b200.build [--force] [-v]
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libhydra_cuda.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def headers():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.hpp")) \
        + glob.glob(os.path.join(INCLUDE, "*.h"))


def nccl_paths():
    """Include and library directories of the NCCL that ships with torch's CUDA wheels (the image
    has no system-wide nccl.h); empty strings when it is not there."""
    try:
        import nvidia.nccl as pkg
        root = list(pkg.__path__)[0]
    except Exception:
        return "", ""
    inc, lib = os.path.join(root, "include"), os.path.join(root, "lib")
    if os.path.exists(os.path.join(inc, "nccl.h")) and glob.glob(os.path.join(lib, "libnccl.so*")):
        return inc, lib
    return "", ""


def _compile(job):
    src, obj, flags, verbose = job
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    subprocess.check_call(cmd, cwd=CSRC)


def build(force: bool = False, verbose: bool = False, defines=(), out: str = LIB) -> str:
    """Compiles what is stale and links `out`.  `defines` (e.g. ["HC_X=1"]) are passed as -D and
    give the objects a directory of their own, so variant builds do not disturb the product's."""
    tag = "obj" if not defines else "obj_" + "_".join(d.replace("=", "-") for d in defines)
    obj_dir = os.path.join(LIB_DIR, tag)
    os.makedirs(obj_dir, exist_ok=True)
    inc, lib = nccl_paths()
    flags = ["-D" + d for d in defines] + (["-I" + inc, "-DHC_HAVE_NCCL=1"] if inc else [])
    newest_header = max([os.path.getmtime(p) for p in headers()] + [os.path.getmtime(__file__)])
    jobs, objects = [], []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), newest_header):
            jobs.append((src, obj, flags, verbose))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as pool:
            list(pool.map(_compile, jobs))
    if jobs or not os.path.exists(out) or any(os.path.getmtime(o) > os.path.getmtime(out) for o in objects):
        nvcc = os.environ.get("NVCC", "nvcc")
        link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a"] + objects + ["-o", out]
        if lib:
            # libnccl.so.2 is found at run time through the rpath, or is already in the process
            # when torch was imported first.
            soname = os.path.basename(sorted(glob.glob(os.path.join(lib, "libnccl.so*")))[0])
            link += ["-L" + lib, "-Xlinker", "-l:" + soname, "-Xlinker", "-rpath," + lib]
        subprocess.check_call(link, cwd=CSRC)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
