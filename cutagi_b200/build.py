"""Builds libtagi_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m cutagi_b200.build [--force] [--verbose]

Objects go to cutagi_b200/csrc/build/, the library to cutagi_b200/libtagi_b200.so. Only files whose sources
(or any header) are newer than their object are recompiled.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libtagi_b200.so")
COMM_SRC = os.path.join(HERE, "csrc_comm", "tagi_comm.cpp")
COMM_LIB = os.path.join(HERE, "libtagi_b200_comm.so")
NVCC = os.environ.get("NVCC", "nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xptxas", "-v", "--expt-relaxed-constexpr"]


def _newer(a, b):
    return not os.path.exists(b) or os.path.getmtime(a) > os.path.getmtime(b)


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(os.path.dirname(HERE), "include", "*.h"))
    jobs = []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s)[:-3] + ".o")
        if force or _newer(s, o) or any(_newer(h, o) for h in hdrs):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        r = subprocess.run([NVCC, *FLAGS, "-c", s, "-o", o], capture_output=True, text=True)
        log = r.stdout + r.stderr
        with open(o + ".log", "w") as f:
            f.write(log)
        if r.returncode != 0:
            if os.path.exists(o):
                os.remove(o)
            raise RuntimeError(f"nvcc failed on {s}:\n{log[-4000:]}")
        if verbose:
            print(log)
        return o

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    objs = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in srcs]
    if force or jobs or not os.path.exists(LIB):
        r = subprocess.run([NVCC, "-shared", "-o", LIB, *objs, "-lcudart"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    build_comm(force)
    return LIB


def build_comm(force=False):
    """libtagi_b200_comm.so: host-only C++ over NCCL (kept apart so that the kernel library does not depend on NCCL)."""
    hdrs = glob.glob(os.path.join(os.path.dirname(HERE), "include", "*.h"))
    if force or _newer(COMM_SRC, COMM_LIB) or any(_newer(h, COMM_LIB) for h in hdrs):
        r = subprocess.run([NVCC, "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-o", COMM_LIB, COMM_SRC,
                            "-lnccl", "-lcudart"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("comm library build failed:\n" + r.stdout + r.stderr)
    return COMM_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
