"""Builds the sm_100a shared library behind include/sgq.h with nvcc, in-tree.

    python soverign-grad_b200/build.py [--force] [--verbose]

Output: soverign-grad_b200/lib/libsgq.so (git-ignored; it travels with the source tree).
nvcc cross-compiles without a GPU.  One object per .cu, compiled in parallel.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(LIB_DIR, "libsgq.so")
SOURCES = ["abi.cu", "quantize.cu", "linear_simt.cu", "gemv.cu", "gemm_tc.cu", "decoder_glue.cu", "peer.cu", "gemv_i8.cu", "linear_kn.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _deps(src: str) -> list[str]:
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    return [src, os.path.join(os.path.dirname(HERE), "include", "sgq.h"), *hdrs]


def _stale(out: str, deps: list[str]) -> bool:
    return not os.path.exists(out) or any(os.path.getmtime(d) > os.path.getmtime(out) for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    jobs = []
    for name in SOURCES:
        src = os.path.join(CSRC, name)
        obj = os.path.join(OBJ_DIR, name.replace(".cu", ".o"))
        if force or _stale(obj, _deps(src)):
            cmd = [NVCC, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", src, "-o", obj]
            jobs.append((name, cmd))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            futs = {ex.submit(subprocess.run, cmd, capture_output=True, text=True): name for name, cmd in jobs}
            for fut in cf.as_completed(futs):
                r = fut.result()
                if verbose or r.returncode != 0:
                    sys.stderr.write(f"--- {futs[fut]} ---\n{r.stdout}{r.stderr}\n")
                if r.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {futs[fut]}")
    objs = [os.path.join(OBJ_DIR, n.replace(".cu", ".o")) for n in SOURCES]
    if force or jobs or _stale(LIB, objs):
        # cudart is linked statically; the driver entry point for tensor maps is resolved at run time
        subprocess.check_call([NVCC, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
                               "-Xcompiler", "-fPIC"])
    return LIB


HOST_DIR = os.path.join(HERE, "host")
HOST_LIB = os.path.join(LIB_DIR, "libsgq_host.so")
HOST_TEST = os.path.join(LIB_DIR, "sgq_host_test")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"


def build_host(force: bool = False) -> str:
    """The C++17 host layer (pool, tensor, quantization API, layers) and its test driver."""
    build()
    srcs = [os.path.join(HOST_DIR, "src", f) for f in sorted(os.listdir(os.path.join(HOST_DIR, "src"))) if f.endswith(".cpp")]
    hdrs = [os.path.join(HOST_DIR, "include", "sovereigngrad", f)
            for f in os.listdir(os.path.join(HOST_DIR, "include", "sovereigngrad"))]
    inc = ["-I", os.path.join(HOST_DIR, "include"), "-I", os.path.join(os.path.dirname(HERE), "include"),
           "-I", os.path.join(CUDA_HOME, "include")]
    link = ["-L", LIB_DIR, "-lsgq", "-L", os.path.join(CUDA_HOME, "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN",
            "-Wl,-rpath," + os.path.join(CUDA_HOME, "lib64")]
    if force or _stale(HOST_LIB, srcs + hdrs + [LIB]):
        subprocess.check_call([CXX, "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", *inc, *srcs, "-o", HOST_LIB, *link])
    test_src = os.path.join(os.path.dirname(HERE), "tests", "host_test.cpp")
    if force or _stale(HOST_TEST, [test_src, HOST_LIB] + hdrs):
        subprocess.check_call([CXX, "-std=c++17", "-O2", "-Wall", *inc, test_src, "-o", HOST_TEST, "-L", LIB_DIR, "-lsgq_host",
                               *link])
    return HOST_LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    print(build_host(a.force))
