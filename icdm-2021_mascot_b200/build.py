"""In-tree build of libmascot.so (hand-written CUDA for sm_100a) and the C++ command-line tools.

    python icdm-2021_mascot_b200/build.py [--force]

nvcc cross-compiles without a GPU, so this also runs on a CPU-only machine.  The shared library
exports exactly the C ABI declared in include/mascot.h.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
CLI = os.path.join(HERE, "cli")
LIB = os.path.join(HERE, "libmascot.so")
BIN = os.path.join(HERE, "bin")

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

LIB_SOURCES = ["mascot_api.cu", "setup.cu", "shard.cu", "train_kernels.cu", "eval_kernels.cu", "prep_kernels.cu", "probe.cu"]
CLI_SOURCES = {"quantized_mf": "quantized_mf.cpp", "test_mf": "test_mf.cpp", "convert_ratings": "convert_ratings.cpp"}


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build_library(force=False, verbose=True, ptxas_verbose=False):
    srcs = [os.path.join(CSRC, s) for s in LIB_SOURCES]
    deps = srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    deps.append(os.path.join(ROOT, "include", "mascot.h"))
    if not force and not _newer(LIB, deps):
        return LIB
    objs = []
    for s in srcs:
        o = s[:-3] + ".o"
        if force or _newer(o, deps):
            cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_verbose else []) + ["-c", s, "-o", o]
            _run(cmd, verbose)
        objs.append(o)
    _run(["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs + ["-lcudart", "-ldl"], verbose)
    return LIB


def build_cli(force=False, verbose=True):
    os.makedirs(BIN, exist_ok=True)
    out = []
    for name, src in CLI_SOURCES.items():
        s = os.path.join(CLI, src)
        if not os.path.exists(s):
            continue
        exe = os.path.join(BIN, name)
        deps = [s, os.path.join(ROOT, "include", "mascot.h")] + \
               [os.path.join(CLI, f) for f in os.listdir(CLI) if f.endswith(".h")]
        if force or _newer(exe, deps) or _newer(exe, [LIB]):
            _run(["g++", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"), s, "-o", exe,
                  "-L", HERE, "-lmascot", "-lpthread", "-Wl,-rpath," + HERE, "-Wl,-rpath,$ORIGIN/.."], verbose)
        out.append(exe)
    return out


def build_all(force=False, verbose=True):
    build_library(force, verbose)
    build_cli(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
