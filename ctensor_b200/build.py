"""In-tree build of libctb200.so for sm_100a (nvcc cross-compiles without a GPU).

    python -m ctensor_b200.build [--force]

The arithmetic flags are part of the numerical contract: no implicit FMA contraction, IEEE
division and square root, denormals kept (the reference's CPU paths keep them).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libctb200.so")
SOURCES = ["ctb_abi.cu", "ctb_elementwise.cu", "ctb_reduce.cu", "ctb_rows.cu", "ctb_index.cu", "ctb_optim.cu", "ctb_norm.cu", "ctb_matmul.cu", "ctb_pool.cu", "ctb_backward.cu", "ctb_comm.cu", "ctb_matmul_tc.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC", "-Wno-deprecated-gpu-targets",
]


def _newest_input() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    paths.append(os.path.join(os.path.dirname(PKG), "include", "ctb200.h"))
    paths.append(os.path.abspath(__file__))
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, extra_flags=(), verbose: bool = False) -> str:
    """CTB_NVCC_EXTRA (environment): extra nvcc flags, e.g. the -D knobs named in the kernels'
    sources, for measurement builds (`CTB_NVCC_EXTRA=-DCTB_GELU_VARIANT=1 python -m ctensor_b200.build --force`)."""
    extra_flags = tuple(extra_flags) + tuple(os.environ.get("CTB_NVCC_EXTRA", "").split())
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_input():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(OBJ, exist_ok=True)

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    subprocess.check_call([nvcc, "-shared", "-Wno-deprecated-gpu-targets", "-o", LIB, *objs, "-ldl"])
    return LIB


HOST_DIR = os.path.join(PKG, "host")
HOST_LIB = os.path.join(PKG, "libctensor_host.so")
HOST_BENCH = os.path.join(HOST_DIR, "bench_host_layer.bin")


def build_host(force: bool = False) -> str:
    """The C++ host layer (the reference's operator API over the C ABI): plain g++, it needs
    neither nvcc nor the CUDA headers — everything CUDA is behind libctb200.so."""
    src = os.path.join(HOST_DIR, "ctensor_host.cpp")
    deps = [src, os.path.join(os.path.dirname(PKG), "include", "ctb200.h"), os.path.join(HOST_DIR, "bench_host_layer.cpp")]
    deps += [os.path.join(HOST_DIR, "include", f) for f in os.listdir(os.path.join(HOST_DIR, "include"))]
    if not force and os.path.exists(HOST_LIB) and os.path.exists(HOST_BENCH) and os.path.getmtime(HOST_LIB) >= max(map(os.path.getmtime, deps)) \
            and os.path.getmtime(HOST_LIB) >= os.path.getmtime(LIB):
        return HOST_LIB
    subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra", "-o", HOST_LIB, src,
                           "-I", HOST_DIR, "-L", PKG, "-lctb200", "-Wl,-rpath,$ORIGIN"])
    # the host layer's own timing program (bench.py runs it for its `host_layer` key)
    subprocess.check_call(["g++", "-std=c++17", "-O2", "-Wall", "-o", HOST_BENCH, os.path.join(HOST_DIR, "bench_host_layer.cpp"),
                           "-I", os.path.join(HOST_DIR, "include"), "-L", PKG, "-lctensor_host", "-lctb200",
                           "-Wl,-rpath,$ORIGIN/.."])
    return HOST_LIB


def reference_root() -> str:
    """Where the reference's sources are, for the steps that compile them as checkers: the
    CTENSOR_REFERENCE environment variable, else a checkout named `reference` beside this
    repository.  Empty when there is none (those steps are then skipped)."""
    cand = os.environ.get("CTENSOR_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(PKG)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src", "core")) else ""


GEN1_DIR = os.path.join(HOST_DIR, "gen1")
GEN1_LIB = os.path.join(PKG, "libctensor_gen1.so")


def build_gen1(force: bool = False) -> str:
    """The first-generation host layer (tensor1.h / opsmp.h / ops1.h of the reference's root tree
    over the C ABI): plain g++ like build_host."""
    src = os.path.join(GEN1_DIR, "ctensor_gen1.cpp")
    deps = [src, os.path.join(os.path.dirname(PKG), "include", "ctb200.h")]
    deps += [os.path.join(GEN1_DIR, "include", f) for f in os.listdir(os.path.join(GEN1_DIR, "include"))]
    # the optimizer vocabulary and classes are shared with the second-generation layer
    shared = os.path.join(HOST_DIR, "include")
    deps += [os.path.join(shared, f) for f in ("ctb_optimizer.h", "optimizer_classes.h")]
    if not force and os.path.exists(GEN1_LIB) and os.path.getmtime(GEN1_LIB) >= max(map(os.path.getmtime, deps)) \
            and os.path.getmtime(GEN1_LIB) >= os.path.getmtime(LIB):
        return GEN1_LIB
    subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra", "-o", GEN1_LIB, src,
                           "-I", GEN1_DIR, "-I", shared, "-L", PKG, "-lctb200", "-Wl,-rpath,$ORIGIN"])
    return GEN1_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
    print(build_host(force="--force" in sys.argv))
    print(build_gen1(force="--force" in sys.argv))
