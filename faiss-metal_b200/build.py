"""In-tree build of libb200flat.so (CUDA kernels + C-ABI + C++ host layer) for sm_100a.

nvcc cross-compiles without a GPU, so this runs on any machine with CUDA 12.9+.
Objects go to build/, the library to lib/ beside this file.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
BUILD_DIR = os.path.join(HERE, "build")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libb200flat.so")

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
HOST_CXX = shutil.which("g++") or "g++"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
CU_SOURCES = ["csrc/rows.cu", "csrc/scan.cu", "csrc/select.cu", "csrc/select_rank.cu", "csrc/gemm_topk.cu", "csrc/search.cu"]
CPP_SOURCES = ["host/Resources.cpp", "host/GrowableArray.cpp", "host/IndexFlat.cpp", "host/Sharded.cpp", "host/capi.cpp",
               "faiss_compat/compat_impl.cpp"]
def _headers():
    """Every header an object may depend on (globbed, so that a new one cannot be forgotten)."""
    import glob
    pats = ["csrc/*.cuh", "csrc/*.h", "host/*.h", "include/faiss-b200/*.h", "faiss_compat/faiss/*.h",
            "faiss_compat/faiss/impl/*.h", "../include/*.h"]
    out = []
    for pat in pats:
        out += sorted(glob.glob(os.path.join(HERE, pat)))
    return out


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), r.stdout))
    return r.stdout


def include_dirs():
    # real FAISS headers win when FAISS_INCLUDE_DIR points at them
    faiss_inc = os.environ.get("FAISS_INCLUDE_DIR")
    dirs = [faiss_inc] if faiss_inc else [os.path.join(HERE, "faiss_compat")]
    dirs += [os.path.join(HERE, "include"), os.path.join(REPO, "include"), os.path.join(CUDA_HOME, "include")]
    return dirs


def build_library(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(BUILD_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    hdrs = _headers() + [os.path.abspath(__file__)]
    incs = []
    for d in include_dirs():
        incs += ["-I", d]
    jobs = []
    objs = []
    for src in CU_SOURCES:
        s = os.path.join(HERE, src)
        o = os.path.join(BUILD_DIR, os.path.basename(src) + ".o")
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            jobs.append([NVCC, "-ccbin", HOST_CXX, *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17",
                         "-Xcompiler", "-fPIC", "-Xptxas", "-v", *incs, "-c", s, "-o", o])
    for src in CPP_SOURCES:
        s = os.path.join(HERE, src)
        o = os.path.join(BUILD_DIR, os.path.basename(src) + ".o")
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            jobs.append([HOST_CXX, "-O2", "-std=c++17", "-fPIC", "-Wall", *incs, "-c", s, "-o", o])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            outs = list(ex.map(_run, jobs))
        if verbose:
            for o in outs:
                sys.stdout.write(o)
    if force or jobs or _newer(LIB_PATH, objs):
        _run([NVCC, "-ccbin", HOST_CXX, *ARCH_FLAGS, "-shared", "-o", LIB_PATH, *objs,
              "-cudart", "static", "-Xlinker", "--no-undefined", "-ldl"])
    return LIB_PATH


def build_contract_test() -> str:
    """C++ test binary of the plugin classes (tests/cpp/contract_test.cpp), linked against
    the in-tree library with a relative rpath so it runs wherever the tree is copied."""
    src = os.path.join(REPO, "tests", "cpp", "contract_test.cpp")
    out_dir = os.path.join(REPO, "tests", "_build")
    out = os.path.join(out_dir, "contract_test")
    os.makedirs(out_dir, exist_ok=True)
    if _newer(out, [src, LIB_PATH]):
        incs = []
        for d in include_dirs():
            incs += ["-I", d]
        _run([HOST_CXX, "-O1", "-std=c++17", "-Wall", *incs, src, "-o", out, "-L", LIB_DIR, "-lb200flat",
              "-Wl,-rpath,$ORIGIN/../../faiss-metal_b200/lib"])
    return out


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_contract_test())
