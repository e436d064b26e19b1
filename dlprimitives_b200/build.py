"""Builds the CUDA library (sm_100a) and the C++ host library in-tree.

    python -m dlprimitives_b200.build          # build what is out of date
    python -m dlprimitives_b200.build --force

nvcc cross-compiles for sm_100a without a GPU.  The outputs sit next to the sources so that they
travel with the tree:  dlprimitives_b200/lib/libdlprim_b200_cuda.so  (kernels + C ABI) and
dlprimitives_b200/lib/libdlprim_b200.so  (the C++ host API above it).
"""
import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")
LIB = os.path.join(HERE, "lib")
OBJ = os.path.join(HERE, "build")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
# the system compiler: other g++ installs in the image link libstdc++ statically, which breaks
# passing C++ objects (and exceptions) between shared libraries
CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")

NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "-ccbin", CXX, "-Xptxas", "-v", "--expt-relaxed-constexpr"]
if os.environ.get("DLP_TC_DIAGNOSTICS"):   # compile the tensor-core kernel's timeline and timing switches in
    NVCC_FLAGS.append("-DDLP_TC_DIAGNOSTICS")
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-fvisibility=hidden", "-I" + os.path.join(ROOT, "include"),
             "-I" + os.path.join(CUDA_HOME, "include")]

CUDA_LIB = os.path.join(LIB, "libdlprim_b200_cuda.so")
HOST_LIB = os.path.join(LIB, "libdlprim_b200.so")


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _headers(*dirs):
    out = []
    for d in dirs:
        for base, _, files in os.walk(d):
            out += [os.path.join(base, f) for f in files if f.endswith((".h", ".hpp", ".cuh"))]
    return out


def _run(cmd, log=None):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.append(r.stdout)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout)
        raise RuntimeError("build step failed: " + cmd[0] + " " + cmd[-1])
    return r.stdout


def build_cuda(force=False, verbose=False):
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdrs = _headers(CSRC, os.path.join(ROOT, "include"))
    objs, jobs, logs = [], [], []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            jobs.append([NVCC] + NVCC_FLAGS + ["-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(lambda c: _run(c, logs), jobs))
    if verbose:
        sys.stdout.write("".join(logs))
    if jobs or force or _newer(CUDA_LIB, objs):
        _run([NVCC, "-shared", "-ccbin", CXX, "-o", CUDA_LIB] + objs + ["-cudart", "shared"])
    return CUDA_LIB


def build_host(force=False):
    if not os.path.isdir(HOST):
        return None
    srcs = sorted(os.path.join(HOST, f) for f in os.listdir(HOST) if f.endswith(".cpp"))
    if not srcs:
        return None
    hdrs = _headers(HOST, os.path.join(ROOT, "include"))
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(OBJ, "host_" + os.path.basename(s)[:-4] + ".o")
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            jobs.append([CXX] + CXX_FLAGS + ["-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(_run, jobs))
    if jobs or force or _newer(HOST_LIB, objs + [CUDA_LIB]):
        _run([CXX, "-shared", "-o", HOST_LIB] + objs + ["-L" + LIB, "-ldlprim_b200_cuda", "-L" + os.path.join(CUDA_HOME, "lib64"),
                                                        "-lcudart", "-Wl,-rpath,$ORIGIN"])
    return HOST_LIB


def build_all(force=False, verbose=False):
    build_cuda(force, verbose)
    build_host(force)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print the ptxas resource usage lines")
    a = ap.parse_args()
    build_all(a.force, a.verbose)
    print("built", CUDA_LIB)
