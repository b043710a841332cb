"""Builds fitre_b200/libfitre_b200.so in-tree with nvcc for sm_100a.

    python -m fitre_b200.build [--verbose]

The library is plain CUDA C++ behind a C ABI (include/fitre_b200.h); it links only the CUDA
runtime (NCCL is loaded at run time when a communicator is requested).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SOURCES = ["gemm.cu", "conv_tma.cu", "conv_tf32.cu", "conv_i8.cu", "layers.cu", "peer.cu", "passes.cu", "kfac.cu", "training.cu", "model.cpp", "comm.cpp", "cabi.cpp"]
LIB = os.path.join(HERE, "libfitre_b200.so")
# C++ functions with the reference's own (mangled) names on top of the C ABI
SHIM_SRC = os.path.join(HERE, "csrc", "reference_shim.cpp")
SHIM_LIB = os.path.join(HERE, "libfitre_reference_shim.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def _stale(obj, src):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    deps = [src, os.path.join(CSRC, "common.h"), os.path.join(CSRC, "tma_util.cuh"), os.path.join(CSRC, "graphs.h"),
            os.path.join(os.path.dirname(HERE), "include", "fitre_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False):
    flags = [f for f in FLAGS if f != "--use_fast_math=false"]
    objs = []
    procs = []
    for s in SOURCES:
        src = os.path.join(CSRC, s)
        obj = os.path.join(CSRC, os.path.splitext(s)[0] + ".o")
        objs.append(obj)
        if force or _stale(obj, src):
            cmd = [NVCC] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", src, "-o", obj]
            procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write("== %s ==\n%s\n" % (s, out))
        failed = failed or p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if procs or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-lcudart", "-ldl"]
        subprocess.check_call(cmd)
    if force or _stale(SHIM_LIB, SHIM_SRC) or os.path.getmtime(SHIM_LIB) < os.path.getmtime(LIB):
        inc = os.path.join(os.path.dirname(HERE), "include")
        cmd = [NVCC, "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-I", inc, "-shared", "-o", SHIM_LIB,
               SHIM_SRC, "-L", HERE, "-lfitre_b200", "-lcudart", "-Xlinker", "-rpath=$ORIGIN"]
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
