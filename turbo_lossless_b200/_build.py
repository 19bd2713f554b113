"""Builds libsplit12_b200.so (sm_100a only) in-tree with nvcc."""
from __future__ import annotations

import os
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_PKG, "csrc")
LIB_PATH = os.path.join(_PKG, "libsplit12_b200.so")
SOURCES = ["runtime.cu", "decompress.cu", "patches.cu", "gemv.cu", "gemv_stream.cu", "gemm.cu", "gemm_tc.cu", "gemm_stream.cu", "pack.cu", "comm.cu", "step.cu", "loader.cu", "moe.cu", "host.cpp"]
# sources compiled without --use_fast_math: the decode-step kernels use sincosf / expf / division on values
# where the fast intrinsics lose digits (RoPE angles of hundreds of radians)
ACCURATE_MATH = {"step.cu", "moe.cu"}
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default", "--use_fast_math"]


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [
        os.path.join(_PKG, "..", "include", "split12_b200.h"), os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a and link the shared library."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    objdir = os.path.join(_PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    objs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        flags = [f for f in NVCC_FLAGS if not (src in ACCURATE_MATH and f == "--use_fast_math")]
        cmd = [nvcc, *flags, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src} ---\n{out}\n")
        elif verbose:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("nvcc failed; see messages above")
    subprocess.run([nvcc, "-Wno-deprecated-gpu-targets", "-shared", "-o", LIB_PATH, *objs, "-lcudart"], check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
