"""Builds libaixb200.so (the C-ABI device library) in-tree with nvcc for sm_100a.

The library links cudart statically, NVRTC dynamically, and opens libcuda / libnccl lazily, so it loads on machines
that have no GPU driver (where only dry-run devices can be created).

Usage: python -m aix_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "lib")
OUT = os.path.join(OUT_DIR, "libaixb200.so")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
SOURCES = ["capi.cpp", "device.cpp", "planner.cpp", "codegen.cpp", "comm.cpp", "reduce.cu", "misc.cu", "gemm_sm100.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "--expt-relaxed-constexpr"]


def _headers():
    hs = [os.path.join(SRC, f) for f in os.listdir(SRC) if f.endswith((".hpp", ".cuh", ".h"))]
    hs.append(os.path.join(HERE, "..", "include", "aixb200.h"))
    return hs


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    newest_header = max(os.path.getmtime(h) for h in _headers())
    objects, procs = [], []
    for s in SOURCES:
        src = os.path.join(SRC, s)
        obj = os.path.join(OBJ_DIR, s + ".o")
        objects.append(obj)
        if not force and os.path.isfile(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), newest_header):
            continue
        cmd = [NVCC] + ARCH + COMMON + ["-c", src, "-o", obj]
        if s.endswith(".cu"):
            cmd += ["-Xptxas", "-v"] if verbose else []
        else:
            cmd = [NVCC] + COMMON + ["-x", "cu" if False else "c++", "-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd))
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            print(f"--- {s} ---\n{out}")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("compilation failed")
    if procs or force or not os.path.isfile(OUT):
        # linked beside the target and renamed into place: a reader never sees a half-written library
        cmd = [NVCC, "-shared", "-o", OUT + ".tmp"] + objects + ["-cudart", "static", "-lnvrtc", "-ldl", "-lpthread"]
        subprocess.run(cmd, check=True)
        os.replace(OUT + ".tmp", OUT)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
