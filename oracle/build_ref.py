"""TEST INFRASTRUCTURE - builds the reference's own CPU device into oracle/_ref/libaixref.so.

The reference sources are compiled where they lie (AIX_REFERENCE_ROOT, default /root/reference); nothing is copied
into this repository and the output directory is git-ignored. Flags follow the reference's Release configuration
(CMakeLists.txt:41,49: C++20, -O3, asserts left on). Only oracle/ref_shim.cpp (a thin C ABI, no arithmetic) is ours.

Usage: python oracle/build_ref.py [--force]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libaixref.so")
REF_ROOT = os.environ.get("AIX_REFERENCE_ROOT", "/root/reference")
LIB_DIR = os.path.join(REF_ROOT, "Targets", "AIXLib")
REF_SOURCES = ["aixDeviceCPU.cpp", "aixDevices.cpp", "aixFuse.cpp"]


def reference_available() -> bool:
    return all(os.path.isfile(os.path.join(LIB_DIR, s)) for s in REF_SOURCES)


def build(force: bool = False) -> str | None:
    """Returns the path of the built library, or None when the reference sources are not present."""
    if not reference_available():
        return OUT if os.path.isfile(OUT) else None
    shim = os.path.join(HERE, "ref_shim.cpp")
    deps = [shim, os.path.join(HERE, "..", "include", "aixb200.h")] + [os.path.join(LIB_DIR, s) for s in REF_SOURCES]
    if not force and os.path.isfile(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-std=c++20", "-O3", "-fPIC", "-shared", "-w", "-I", LIB_DIR, shim]
    cmd += [os.path.join(LIB_DIR, s) for s in REF_SOURCES] + ["-o", OUT]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    path = build(force="--force" in sys.argv)
    print(path if path else "reference sources not found; nothing built")
