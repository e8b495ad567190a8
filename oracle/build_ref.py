"""TEST INFRASTRUCTURE - builds the reference's own CPU device into oracle/_ref/libaixref.so.

The reference sources are compiled where they lie (the checkout named by AIX_REFERENCE_ROOT); nothing is copied
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


ADAPTER_OUT = os.path.join(OUT_DIR, "adapter_check")


def build_adapter_check(force: bool = False) -> str | None:
    """Builds the drop-in check: the reference's unmodified front end + aix_b200/adapter/aixDeviceB200.hpp, linked
    against libaixb200.so. Needs the reference headers, hence lives with the oracle artefacts."""
    if not reference_available():
        return ADAPTER_OUT if os.path.isfile(ADAPTER_OUT) else None
    root = os.path.join(HERE, "..")
    adapter_dir = os.path.join(root, "aix_b200", "adapter")
    lib_dir = os.path.join(root, "aix_b200", "lib")
    src = os.path.join(adapter_dir, "adapter_check.cpp")
    deps = [src, os.path.join(adapter_dir, "aixDeviceB200.hpp"), os.path.join(root, "include", "aixb200.h")]
    if not os.path.isfile(os.path.join(lib_dir, "libaixb200.so")):
        return None
    if not force and os.path.isfile(ADAPTER_OUT) and all(os.path.getmtime(ADAPTER_OUT) >= os.path.getmtime(d) for d in deps):
        return ADAPTER_OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-std=c++20", "-O2", "-w", "-I", LIB_DIR, "-I", os.path.join(root, "include"), "-I", adapter_dir, src]
    cmd += [os.path.join(LIB_DIR, s) for s in REF_SOURCES]
    cmd += ["-L", lib_dir, "-laixb200", "-Wl,-rpath,$ORIGIN/../../aix_b200/lib", "-o", ADAPTER_OUT]
    subprocess.run(cmd, check=True)
    return ADAPTER_OUT


if __name__ == "__main__":
    path = build(force="--force" in sys.argv)
    print(path if path else "reference sources not found; nothing built")
    print(build_adapter_check(force="--force" in sys.argv))
