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
# the reference checkout: AIX_REFERENCE_ROOT, else a directory named "reference" beside this repository
REF_ROOT = os.environ.get("AIX_REFERENCE_ROOT") or os.path.abspath(os.path.join(HERE, "..", "..", "reference"))
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
ADAPTER_BENCH_OUT = os.path.join(OUT_DIR, "adapter_bench")


def _build_front_end_program(source_name: str, out: str, force: bool) -> str | None:
    """Compiles tests/cpp/<source_name>: the reference's unmodified front end + aix_b200/adapter/aixDeviceB200.hpp, linked
    against libaixb200.so. Needs the reference headers, hence the binary lives with the oracle artefacts."""
    if not reference_available():
        return out if os.path.isfile(out) else None
    root = os.path.join(HERE, "..")
    adapter_dir = os.path.join(root, "aix_b200", "adapter")
    lib_dir = os.path.join(root, "aix_b200", "lib")
    src = os.path.join(root, "tests", "cpp", source_name)
    deps = [src, os.path.join(adapter_dir, "aixDeviceB200.hpp"), os.path.join(root, "include", "aixb200.h")]
    if not os.path.isfile(os.path.join(lib_dir, "libaixb200.so")):
        return None
    if not force and os.path.isfile(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps):
        return out
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-std=c++20", "-O2", "-w", "-I", LIB_DIR, "-I", os.path.join(root, "include"), "-I", adapter_dir, src]
    cmd += [os.path.join(LIB_DIR, s) for s in REF_SOURCES]
    cmd += ["-L", lib_dir, "-laixb200", "-Wl,-rpath,$ORIGIN/../../aix_b200/lib", "-o", out]
    subprocess.run(cmd, check=True)
    return out


def build_adapter_check(force: bool = False) -> str | None:
    """The drop-in correctness check (tests/test_gpu_adapter.py runs it)."""
    return _build_front_end_program("adapter_check.cpp", ADAPTER_OUT, force)


def build_adapter_bench(force: bool = False) -> str | None:
    """The drop-in timing program (bench.py runs it and reports its line as extras.cpp_front_end)."""
    return _build_front_end_program("adapter_bench.cpp", ADAPTER_BENCH_OUT, force)


if __name__ == "__main__":
    path = build(force="--force" in sys.argv)
    print(path if path else "reference sources not found; nothing built")
    print(build_adapter_check(force="--force" in sys.argv))
    print(build_adapter_bench(force="--force" in sys.argv))
