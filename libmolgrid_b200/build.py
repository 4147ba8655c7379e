"""Builds liblmg_b200.so (the CUDA kernels and their C ABI) in-tree with nvcc for sm_100a.

Run as ``python -m libmolgrid_b200.build`` or call :func:`build_library`.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "liblmg_b200.so")
SOURCES = ["lmg_gridmaker.cu", "lmg_misc.cu", "lmg_cabi.cu", "lmg_noalloc.cu", "lmg_records.cu"]
HEADERS = ["lmg_device.cuh", "lmg_launch.h", "lmg_misc.h", os.path.join("..", "..", "include", "lmg_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    # no fused multiply-add in host code either: the host computes GridMaker's constants
    "-Xcompiler", "-fPIC,-ffp-contract=off,-fvisibility=default",
    "--shared",
]


def _nvcc():
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def up_to_date():
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return all(os.path.getmtime(d) <= t for d in deps)


def build_library(force=False, verbose=False):
    """Compile the library if sources are newer than the built file. Returns its path."""
    if not force and up_to_date():
        return LIB
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
        [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return LIB


NATIVE_SRCS = [os.path.join(HERE, "cpp", "bindings.cpp"), os.path.join(HERE, "cpp", "bindings_objects.cpp")]


def native_module_path():
    import sysconfig
    return os.path.join(HERE, "molgrid_native" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_native_module(force=False):
    """Compile the pybind11 module over the C++ host layer (g++; links liblmg_b200.so by $ORIGIN)."""
    import pybind11
    import sysconfig
    out = native_module_path()
    deps = NATIVE_SRCS + [os.path.join(HERE, "cpp", "bindings_common.h"), LIB] + [os.path.join(HERE, "cpp", "include", "libmolgrid", f)
                                for f in os.listdir(os.path.join(HERE, "cpp", "include", "libmolgrid"))]
    if not force and os.path.exists(out) and all(os.path.getmtime(d) <= os.path.getmtime(out) for d in deps):
        return out
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"],
           "-I" + os.path.join(HERE, "cpp", "include"), "-I" + os.path.join(HERE, "..", "include"),
           "-I" + os.path.join(cuda, "include")] + NATIVE_SRCS + ["-o", out,
           "-L" + HERE, "-llmg_b200", "-L" + os.path.join(cuda, "lib64"), "-lcudart",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    return out


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_native_module(force="--force" in sys.argv))
