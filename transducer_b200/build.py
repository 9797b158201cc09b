"""In-tree build of the native code: ``python -m transducer_b200.build``.

Produces, next to this file,
  libtransducer_b200.so                 kernels + C ABI (nvcc, sm_100a only)
  _transducer.<python-abi>.so           pybind11 module bound to that library

nvcc cross-compiles without a GPU; the built files are what a GPU machine loads.
"""
import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtransducer_b200.so")
EXT = os.path.join(HERE, "_transducer" + sysconfig.get_config_var("EXT_SUFFIX"))

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "--threads", "0", "-ccbin", "g++",
]


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_library(force=False, verbose=False, extra_flags=()):
    cu = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = cu + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) \
        + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    if not force and _newer(LIB, deps):
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-shared", "-o", LIB, *cu]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return LIB


def build_extension(force=False, verbose=False):
    import pybind11
    src = os.path.join(CSRC, "_transducer.cpp")
    deps = [src, LIB] + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    if not force and _newer(EXT, deps):
        return EXT
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           src, "-L", HERE, "-ltransducer_b200", "-Wl,-rpath,$ORIGIN", "-o", EXT]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return EXT


def build_all(force=False, verbose=False):
    build_library(force, verbose)
    build_extension(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
