"""Builds the native library in-tree: ``python -m flextensor_b200.build``.

nvcc cross-compiles for sm_100a without a GPU; the result is
``flextensor_b200/lib/libftb200.so`` (git-ignored, loaded by ``backend.lib()``).
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libftb200.so")
SOURCES = ["ftb_core.cu", "ftb_gemm.cu", "ftb_dwconv.cu", "ftb_noalloc.cu", "ftb_simt_gemm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def needs_build():
    if not os.path.exists(LIB):
        return True
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "ftb200.h"))
    return _newest(deps) > os.path.getmtime(LIB)


PROFILE_LIB = os.path.join(LIB_DIR, "libftb200_prof.so")


def build_profile_waits():
    """The same sources with -DFTB_PROFILE_WAITS (per-role wait counters in the GEMM kernel), as a
    second library beside the product one; load it with FTB200_LIBRARY=<path>."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [nvcc] + NVCC_FLAGS + ["-DFTB_PROFILE_WAITS", "-o", PROFILE_LIB] + sources()
    proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n%s\n%s" % (proc.stdout, proc.stderr))
    return PROFILE_LIB


def build(force=False, verbose=False):
    """Compile the library if it is missing or older than its sources; returns its path."""
    if not force and not needs_build():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the sm_100a kernels cannot be built")
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + sources()
    proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n%s\n%s" % (proc.stdout, proc.stderr))
    if verbose:
        print(proc.stderr)
    return LIB


if __name__ == "__main__":
    if "--profile-waits" in sys.argv:
        print(build_profile_waits())
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
