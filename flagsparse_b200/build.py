"""Build libfsb.so (the sm_100a CUDA library) in-tree with nvcc.

Usage: python -m flagsparse_b200.build [--force] [--verbose] [--check]
The shared library lands next to the sources (flagsparse_b200/csrc/libfsb.so), where the ctypes loader
looks for it.  nvcc cross-compiles for sm_100a, so no GPU is needed to build.  --check builds the checking
variant instead (the same sources with -DFSB_BOUNDS_CHECK, into libfsb_check.so; the loader takes it when the
environment has FSB_BOUNDS_CHECK=1): its entry points walk the index arrays they are given before any product
kernel runs and refuse a call that would leave its arrays.
"""

import os
import subprocess
import sys

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
INCLUDE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
LIB = os.path.join(CSRC, "libfsb.so")
CHECK_LIB = os.path.join(CSRC, "libfsb_check.so")
SOURCES = ("csr_analyze.cu", "spmv_csr.cu", "spmv_panel.cu", "spmv_wide.cu", "spmm_csr.cu", "sddmm_csr.cu",
           "bounds_check.cu", "panel_build.cu")
NVCC_FLAGS = (
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-DFSB_BUILD",
)


def _newest_source_mtime():
    paths = [os.path.join(CSRC, s) for s in SOURCES]
    paths += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    paths.append(os.path.join(INCLUDE, "fsb.h"))
    return max(os.path.getmtime(p) for p in paths)


def build(force=False, verbose=False, check=False):
    """Compile every .cu file into object files and link them into libfsb.so (libfsb_check.so for the checking
    variant).  Returns the library path."""
    lib = CHECK_LIB if check else LIB
    if not force and os.path.exists(lib) and os.path.getmtime(lib) >= _newest_source_mtime():
        return lib
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".check.o" if check else ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        if check:
            cmd.insert(1, "-DFSB_BOUNDS_CHECK")
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib, *objs, "-lcudart"]
    subprocess.run(link, check=True)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, check="--check" in sys.argv))
