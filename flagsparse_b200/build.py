"""Build libfsb.so (the sm_100a CUDA library) in-tree with nvcc.

Usage: python -m flagsparse_b200.build [--force] [--verbose]
The shared library lands next to the sources (flagsparse_b200/csrc/libfsb.so), where the ctypes loader
looks for it.  nvcc cross-compiles for sm_100a, so no GPU is needed to build.
"""

import os
import subprocess
import sys

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
INCLUDE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
LIB = os.path.join(CSRC, "libfsb.so")
SOURCES = ("csr_analyze.cu", "spmv_csr.cu", "spmv_panel.cu", "spmv_wide.cu", "spmm_csr.cu", "sddmm_csr.cu")
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


def build(force=False, verbose=False):
    """Compile every .cu file into object files and link them into libfsb.so.  Returns the library path."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source_mtime():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
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
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs, "-lcudart"]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
