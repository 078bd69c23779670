"""Build recipe for libapus_cuda.so (sm_100a only)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libapus_cuda.so")
SRC = os.path.join(HERE, "csrc", "backend_cuda.cu")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
    "-std=c++17", "-Xcompiler", "-fPIC,-fopenmp", "-shared",
]


def sources():
    d = os.path.join(HERE, "csrc")
    out = [os.path.join(d, f) for f in sorted(os.listdir(d))]
    out.append(os.path.join(HERE, "..", "include", "backend_cuda.h"))
    return out


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(s) > t for s in sources())


def build(force=False, verbose=False):
    """Compile the CUDA library in-tree.  nvcc cross-compiles for sm_100a
    without a GPU present."""
    if not force and not stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
        ["-o", LIB, SRC, "-lgomp"]
    subprocess.run(cmd, check=True)
    return LIB
