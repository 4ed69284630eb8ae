"""Ahead-of-time build of the CUDA library: nvcc for sm_100a only, in-tree (libprism_b200.so beside this file).

    python -m prism_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "prism_b200.cu")
LIB = os.path.join(HERE, "libprism_b200.so")
FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC",
         "-shared"]


def sources():
    d = os.path.join(HERE, "csrc")
    inc = os.path.join(HERE, "..", "include")
    return [os.path.join(d, f) for f in sorted(os.listdir(d))] + [os.path.join(inc, f) for f in sorted(os.listdir(inc))]


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(s) > t for s in sources())


def build(force=False, verbose=False):
    """Compile csrc/prism_b200.cu (which includes every kernel header) into libprism_b200.so; returns its path."""
    if not force and not stale():
        return LIB
    nvcc = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB + ".tmp", SRC]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    os.replace(LIB + ".tmp", LIB)
    if verbose:
        print(r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
