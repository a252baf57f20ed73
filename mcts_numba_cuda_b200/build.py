"""Builds ``libmctsnc_b200.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB_PATH = os.path.join(HERE, "libmctsnc_b200.so")
SOURCES = [os.path.join(HERE, "csrc", n) for n in ("mctsnc_abi.cu", "peer_exchange.cu", "puct_select.cu", "puct_select_v2.cu", "duct_select.cu")]
HEADERS = [os.path.join(HERE, "csrc", n) for n in ("c4_search.cuh", "gomoku_search.cuh", "common.cuh", "rng.cuh")] + [
    os.path.join(ROOT, "include", "mctsnc_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
              "-Xcompiler", "-fPIC"]


def nvcc_path():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found: libmctsnc_b200.so cannot be built")
    return path


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.exists(p) and os.path.getmtime(p) > built for p in SOURCES + HEADERS)


def build(force=False, verbose=False):
    """Compiles the library if it is missing or older than its sources; returns its path."""
    if force or is_stale():
        cmd = [nvcc_path()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH] + SOURCES
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose:
            print(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose=True))
