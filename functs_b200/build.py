"""Builds the C-ABI shared library (and, on request, the TorchScript operator extension) in-tree.

The kernels target sm_100a only.  The library is plain CUDA C++ without any torch dependency.
"""
import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libfuncts_b200.so")

SOURCES = [
    "capi.cu",
    "kernels_basic.cu",
    "kernels_select_nms.cu",
    "kernels_yolo.cu",
    "kernels_ssd.cu",
    "kernels_yolact.cu",
    "kernels_lstm.cu",
    "kernels_lstm_tc.cu",
    "no_alloc.cu",
    "kernels_generic.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",  # products and sums round separately unless the code asks for fmaf()
    "-Xcompiler", "-fPIC", "-shared",
]


def _sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _deps():
    out = _sources()
    for name in os.listdir(CSRC):
        if name.endswith((".cuh", ".h")):
            out.append(os.path.join(CSRC, name))
    out.append(os.path.join(PKG_DIR, "..", "include", "functs_b200.h"))
    return out


def library_is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > built for p in _deps())


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compiles csrc/*.cu into libfuncts_b200.so next to this file.  Returns the library path."""
    if not force and not library_is_stale():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH] + _sources()
    res = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
