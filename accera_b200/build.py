"""Builds libaccera_b200.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

    python -m accera_b200.build [--force] [--verbose]

No GPU is needed: nvcc cross-compiles for sm_100a.  Objects go to
accera_b200/csrc/build/, the library to accera_b200/libaccera_b200.so.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

_PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_PKG, "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(_PKG, "libaccera_b200.so")
INCLUDE_DIR = os.path.join(os.path.dirname(_PKG), "include")

SOURCES = ["abi.cu", "gemm_simt.cu", "gemm_umma.cu", "gemm_splitk.cu", "repack.cu", "reduce_mean.cu", "gather.cu", "range.cu"]
HEADERS = ["accb_internal.h", os.path.join(INCLUDE_DIR, "accera_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")


def _newest(paths) -> float:
    return max(os.path.getmtime(p if os.path.isabs(p) else os.path.join(CSRC, p)) for p in paths)


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    return os.path.getmtime(LIB_PATH) < _newest(SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a and link the shared library. Returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = find_nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr_time = _newest(HEADERS)

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        src_path = os.path.join(CSRC, src)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src_path), hdr_time):
            return obj
        cmd = [nvcc, *NVCC_FLAGS, "-c", src_path, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = os.path.join(OBJ_DIR, src.replace(".cu", ".ptxas.log"))
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    # cudart is linked statically (nvcc default) and the driver API is resolved at run time, so the
    # library loads on a machine without a GPU driver (symbol checks, packaging) and fails only when used.
    cmd = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
