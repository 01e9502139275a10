"""Builds libtile_sm100.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

Run as a script (``python tile-rs_b200/build.py``) or through ``build_library()``.
The shared object lands next to this file so that it travels with the source
tree; cudart is linked statically, so the library loads (and reports
TSM100_ERR_NO_DEVICE) on a machine without a GPU or driver.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
BUILD_DIR = PKG_DIR / "_build"
LIB_PATH = PKG_DIR / "libtile_sm100.so"

CUDA_SOURCES = ["runtime.cu", "capi_ops.cu", "multi.cu"]
CXX_SOURCES = ["inputs.cpp", "emit.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fopenmp,-Wall",
    "-Xptxas", "-v",
    f"-I{INCLUDE}",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libtile_sm100 cannot be built")
    return exe


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*")) + [INCLUDE / "tile_sm100.h", Path(__file__)]):
        if p.is_file():
            h.update(p.name.encode())
            h.update(p.read_bytes())
    return h.hexdigest()


def _compile(src: str) -> Path:
    obj = BUILD_DIR / (src + ".o")
    log = BUILD_DIR / (src + ".log")
    cmd = [nvcc(), *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
    if src.endswith(".cpp"):
        cmd = [nvcc(), *[f for f in NVCC_FLAGS if f not in ("-Xptxas", "-v")], "-x", "cu", "-c", str(CSRC / src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the library unless an up-to-date one exists. Returns its path."""
    BUILD_DIR.mkdir(exist_ok=True)
    stamp = BUILD_DIR / "digest.txt"
    digest = _digest()
    if not force and LIB_PATH.exists() and stamp.exists() and stamp.read_text() == digest:
        return LIB_PATH
    with ThreadPoolExecutor(max_workers=4) as pool:
        objs = list(pool.map(_compile, CUDA_SOURCES + CXX_SOURCES))
    cmd = [nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs), "-cudart", "static", "-Xcompiler", "-fopenmp", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(digest)
    if verbose:
        for src in CUDA_SOURCES:
            print((BUILD_DIR / (src + ".log")).read_text())
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)


def build_module(source: str, out_path: Path) -> Path:
    """Compiles a translation unit produced by the ``cuda_sm100`` target into a shared
    library that ``KernelLauncher.load`` / ``tsm100_module_load`` accepts.  This is the
    step the reference leaves to the host build crate (crates/tile_codegen/src/target.rs:4-10)."""
    out_path = Path(out_path)
    out_path.parent.mkdir(parents=True, exist_ok=True)
    cu = out_path.with_suffix(".cu")
    cu.write_text(source)
    cmd = [nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
           "--expt-relaxed-constexpr", "-shared", "-Xcompiler", "-fPIC", f"-I{CSRC}", f"-I{INCLUDE}",
           "-cudart", "static", "-o", str(out_path), str(cu)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on emitted module:\n{r.stdout}\n{r.stderr}")
    return out_path
