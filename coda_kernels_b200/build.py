"""Builds ``libcoda_b200.so`` in-tree with nvcc for sm_100a, and the PyTorch dispatch shim next to it.

Run as ``python -m coda_kernels_b200.build``; ``build_library()`` is also what
``__graft_entry__.build()`` calls.  Each ``csrc/*.cu`` is compiled to an object
file (in parallel) and the objects are linked into one shared library that sits
next to this file, so that the binary travels with the source tree.
``csrc_torch/torch_binding.cpp`` (TORCH_LIBRARY registrations that call the C
ABI) is compiled with g++ against the installed torch into
``libcoda_b200_torch.so``, which links ``libcoda_b200.so`` by ``$ORIGIN``.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libcoda_b200.so"
TORCH_SRC = PKG_DIR / "csrc_torch" / "torch_binding.cpp"
TORCH_LIB_PATH = PKG_DIR / "libcoda_b200_torch.so"
HASH_PATH = PKG_DIR / "libcoda_b200.srchash"
OBJ_DIR = PKG_DIR / "build"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build libcoda_b200.so")
    return nvcc


def have_nvcc() -> bool:
    return bool(shutil.which("nvcc")) or os.path.exists("/usr/local/cuda/bin/nvcc")


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def source_hash() -> str:
    """Digest of every file the library is built from (content, not mtime: copies of the tree keep it)."""
    h = hashlib.sha256()
    files = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "coda_b200.h", TORCH_SRC]
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_stale() -> bool:
    if not LIB_PATH.exists() or not TORCH_LIB_PATH.exists() or not HASH_PATH.exists():
        return True
    return HASH_PATH.read_text().strip() != source_hash()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel for sm_100a and link the shared library."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    # Several ranks may import the package at once: one builds, the others wait and then find a fresh library.
    lock = open(OBJ_DIR / ".lock", "w")
    fcntl.flock(lock, fcntl.LOCK_EX)
    try:
        if not force and not is_stale():
            return LIB_PATH
        return _build_locked(nvcc, force, verbose)
    finally:
        fcntl.flock(lock, fcntl.LOCK_UN)
        lock.close()


def _build_locked(nvcc: str, force: bool, verbose: bool) -> Path:
    header_mtime = max(f.stat().st_mtime for f in list(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "coda_b200.h"])

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        if not force and obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, header_mtime):
            return obj
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose:
            sys.stderr.write(res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, _sources()))
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-cudart", "static"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    _build_torch_shim()
    HASH_PATH.write_text(source_hash() + "\n")
    return LIB_PATH


def _build_torch_shim() -> None:
    """g++ only: the shim holds no device code.  It is linked against the torch of this interpreter."""
    import torch
    from torch.utils import cpp_extension

    cxx = shutil.which("g++") or "g++"
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           str(TORCH_SRC), "-o", str(TORCH_LIB_PATH)]
    cmd += [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{cuda_home}/include"]
    cmd += [f"-L{p}" for p in cpp_extension.library_paths()] + ["-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda", "-ltorch_cuda"]
    cmd += [f"-L{PKG_DIR}", f"-l:{LIB_PATH.name}", "-Wl,-rpath,$ORIGIN"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building {TORCH_LIB_PATH.name} failed:\n{res.stdout}\n{res.stderr}")


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
