"""Build and load ``libtspipe_b200.so`` (the sm_100a kernels under ``csrc/``).

The library is plain CUDA C with ``extern "C"`` launchers (no framework headers), compiled in-tree
with ``nvcc -gencode arch=compute_100a,code=sm_100a`` and loaded through ``ctypes``; tensors cross
the boundary as raw pointers plus the current CUDA stream handle.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading
from typing import List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(_HERE))
CSRC = os.path.join(REPO, "csrc")
LIB_DIR = os.path.join(_HERE, "_lib")
LIB_PATH = os.path.join(LIB_DIR, "libtspipe_b200.so")
HASH_PATH = LIB_PATH + ".srchash"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


def sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _source_hash() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode())
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def nvcc_path() -> Optional[str]:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def is_fresh() -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(HASH_PATH)):
        return False
    with open(HASH_PATH) as f:
        return f.read().strip() == _source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every ``csrc/*.cu`` into one shared library (cross-compiles without a GPU)."""
    with _lock:
        if not force and is_fresh():
            return LIB_PATH
        nvcc = nvcc_path()
        if nvcc is None:
            raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")
        os.makedirs(LIB_DIR, exist_ok=True)
        tmp = LIB_PATH + f".tmp{os.getpid()}"
        cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp] + sources() + ["-lcuda"]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(res.stderr)
        os.replace(tmp, LIB_PATH)
        with open(HASH_PATH, "w") as f:
            f.write(_source_hash())
        return LIB_PATH


def load() -> ctypes.CDLL:
    """Load the library, building it first when it is missing or stale.  Raises when neither a
    library nor a compiler is available - the CUDA ops never fall back silently."""
    global _lib
    if _lib is not None:
        return _lib
    if not is_fresh():
        if nvcc_path() is not None:
            build()
        elif not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing and nvcc is unavailable; run __graft_entry__.build()")
    with _lock:
        if _lib is None:
            _lib = ctypes.CDLL(LIB_PATH)
    return _lib
