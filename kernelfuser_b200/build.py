"""Build libkf_b200.so in-tree with nvcc for sm_100a.

    python -m kernelfuser_b200.build [--force] [--verbose]

The library is a plain C-ABI shared object (no torch, no pybind); it is built
next to this file so that it ships with the source tree.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libkf_b200.so"
STAMP = PKG / "libkf_b200.srchash"  # content hash of the sources the library was built from
SOURCES = [CSRC / "kf_api.cu"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def have_nvcc() -> bool:
    n = _nvcc()
    return os.path.exists(n) or shutil.which(n) is not None


def _deps():
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "kf_b200.h"])


def _source_hash() -> str:
    h = hashlib.sha256()
    for d in _deps():
        h.update(d.name.encode())
        h.update(d.read_bytes())
    return h.hexdigest()


def stale() -> bool:
    """True when the library is missing or was built from other sources than the ones in the tree (compared by
    content, so that copying the tree to another machine does not make a fresh library look old)."""
    if not LIB.exists() or not STAMP.exists():
        return True
    return STAMP.read_text().strip() != _source_hash()


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
           "-Xcompiler", "-fPIC", "-shared",
           "-Xptxas", "-v" if verbose else "-warn-spills",
           "-o", str(LIB)] + [str(s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libkf_b200.so")
    STAMP.write_text(_source_hash() + "\n")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
