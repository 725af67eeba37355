"""Builds libsimplicial_attn_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m simplical_attn_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIB_DIR, "libsimplicial_attn_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def nvcc_path() -> str:
    return os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def have_compiler() -> bool:
    return os.path.exists(nvcc_path())


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


STAMP = LIB + ".sources"      # digest of the sources the library was built from


def _deps():
    deps = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC))
    deps.append(os.path.join(os.path.dirname(PKG), "include", "simplicial_attn_b200.h"))
    return deps


def source_digest() -> str:
    """Digest of every file the library is compiled from and of the compiler flags.  File times are not
    used: a copy of the tree (a checkout, an archive) need not preserve them."""
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for d in _deps():
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale() -> bool:
    if not os.path.exists(LIB) or not os.path.exists(STAMP):
        return True
    with open(STAMP) as f:
        return f.read().strip() != source_digest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or was built from other sources; returns its path.  Every
    .cu file of csrc/ is one translation unit; the units compile side by side and are then linked."""
    if not force and not _stale():
        return LIB
    nvcc = nvcc_path()
    os.makedirs(LIB_DIR, exist_ok=True)
    digest = source_digest()
    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"]

    def compile_one(src: str):
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        res = subprocess.run([nvcc] + compile_flags + ["-c", "-o", obj, src], capture_output=True, text=True)
        return obj, res

    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(len(sources()), os.cpu_count() or 1))) as pool:
        results = list(pool.map(compile_one, sources()))
    for _, res in results:
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
    if any(res.returncode != 0 for _, res in results):
        raise RuntimeError("nvcc failed building " + LIB)
    link = subprocess.run([nvcc, "-shared", "-o", LIB] + [obj for obj, _ in results], capture_output=True, text=True)
    if verbose or link.returncode != 0:
        sys.stderr.write(link.stdout + link.stderr)
    if link.returncode != 0:
        raise RuntimeError("nvcc failed linking " + LIB)
    with open(STAMP, "w") as f:
        f.write(digest + "\n")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
