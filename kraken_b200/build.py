"""Builds kraken_b200/libkrk_cuda.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m kraken_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. Objects are cached under kraken_b200/build/ by source
hash, so a rebuild only recompiles what changed.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libkrk_cuda.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-I", os.path.join(ROOT, "include"), "-I", CSRC]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-I", os.path.join(ROOT, "include"), "-I", CSRC]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _sources():
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpp = sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp"))
    return cu, cpp


def _digest(path: str, flags) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(open(path, "rb").read())
    for dep_dir in (CSRC, os.path.join(ROOT, "include")):
        for f in sorted(os.listdir(dep_dir)):
            if f.endswith((".cuh", ".h", ".hpp")):
                h.update(open(os.path.join(dep_dir, f), "rb").read())
    return h.hexdigest()[:16]


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    cu, cpp = _sources()
    cc = nvcc()
    jobs = []
    objs = []
    for f in cu + cpp:
        src = os.path.join(CSRC, f)
        is_cu = f.endswith(".cu")
        flags = (ARCH + NVCC_FLAGS) if is_cu else CXX_FLAGS
        if verbose and is_cu:
            flags = flags + ["-Xptxas", "-v"]
        obj = os.path.join(OBJ, f"{f}.{_digest(src, flags)}.o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            cmd = ([cc] + flags + ["-c", src, "-o", obj]) if is_cu else \
                  ([cc, "-x", "c++", "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-I",
                   os.path.join(ROOT, "include"), "-I", CSRC, "-c", src, "-o", obj])
            jobs.append((f, cmd))
    def run(job):
        name, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"compiling {name} failed:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(f"== {name}\n{r.stderr}\n")
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    # drop objects of older source revisions
    keep = set(objs)
    for f in os.listdir(OBJ):
        p = os.path.join(OBJ, f)
        if p.endswith(".o") and p not in keep:
            os.remove(p)
    if jobs or force or not os.path.exists(LIB):
        cmd = [cc] + ARCH + ["-shared", "-o", LIB] + objs + ["-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking libkrk_cuda.so failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
