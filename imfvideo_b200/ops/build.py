"""Build the sm_100a kernel library in-tree with plain nvcc.

``python -m imfvideo_b200.ops.build`` compiles every ``csrc/*.cu`` with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` and links
``ops/libimf_b200.so``.  Objects are cached by source hash, so an unchanged
file is not recompiled.  nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libimf_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-O2",
              "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _hash(path: str, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for dep in [path] + sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)
                               if f.endswith((".cuh", ".h"))):
        with open(dep, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def build(verbose: bool = True, ptxas_info: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else [])
    objs, jobs = [], []
    for src in sources():
        tag = _hash(src, " ".join(flags))
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + f".{tag}.o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc] + flags + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(f"[build] {os.path.basename(src)}", flush=True)
            if ptxas_info:
                print(r.stderr, flush=True)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    stale = not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB)
                                           for o in objs)
    if jobs or stale or force:
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(f"[build] linked {LIB}", flush=True)
    # drop objects of older source versions
    keep = set(objs)
    for f in os.listdir(OBJ_DIR):
        full = os.path.join(OBJ_DIR, f)
        if full.endswith(".o") and full not in keep:
            os.remove(full)
    return LIB


if __name__ == "__main__":
    build(ptxas_info="-v" in sys.argv, force="--force" in sys.argv)
