"""Builds libsmelt_cuda.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m smelt_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(OUT_DIR, "libsmelt_cuda.so")
SOURCES = ["runtime.cu", "dispatch.cu", "builder.cu", "tp.cu", "affine_matvec.cu", "affine_stream.cu", "affine_imma.cu", "affine_qmm.cu", "affine_qmm_wide.cu", "attention.cu", "glue.cu", "signed_matvec.cu", "signed_imma.cu", "no_alloc.cu", "package_reader.cu", "snapshot.cu", "prefill.cu", "deltanet.cu", "recurrence_steps.cu", "bitplane.cu", "elementwise.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-DSMELT_BUILD",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _deps(src: str):
    yield src
    for f in os.listdir(CSRC):
        if f.endswith((".h", ".cuh")):
            yield os.path.join(CSRC, f)
    yield os.path.join(os.path.dirname(HERE), "include", "smelt_cuda.h")


def _compile(src: str, force: bool, verbose: bool) -> str:
    obj = os.path.join(OUT_DIR, os.path.basename(src).replace(".cu", ".o"))
    path = os.path.join(CSRC, src)
    if not force and os.path.exists(obj) and all(os.path.getmtime(obj) >= os.path.getmtime(d) for d in _deps(path)):
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", path, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), file=sys.stderr)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr, file=sys.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose), SOURCES))
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-Xlinker", "--no-undefined", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
