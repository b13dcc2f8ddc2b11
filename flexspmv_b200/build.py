"""Builds libflexspmv_b200.so in-tree: generates one CUDA translation unit per (graph, value type)
from the IR (codegen/emit_cuda.py), compiles everything for sm_100a with nvcc and links one shared
library with a plain C ABI (include/flexspmv.h).  No torch headers are involved.

    python -m flexspmv_b200.build [--force] [--jobs N] [--verbose-ptxas]
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import subprocess
import sys

from .codegen.emit_cuda import CTYPE, emit_graph
from .graphs import ALL_GRAPHS, GRAPH_DTYPES

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
BUILD = os.environ.get("FLEXSPMV_BUILD_DIR", os.path.join(ROOT, "build", "flexspmv"))
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.environ.get("FLEXSPMV_LIB_OUT", os.path.join(LIB_DIR, "libflexspmv_b200.so"))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",            # one IEEE operation per map operation, as the reference CPU code evaluates it
    "--expt-relaxed-constexpr", "-diag-suppress", "177", "-Xcompiler", "-fPIC", "-Xcompiler", "-O2",
    "-I", CSRC, "-I", os.path.join(ROOT, "include"),
] + os.environ.get("FLEXSPMV_NVCC_EXTRA", "").split()


def _headers_digest() -> str:
    h = hashlib.sha1()
    for d in (CSRC, os.path.join(ROOT, "include")):
        for f in sorted(os.listdir(d)):
            if f.endswith((".cuh", ".h")):
                with open(os.path.join(d, f), "rb") as fh:
                    h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _compile(src: str, obj: str, extra=()) -> str:
    cmd = [NVCC] + NVCC_FLAGS + list(extra) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def generated_units():
    """[(symbol, source text)] for every built-in (graph, value type)."""
    units = []
    only = [g for g in os.environ.get("FLEXSPMV_ONLY_GRAPHS", "").split(",") if g]      # tuning builds: a subset of the graphs
    for name, make in ALL_GRAPHS.items():
        if only and name not in only:
            continue
        ir = make()
        for dt in GRAPH_DTYPES[name]:
            sym = f"{name}_{CTYPE[dt][1]}"
            # the fp64 SpMV also gets the entry point that keeps its scratch in a static device array
            static_bytes = (2 << 20) if sym == "spmv_f64" else 0
            units.append((sym, emit_graph(ir, dt, sym, static_scratch_bytes=static_bytes)))
    return units


def build(force: bool = False, jobs: int | None = None, verbose_ptxas: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    os.makedirs(os.path.dirname(LIB_PATH), exist_ok=True)
    hd = _headers_digest()
    extra = ["-Xptxas", "-v"] if verbose_ptxas else []
    work = []   # (src, obj)
    core_src = os.path.join(CSRC, "flex_core.cu")
    work.append((core_src, os.path.join(BUILD, "flex_core.o")))
    work.append((os.path.join(CSRC, "flex_sort.cu"), os.path.join(BUILD, "flex_sort.o")))
    for sym, text in generated_units():
        src = os.path.join(BUILD, f"graph_{sym}.cu")
        old = open(src).read() if os.path.exists(src) else None
        if old != text:
            with open(src, "w") as f:
                f.write(text)
        work.append((src, os.path.join(BUILD, f"graph_{sym}.o")))
    stamp_path = os.path.join(BUILD, "stamp.txt")
    stamps = {}
    if os.path.exists(stamp_path):
        for line in open(stamp_path):
            k, _, v = line.strip().partition(" ")
            stamps[k] = v
    todo = []
    for src, obj in work:
        key = hashlib.sha1(open(src, "rb").read()).hexdigest()[:16] + hd
        if force or verbose_ptxas or not os.path.exists(obj) or stamps.get(obj) != key:
            todo.append((src, obj, key))
    logs = {}
    if todo:
        with cf.ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 4)) as ex:
            futs = {ex.submit(_compile, s, o, extra): (s, o, k) for s, o, k in todo}
            for fu in cf.as_completed(futs):
                s, o, k = futs[fu]
                logs[s] = fu.result()
                stamps[o] = k
        with open(stamp_path, "w") as f:
            for k, v in stamps.items():
                f.write(f"{k} {v}\n")
    if todo or not os.path.exists(LIB_PATH):
        objs = [o for _, o in work]
        cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH] + objs
        subprocess.check_call(cmd)
    if verbose_ptxas:
        for s, lg in logs.items():
            print("====", os.path.basename(s))
            print(lg)
    return LIB_PATH


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose_ptxas="--verbose-ptxas" in sys.argv)
    print("built", p)
