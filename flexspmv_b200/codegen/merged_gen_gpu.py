"""Entry points with the reference's names: IR (or FX sub-graph) -> CUDA -> loadable operator.

Reference flow (codegen/merged_gen_gpu.py:17-465, test_full/easier_full.py:283-373):
``generate_cuda_code_from_graph(submodule, traced_model)`` traces the FX sub-graph into the 6-tuple,
writes generated headers into the source tree and a pybind11 binding, then the driver JIT-builds it
with ``torch.utils.cpp_extension.load`` and hands the module to ``dynamic_replace_submodule``.

Here the same three steps are: ``trace_graph`` (flexspmv_b200/trace/graph_trace.py; needs the third-party
``easier`` package only for real FX graphs) -> ``emit_cuda.emit_graph`` (one self-contained ``.cu`` per
value type, nothing is written into the source tree) -> ``nvcc -shared`` into a per-graph cache
directory -> ``GraphExtension`` (binding.py), the object whose ``merged_spmv_launch`` the wrapper calls.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
from typing import Iterable, Optional

from ..graphs import GraphIR
from .emit_cuda import CTYPE, emit_graph

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_ROOT = os.path.dirname(_PKG)


def _cache_dir() -> str:
    d = os.environ.get("FLEXSPMV_CACHE_DIR", os.path.join(_ROOT, "build", "jit"))
    os.makedirs(d, exist_ok=True)
    return d


def generate_cuda_code_from_ir(ir: GraphIR, dtypes: Iterable[str] = ("float32", "float64"),
                               out_dir: Optional[str] = None) -> list:
    """Writes one translation unit per value type and returns their paths."""
    out_dir = out_dir or os.path.join(_cache_dir(), f"{ir.name}_{ir.digest()}")
    os.makedirs(out_dir, exist_ok=True)
    paths = []
    for dt in dtypes:
        sym = f"{ir.name}_{CTYPE[dt][1]}"
        path = os.path.join(out_dir, f"graph_{sym}.cu")
        text = emit_graph(ir, dt, sym)
        if not os.path.exists(path) or open(path).read() != text:
            with open(path, "w") as f:
                f.write(text)
        paths.append(path)
    return paths


def build_extension(ir: GraphIR, dtypes: Iterable[str] = ("float32", "float64"), force: bool = False, **ext_kw):
    """Generates, compiles (nvcc, sm_100a) and loads the operator for ``ir``; returns the object with
    ``merged_spmv_launch``.  The shared object is cached by IR digest, tool flags and kernel headers."""
    from .. import build as lib_build
    from ..binding import GraphExtension
    dtypes = tuple(dtypes)
    srcs = generate_cuda_code_from_ir(ir, dtypes)
    key = hashlib.sha1((ir.digest() + "".join(dtypes) + lib_build._headers_digest()).encode()).hexdigest()[:16]
    so = os.path.join(os.path.dirname(srcs[0]), f"libflexspmv_{ir.name}_{key}.so")
    if force or not os.path.exists(so):
        core = os.path.join(lib_build.CSRC, "flex_core.cu")
        cmd = [lib_build.NVCC] + lib_build.NVCC_FLAGS + ["-shared", "-o", so, core] + srcs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for graph '{ir.name}':\n{r.stdout}\n{r.stderr}")
    return GraphExtension(ir, lib_path=so, **ext_kw)


def generate_cuda_code_from_graph(submodule, traced_model, dtypes: Iterable[str] = ("float32", "float64"),
                                  name: Optional[str] = None, row_identity_selectors: Iterable[str] = ()):
    """Reference-named entry point: FX sub-graph -> IR -> generated sources.  Returns (ir, paths).
    ``row_identity_selectors`` names selectors whose index array equals the row id of every edge (e.g.
    the source selector of a graph reduced by source vertex); the kernel then skips that index array."""
    from ..trace.graph_trace import trace_graph
    six = trace_graph(submodule, traced_model)
    ir = GraphIR(name or "fused", *six)
    marked = set(row_identity_selectors)
    for s in ir.selector_register:
        if s.get("selector") == 1 and s["selector_name"] in marked:
            s["row_identity"] = True
    return ir, generate_cuda_code_from_ir(ir, dtypes)
