"""CPU ORACLE -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Calls the reference's own generated CPU operator (the shared objects ref_build.py compiles into
oracle/_ref from the reference's sources).  Used to pin the numpy/C restatement, to generate the
golden fixtures and as the timed "reference" CPU baseline.  Output shapes follow the reference
binding (codegen/merged_gen_binding_cpu.py:100-123): reducers (num_rows, dim), ``sum`` aggregators
(dim,), per-edge map outputs (ne, dim); all zero-initialised like the binding's torch::zeros.
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Dict, List, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_OUT = os.path.join(_HERE, "_ref")
_SFX = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64", np.dtype(np.int64): "i64"}
_libs: Dict[str, ctypes.CDLL] = {}
_manifest = None


def available(graph: Optional[str] = None) -> bool:
    mp = os.path.join(REF_OUT, "manifest.json")
    if not os.path.exists(mp):
        return False
    if graph is None:
        return True
    m = manifest()
    return graph in m and os.path.exists(os.path.join(REF_OUT, m[graph]["so"]))


def manifest() -> dict:
    global _manifest
    if _manifest is None:
        with open(os.path.join(REF_OUT, "manifest.json")) as f:
            _manifest = json.load(f)
    return _manifest


def _lib(graph: str, variant: str = "so") -> ctypes.CDLL:
    key = graph + ":" + variant
    if key not in _libs:
        _libs[key] = ctypes.CDLL(os.path.join(REF_OUT, manifest()[graph][variant]))
    return _libs[key]


def cpu_supports_x86_64_v3() -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            flags = next((ln for ln in f if ln.startswith("flags")), "")
    except OSError:
        return False
    return all(k in flags.split() for k in ("avx2", "fma", "bmi2", "movbe"))


def variants(graph: str) -> List[str]:
    """Objects of this graph that can run on this host: "so" (portable) and, where it was built and the CPU has
    AVX2 + FMA, "so_x86_64_v3"."""
    out = ["so"]
    ent = manifest()[graph]
    if "so_x86_64_v3" in ent and os.path.exists(os.path.join(REF_OUT, ent["so_x86_64_v3"])) and cpu_supports_x86_64_v3():
        out.append("so_x86_64_v3")
    return out


def reference_merge_path_search(row_offsets: np.ndarray, diagonals) -> np.ndarray:
    """The reference header's own MergePathSearch (cpu_template/merged_spmv_template_reducer.h:27-51) on the
    row END offsets of a CSR offset array with the leading 0, for each diagonal: (len(diagonals), 2) int32."""
    fn = _lib("spmv").ref_merge_path_search
    ro = np.ascontiguousarray(row_offsets.astype(np.int32))
    num_rows, nnz = int(ro.shape[0] - 1), int(ro[-1])
    ends = ro[1:]
    out = np.zeros((len(diagonals), 2), np.int32)
    xy = (ctypes.c_int * 2)()
    for i, d in enumerate(diagonals):
        fn(ctypes.c_int(int(d)), ends.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(num_rows), ctypes.c_int(nnz), xy)
        out[i, 0], out[i, 1] = xy[0], xy[1]
    return out


class PreparedCall:
    """Arguments marshalled once so a timing loop measures only the reference operator."""

    def __init__(self, ir, problem, dtype=None, num_threads: int = 8, variant: str = "so", copy_inputs: bool = True):
        """``copy_inputs=False`` passes arrays that already have the right dtype without a private copy (large
        timing problems; graphs with in-place map ops then write through the caller's arrays)."""
        from flexspmv_b200.graphs import dim_of
        ent = manifest()[ir.name]
        first = next(iter(problem.values.values()))
        self.dt = np.dtype(dtype or first.dtype)
        self.fn = getattr(_lib(ir.name, variant), f"ref_run_{_SFX[self.dt]}")
        self.num_threads = min(int(num_threads), 256)   # carry-outs are [256] arrays (merged_gen_core.py:75-77)
        some_idx = next(iter(problem.indices.values()), None)
        self.ne = int(some_idx.shape[0]) if some_idx is not None else int(problem.num_cols)
        self.num_rows = int(problem.num_rows)
        self.keep: List[np.ndarray] = []
        self.inputs: Dict[str, np.ndarray] = {}
        self.outputs: List[np.ndarray] = []
        out_by_name = {}
        for o in ir.outputs:
            d = dim_of(o["shape"])
            tgt = str(o["target"])
            if tgt == "reducer":
                shape = (self.num_rows,) if d == 1 else (self.num_rows, d)
            elif "sum" in tgt:
                shape = (d,)
            else:
                shape = (self.ne,) if d == 1 else (self.ne, d)
            a = np.zeros(shape, self.dt)
            self.outputs.append(a)
            out_by_name["output_y_" + o["name"]] = a
        ptrs = []
        for kind, name in ent["params"]:
            if name in out_by_name:
                a = out_by_name[name]
            elif kind == "index":
                a = np.ascontiguousarray(problem.indices[name].astype(np.int32, copy=False))
            else:
                a = np.ascontiguousarray(problem.values[name].astype(self.dt, copy=copy_inputs))
                self.inputs[name] = a
            self.keep.append(a)
            ptrs.append(a.ctypes.data)
        self.ptrs = (ctypes.c_void_p * len(ptrs))(*ptrs)
        if ent["has_rows"]:
            self.ro = np.ascontiguousarray(problem.row_offsets.astype(np.int32, copy=False))
        else:
            self.ro = np.zeros(1, np.int32)

    def run(self):
        self.fn(ctypes.c_int(self.num_threads), self.ro.ctypes.data_as(ctypes.c_void_p), self.ptrs,
                ctypes.c_int(self.num_rows), ctypes.c_int(self.ne))
        return self.outputs


def run_graph(ir, problem, dtype=None, num_threads: int = 8):
    """Returns (outputs in IR order, dict of input arrays after the call (in-place ops))."""
    pc = PreparedCall(ir, problem, dtype, num_threads)
    outs = pc.run()
    return outs, pc.inputs
