"""CPU ORACLE -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

numpy restatement of what the reference's *generated* CPU operator computes for a fused graph:

* the per-edge selector loads and map chain the emitters write
  (codegen/merged_gen_core.py:88-116 selectors, :122-236 map ops), with the value semantics of the
  reference's ``Tensor<ValueT, Dim>`` (data_struct_shared.cuh): element-wise + - *; ``/`` between
  tensors of EQUAL width and ``scalar / tensor`` return 0 where the divisor is 0 (:194-200,
  :402-408) while ``tensor / scalar`` (:238-244) and the mixed-width broadcast ``/`` (:611-625) are
  unguarded; ``^`` is pow; lt/gt give 0/1 in ValueT; ``_where`` selects on ``c != 0``; tensors of
  different width broadcast by index modulo (:611-625); ``l2Norm`` accumulates v*v left to right and
  takes one sqrt, producing a plain scalar (:346-353); in-place ops (add_, copy_, setitem) write
  through the input array at the edge's own slot (:160-165, :186-205);
* the reduction order of ``OmpMergeSystem`` (flex_oracle.c, compiled from this directory).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.  The map is
evaluated for all edges at once (numpy, in ValueT precision, one IEEE operation per reference
operation so float32/float64 results are bit-identical to the compiled reference for + - * / sqrt);
the per-row sums run in the C helper in the reference's order.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Dict, List, Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build_oracle_lib(force: bool = False) -> str:
    """gcc -O2 the C restatement into oracle/liboracle.so (no -march, no -ffast-math)."""
    src = os.path.join(_HERE, "flex_oracle.c")
    so = os.path.join(_HERE, "liboracle.so")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
        subprocess.check_call([cc, "-O2", "-fPIC", "-shared", "-ffp-contract=off", "-o", so, src])
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build_oracle_lib())
    return _LIB


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


_SUFFIX = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64", np.dtype(np.int64): "i64"}


# ----------------------------------------------------------------------------------------------
# partition helpers
# ----------------------------------------------------------------------------------------------

def merge_path_search(diagonal: int, row_offsets: np.ndarray, nnz: Optional[int] = None) -> Tuple[int, int]:
    """(row, nz) where `diagonal` crosses the merge path; row_offsets includes the leading 0."""
    n = row_offsets.shape[0] - 1
    nnz = int(row_offsets[-1]) if nnz is None else nnz
    if row_offsets.dtype == np.int32:
        x, y = ctypes.c_int32(), ctypes.c_int32()
        a = np.ascontiguousarray(row_offsets[1:])
        lib().merge_path_search_i32(ctypes.c_int32(diagonal), _p(a), ctypes.c_int32(n), ctypes.c_int32(nnz),
                                    ctypes.byref(x), ctypes.byref(y))
    else:
        x, y = ctypes.c_int64(), ctypes.c_int64()
        a = np.ascontiguousarray(row_offsets[1:].astype(np.int64))
        lib().merge_path_search_i64(ctypes.c_int64(diagonal), _p(a), ctypes.c_int64(n), ctypes.c_int64(nnz),
                                    ctypes.byref(x), ctypes.byref(y))
    return int(x.value), int(y.value)


def tile_coordinates(row_offsets: np.ndarray, tile_items: int) -> np.ndarray:
    """(num_tiles+1, 2) merge-path coordinates of the diagonals t*tile_items."""
    n = row_offsets.shape[0] - 1
    nnz = int(row_offsets[-1]) - int(row_offsets[0])
    assert int(row_offsets[0]) == 0
    tiles = (n + nnz + tile_items - 1) // tile_items
    ro = np.ascontiguousarray(row_offsets)
    if ro.dtype == np.int32:
        out = np.empty((tiles + 1, 2), np.int32)
        lib().tile_coordinates_i32(_p(ro), ctypes.c_int32(n), ctypes.c_int32(nnz), ctypes.c_int32(tile_items),
                                   ctypes.c_int32(tiles), _p(out))
    else:
        ro = ro.astype(np.int64)
        out = np.empty((tiles + 1, 2), np.int64)
        lib().tile_coordinates_i64(_p(ro), ctypes.c_int64(n), ctypes.c_int64(nnz), ctypes.c_int64(tile_items),
                                   ctypes.c_int64(tiles), _p(out))
    return out


def snap_cta_boundaries(coords: np.ndarray, row_offsets: np.ndarray, grid: int):
    """Restatement of the plan step that moves the tile boundaries in front of the CTAs of a ``grid``-CTA launch
    onto row ends (this package's own step, no reference counterpart).  CTA c starts at tile
    ``c q + min(c, r)`` (q, r = divmod(tiles, grid)); a boundary (x, y) that cuts row x moves back to
    ``(x, row_offsets[x])`` when the cut-off part fits the tile behind it (at most as many edges as that tile
    holds row ends) and the row starts inside the tile in front.  All boundaries or none.
    Returns (coords', snapped)."""
    tiles = coords.shape[0] - 1
    n = row_offsets.shape[0] - 1
    if grid < 2 or tiles < grid:
        return coords, False
    q, r = divmod(tiles, grid)
    out = coords.copy()
    for c in range(1, grid):
        t = c * q + min(c, r)
        x, y = int(coords[t, 0]), int(coords[t, 1])
        if x >= n:
            continue
        begin = int(row_offsets[x])
        if y - begin > int(coords[t + 1, 0]) - x or begin < int(coords[t - 1, 1]):
            return coords, False
        out[t, 1] = begin
    return out, True


def gather_window_plan(coords: np.ndarray, idx: np.ndarray, rec_bytes: int, win_bytes: int,
                       max_segs: int = 12, max_buckets: int = 160):
    """Restatement of the gather-window plan (this package's own format, no reference counterpart): per tile
    the columns are bucketed by 16, runs of buckets with at most one empty bucket between them become
    segments with exact column bounds, laid out consecutively at 16-byte boundaries (each shifted by
    ``(first * rec_bytes) & 15``); a tile with more than ``max_buckets`` buckets, more than ``max_segs``
    segments or more than ``win_bytes`` of window area gets none.  Returns (table (tiles, 2 + 2*max_segs) with
    [count, bytes, first0, len0, ...], positions (nnz,) uint16)."""
    tiles = coords.shape[0] - 1
    table = np.zeros((tiles, 2 + 2 * max_segs), np.int64)
    pos = np.zeros(idx.shape[0], np.uint16)
    for t in range(tiles):
        nz0, nz1 = int(coords[t, 1]), int(coords[t + 1, 1])
        c = idx[nz0:nz1].astype(np.int64)
        if c.size == 0:
            continue
        b = np.unique(c >> 4)
        if b.size > max_buckets:
            continue
        heads = np.concatenate([[True], np.diff(b) > 2])
        b0 = b[heads]
        if b0.size > max_segs:
            continue
        k = np.searchsorted(b0, c >> 4, side="right") - 1
        lo = np.array([c[k == j].min() for j in range(b0.size)])
        hi = np.array([c[k == j].max() for j in range(b0.size)])
        off, eoff = 0, []
        for j in range(b0.size):
            lead = (int(lo[j]) * rec_bytes) & 15
            eoff.append((off + lead) // rec_bytes)
            off += (lead + int(hi[j] - lo[j] + 1) * rec_bytes + 15) & ~15
        table[t, 1] = off
        if off > win_bytes or off // rec_bytes > 65535:
            continue
        table[t, 0] = b0.size
        table[t, 2:2 + 2 * b0.size:2] = lo
        table[t, 3:3 + 2 * b0.size:2] = hi - lo + 1
        pos[nz0:nz1] = (np.array(eoff)[k] + (c - lo[k])).astype(np.uint16)
    return table, pos


def nnz_balanced_row_blocks(row_offsets: np.ndarray, parts: int, snap: int = 1) -> np.ndarray:
    ro = np.ascontiguousarray(row_offsets.astype(np.int64))
    out = np.empty(parts + 1, np.int64)
    lib().nnz_balanced_row_blocks(_p(ro), ctypes.c_int64(ro.shape[0] - 1), ctypes.c_int32(parts),
                                  ctypes.c_int64(snap), _p(out))
    return out


# ----------------------------------------------------------------------------------------------
# Tensor<ValueT, Dim> semantics on (E, dim) arrays
# ----------------------------------------------------------------------------------------------

class Scalar:
    """A per-edge plain ValueT (the result of ``norm``), shape (E,)."""
    def __init__(self, a: np.ndarray):
        self.a = a


def _bcast(a: np.ndarray, out_dim: int) -> np.ndarray:
    d = a.shape[1]
    return a if d == out_dim else a[:, np.arange(out_dim) % d]


def _is_int(dt) -> bool:
    return np.issubdtype(np.dtype(dt), np.integer)


def _div(a, b, dt):
    if _is_int(dt):   # C++ integer division truncates toward zero
        q = np.abs(a) // np.maximum(np.abs(b), 1)
        return (q * np.sign(a) * np.sign(b)).astype(dt)
    with np.errstate(divide="ignore", invalid="ignore"):
        return (a / b).astype(dt)


def _guarded_div(a, b, dt):
    safe = np.where(b != 0, b, np.ones_like(b))
    return np.where(b != 0, _div(a, safe, dt), np.zeros_like(safe)).astype(dt)


def _pow(a, b, dt):
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        if _is_int(dt):   # tensor_pow<long> goes through double pow and truncates back
            return np.power(a.astype(np.float64), np.asarray(b, np.float64)).astype(dt)
        return np.power(a, b).astype(dt)


class IREvaluator:
    def __init__(self, ir, dtype):
        self.ir = ir
        self.dt = np.dtype(dtype)

    # -- operand handling -------------------------------------------------------------------
    def _lit(self, v):
        return self.dt.type(v)        # static_cast<ValueT>(literal)

    def _arg(self, env, a):
        if isinstance(a, str):
            return env[a]
        return self._lit(a)

    def _binary(self, op: str, A, B):
        dt = self.dt
        tA, tB = isinstance(A, np.ndarray), isinstance(B, np.ndarray)
        a = A.a[:, None] if isinstance(A, Scalar) else A
        b = B.a[:, None] if isinstance(B, Scalar) else B
        if not isinstance(a, np.ndarray) and not isinstance(b, np.ndarray):
            raise ValueError("binary op on two literals")
        same_width = True
        if tA and tB and A.shape[1] != B.shape[1]:        # index-modulo broadcast template
            od = max(A.shape[1], B.shape[1])
            a, b = _bcast(a, od), _bcast(b, od)
            same_width = False
        with np.errstate(over="ignore", invalid="ignore"):
            if op == "add":
                r = a + b
            elif op == "sub":
                r = a - b
            elif op == "mul":
                r = a * b
            elif op == "pow":
                r = _pow(a, b, dt)
            elif op == "truediv":
                if tA and tB:
                    # member operator/ (equal widths) is guarded, the broadcast template is not
                    r = _guarded_div(a, b, dt) if same_width else _div(a, b, dt)
                elif tB:                                   # scalar / tensor: guarded
                    r = _guarded_div(np.broadcast_to(np.asarray(a, dt), b.shape), b, dt)
                else:                                      # tensor / scalar: unguarded
                    r = _div(a, b, dt)
            elif op == "lt":
                r = (a < b)
            elif op == "gt":
                r = (a > b)
            else:
                raise ValueError(op)
        return np.asarray(r).astype(dt)

    # -- the whole map --------------------------------------------------------------------------
    def run_map(self, values: Dict[str, np.ndarray], indices: Dict[str, np.ndarray], num_edges: int):
        """Returns (env, written) where env maps every variable name to its per-edge value and
        `written` maps input-array names to their contents after in-place ops."""
        dt = self.dt
        env: Dict[str, object] = {}
        arrays = {k: (v.reshape(v.shape[0], -1).astype(dt, copy=True)) for k, v in values.items()}
        written = {}
        for s in self.ir.selector_register:
            if s.get("selector") == 1:
                idx = indices[s["selector_name"]].astype(np.int64)
                env[s["name"]] = arrays[s["target"]][idx]
            else:
                env[s["selector_name"]] = arrays[s["target"]][:num_edges].copy()
        for op in self.ir.map_operations:
            kind, name, args = op["op"], op["name"], op["args"]
            if kind in ("add", "sub", "mul", "pow", "truediv", "lt", "gt"):
                env[name] = self._binary(kind, self._arg(env, args[0]), self._arg(env, args[1]))
            elif kind == "neg":
                env[name] = (-env[args[0]]).astype(dt)
            elif kind == "exp":
                with np.errstate(over="ignore"):
                    env[name] = np.exp(env[args[0]]).astype(dt)
            elif kind == "abs":
                env[name] = np.abs(env[args[0]]).astype(dt)
            elif kind == "sign":
                env[name] = np.sign(env[args[0]]).astype(dt)
            elif kind == "norm":
                v = env[args[0]]
                acc = np.zeros(v.shape[0], dt)
                for i in range(v.shape[1]):
                    acc = (acc + (v[:, i] * v[:, i]).astype(dt)).astype(dt)
                env[name] = Scalar(np.sqrt(acc).astype(dt))
            elif kind == "getitem":
                env[name] = env[args[0]][:, [int(args[1][1])]].copy()
            elif kind == "clone":
                env[name] = env[args[0]].copy()
            elif kind == "where":
                c = env[args[0]]
                x, y = self._arg(env, args[1]), self._arg(env, args[2])
                od = max([c.shape[1]] + [t.shape[1] for t in (x, y) if isinstance(t, np.ndarray)])
                xb = _bcast(x, od) if isinstance(x, np.ndarray) else x
                yb = _bcast(y, od) if isinstance(y, np.ndarray) else y
                env[name] = np.where(_bcast(c, od) != 0, xb, yb).astype(dt)
            elif kind == "add_":
                env[args[0]] = self._binary("add", env[args[0]], self._arg(env, args[1]))
                arrays[args[0]][:num_edges] = env[args[0]]
                written[args[0]] = arrays[args[0]]
            elif kind == "copy_":
                arrays[args[0]][:num_edges] = env[args[1]]
                written[args[0]] = arrays[args[0]]
            elif kind == "setitem":
                arrays[args[0]][:num_edges] = env[args[2]]
                env[args[0]] = env[args[2]].copy()
                written[args[0]] = arrays[args[0]]
            elif kind in ("reducer", "sum"):
                pass
            else:
                raise ValueError(f"Operation {kind} not supported")
        return env, written


def _as_edge_array(v, dim: int, dt) -> np.ndarray:
    if isinstance(v, Scalar):
        return np.repeat(v.a[:, None], dim, axis=1).astype(dt)
    return np.ascontiguousarray(v.astype(dt))


def run_graph(ir, problem, dtype=None, num_threads: int = 8, want_abs_sums: bool = False):
    """Evaluate the operator on CPU.  Returns (outputs, written[, abs_sums]) where ``outputs`` follows
    the IR's ``outputs`` order with the operator's shapes (codegen/merged_gen_binding.py:100-123)."""
    from flexspmv_b200.graphs import dim_of   # IR helper only (no product code path)
    first = next(iter(problem.values.values()))
    dt = np.dtype(dtype or first.dtype)
    ev = IREvaluator(ir, dt)
    some_idx = next(iter(problem.indices.values()), None)
    ne = int(some_idx.shape[0]) if some_idx is not None else int(problem.num_cols)
    env, written = ev.run_map(problem.values, problem.indices, ne)
    sfx = _SUFFIX[dt]
    outputs, abs_sums = [], []
    for o in ir.outputs:
        d = dim_of(o["shape"])
        tgt = str(o["target"])
        if tgt == "reducer":
            red = next(r for r in ir.reducer_operations if r["name"] == o["name"])
            ev_arr = _as_edge_array(env[red["args"][0]], d, dt)
            ro = np.ascontiguousarray(problem.row_offsets.astype(np.int32))
            y = np.zeros((problem.num_rows, d), dt)
            getattr(lib(), f"omp_merge_reduce_{sfx}")(
                ctypes.c_int(num_threads), _p(ro), _p(ev_arr), ctypes.c_int(d),
                ctypes.c_int(problem.num_rows), ctypes.c_int(ne), _p(y))
            outputs.append(y[:, 0].copy() if d == 1 else y)
            if want_abs_sums:
                at = np.ascontiguousarray(np.abs(ev_arr.astype(np.float64)))
                s = np.zeros((problem.num_rows, d), np.float64)
                lib().row_abs_sum_f64(_p(ro), _p(at), ctypes.c_int(d), ctypes.c_int(problem.num_rows), _p(s))
                abs_sums.append(s[:, 0].copy() if d == 1 else s)
        elif "sum" in tgt:
            agg = next(a for a in ir.aggregator_operations if a["name"] == o["name"])
            ev_arr = _as_edge_array(env[agg["args"][0]], d, dt)
            res = np.zeros(d, dt)
            getattr(lib(), f"omp_merge_sum_{sfx}")(
                ctypes.c_int(num_threads), _p(ev_arr), ctypes.c_int(d), ctypes.c_int(problem.num_rows),
                ctypes.c_int(ne), _p(res))
            outputs.append(res)
            if want_abs_sums:
                abs_sums.append(np.abs(ev_arr.astype(np.float64)).sum(axis=0))
        else:
            v = _as_edge_array(env[o["name"]], d, dt)
            outputs.append(v[:, 0].copy() if d == 1 else v)
            if want_abs_sums:
                abs_sums.append(np.abs(v.astype(np.float64)))
    written = {k: (v[:, 0].copy() if problem.values[k].ndim == 1 else v) for k, v in written.items()}
    if want_abs_sums:
        return outputs, written, abs_sums
    return outputs, written
