"""One time step of the reference's shallow-water model on the fused operators.

The reference model (shallow_water_equation/swe_main.py:12-146) is an ``easier`` module whose ``forward``
is a classical Runge-Kutta step; each of its four ``delta`` evaluations gathers h, uh, vh over the edges
(``gather_src`` / ``gather_dst``), blends them to face values, and scatters three flux sums per cell
(``scatter``) plus two wall terms on the boundary cells (``scatter_b``).  The reference replaces those
fused regions by generated operators and leaves the per-cell arithmetic to torch.  ``ShallowWaterStep``
runs the step on this package's kernels: per ``delta`` one launch of the ``swe_delta`` graph and one of
the ``swe_boundary`` graph (both bound once with ``GraphExtension.prepare``: no per-call marshalling, no
allocation), then one launch of ``flexspmv_swe_rk_stage`` for ``-(...)/area`` and the Runge-Kutta update
of that stage (about 60 torch element-wise kernels per step in the reference).  ``capture()`` records the
whole step (12 launches) into one CUDA graph.

Edges must be sorted by destination cell and ``bcells`` ascending: both Reducers then see sorted indices,
which is what the merge-path kernels need (python_wrapper/dynamic_replace_submodule.py:20-41 makes the
same assumption when it converts COO rows to CSR offsets).
"""
from __future__ import annotations

from typing import Dict, Optional

import ctypes

import torch

from .binding import GraphExtension, check, load_builtin
from .python_wrapper.dynamic_replace_submodule import coo_rows_to_csr_ptr


class ShallowWaterStep:
    def __init__(self, mesh: Dict[str, torch.Tensor], dt: float = 0.005,
                 delta_ext: Optional[GraphExtension] = None, boundary_ext: Optional[GraphExtension] = None):
        """``mesh``: CUDA tensors named as the reference module's attributes -- src, dst (int32, sorted by dst),
        bcells (int32, ascending), alpha, sx, sy (per edge), bsx, bsy (per boundary cell), area, h, uh, vh (per
        cell).  h, uh, vh are advanced in place."""
        self.dt = float(dt)
        m = self.m = mesh
        dev = m["h"].device
        self.nc = int(m["h"].numel())
        self.ne = int(m["src"].numel())
        self.nbc = int(m["bcells"].numel())
        self.delta_ext = delta_ext or load_builtin("swe_delta")
        self.boundary_ext = boundary_ext or load_builtin("swe_boundary")
        self.ro = coo_rows_to_csr_ptr(m["dst"], self.nc)
        self.ro_b = coo_rows_to_csr_ptr(m["bcells"], self.nc)
        dt_ = m["h"].dtype
        # stage inputs (the state the current delta is evaluated at) and the reducers' outputs
        self.stage = [torch.empty(self.nc, dtype=dt_, device=dev) for _ in range(3)]
        self.red = [torch.empty(self.nc, dtype=dt_, device=dev) for _ in range(3)]
        self.red_b = [torch.empty(self.nc, dtype=dt_, device=dev) for _ in range(2)]
        self._on_state = self._bind(m["h"], m["uh"], m["vh"])
        self._on_stage = self._bind(*self.stage)
        self.acc = [torch.empty(self.nc, dtype=dt_, device=dev) for _ in range(3)]
        ptrs = lambda ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
        self._p_red, self._p_red_b, self._p_acc, self._p_stage = ptrs(self.red), ptrs(self.red_b), ptrs(self.acc), ptrs(self.stage)
        self._p_x = ptrs([m["h"], m["uh"], m["vh"]])
        self.delta_ext.lib.flexspmv_swe_rk_stage.restype = ctypes.c_int
        self._graph: Optional[torch.cuda.CUDAGraph] = None

    def _bind(self, h, uh, vh):
        m = self.m
        d = self.delta_ext.prepare([m["alpha"], m["sx"], m["sy"], h, uh, vh], [m["src"], m["dst"]], self.ro,
                                   self.red, self.nc, self.ne, self.nc)
        b = self.boundary_ext.prepare([m["bsx"], m["bsy"], h], [m["bcells"]], self.ro_b, self.red_b, self.nc,
                                      self.nbc, self.nc)
        return d, b

    def _stage(self, c: float, first: bool, last: bool) -> None:
        fn = self.delta_ext.lib.flexspmv_swe_rk_stage
        st = fn(ctypes.c_int32(self.m["h"].element_size()), self._p_red, self._p_red_b,
                ctypes.c_void_p(self.m["area"].data_ptr()), self._p_x, self._p_acc, self._p_stage,
                ctypes.c_double(c), ctypes.c_double(self.dt / 6), ctypes.c_int64(self.nc),
                ctypes.c_int32(int(first)), ctypes.c_int32(int(last)),
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        check(self.delta_ext.lib, st, "swe_rk_stage")

    def forward(self) -> None:
        """swe_main.py:121-146: four delta evaluations (:86-119), each followed by its stage update."""
        dt = self.dt
        for k, c in enumerate((0.5 * dt, 0.5 * dt, dt, 0.0)):
            bound = self._on_state if k == 0 else self._on_stage
            bound[0].launch()
            bound[1].launch()
            self._stage(c, first=(k == 0), last=(k == 3))

    __call__ = forward

    # -- CUDA graph --------------------------------------------------------------------------------------
    def capture(self) -> None:
        """Records one step into a CUDA graph (after one eager step on a side stream to warm the allocator);
        ``replay()`` then advances the state by one step per call.  The warm-up step is undone."""
        saved = [self.m[k].clone() for k in ("h", "uh", "vh")]
        side = torch.cuda.Stream()          # warm-up and capture on one stream: the prepared launches are
        side.wait_stream(torch.cuda.current_stream())   # already ordered after their plans there
        with torch.cuda.stream(side):
            self.forward()
            for k, v in zip(("h", "uh", "vh"), saved):
                self.m[k].copy_(v)
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            self.forward()
        self._graph = g

    def replay(self) -> None:
        if self._graph is None:
            raise RuntimeError("capture() first")
        self._graph.replay()


def assemble_shallow_water(mesh: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """The reference's mesh assembler (``assemble_shallow_water``, shallow_water_equation/assemble_shallow_water.py:
    251-291) on the fused operators, with tensors where the reference reads and writes HDF5 data sets.

    ``mesh``: CUDA tensors named as the mesh file's data sets -- points (np, 2) float64, cells (nc, 3), src, dst (ne,),
    bcells (nbc,), bpoints (nbc, 2), all integer.  Returns what the reference saves: src_p0..2, dst_p0..2, cells_p0..2,
    bp0..1 (int64) and x, y, area, sx, sy, bsx, bsy, h, alpha (float64).  Four launches: the components collector's
    gathers (``swe_components``), then the initializer's per-edge, per-cell and boundary parts (``swe_init_edges``,
    ``swe_init_cells``, ``swe_init_boundary``); the column slices the collector also copies (:74-78) are torch slices.
    """
    points = mesh["points"].contiguous()
    dev = points.device
    cells = mesh["cells"].to(torch.int64).contiguous()
    nc, ne, nbc, npnt = int(cells.shape[0]), int(mesh["src"].numel()), int(mesh["bcells"].numel()), int(points.shape[0])
    i32 = lambda t: t.to(torch.int32).contiguous()
    dummy = torch.zeros(1, dtype=torch.int32, device=dev)      # row_end_offsets of a graph without a reducer
    out: Dict[str, torch.Tensor] = {}

    # ShallowWaterMeshComponentsCollector.forward (:62-78)
    comp = [torch.zeros(ne, dtype=torch.int64, device=dev) for _ in range(6)]
    load_builtin("swe_components").launch_into(comp + [cells], [i32(mesh["src"]), i32(mesh["dst"])], dummy, [], 0, ne, nc)
    for i in range(3):
        out[f"src_p{i}"], out[f"dst_p{i}"] = comp[i], comp[3 + i]
        out[f"cells_p{i}"] = cells[:, i].clone()
    bpoints = mesh["bpoints"].to(torch.int64)
    for i in range(2):
        out[f"bp{i}"] = bpoints[:, i].clone()

    # ShallowWaterInitializer.forward (:178-248)
    f64 = lambda n_: torch.zeros(n_, dtype=torch.float64, device=dev)
    for k in ("sx", "sy", "alpha"):
        out[k] = f64(ne)
    load_builtin("swe_init_edges").launch_into([out["sx"], out["sy"], out["alpha"], points],
                                               [i32(c) for c in comp], dummy, [], 0, ne, npnt)
    for k in ("area", "x", "y", "h"):
        out[k] = f64(nc)
    load_builtin("swe_init_cells").launch_into([out["area"], out["x"], out["y"], out["h"], points],
                                               [i32(out[f"cells_p{i}"]) for i in range(3)], dummy, [], 0, nc, npnt)
    centroid = torch.stack([out["x"], out["y"]], dim=1).contiguous()
    out["bsx"], out["bsy"] = f64(nbc), f64(nbc)
    load_builtin("swe_init_boundary").launch_into([out["bsx"], out["bsy"], points, centroid],
                                                  [i32(out["bp0"]), i32(out["bp1"]), i32(mesh["bcells"])], dummy, [], 0, nbc, npnt)
    return out
