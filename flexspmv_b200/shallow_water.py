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
