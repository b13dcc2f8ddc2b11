"""Seeded synthetic problems for the five benchmark configurations and for the unit tests.

The reference measures on no public data set: its harnesses draw a seeded random CSR problem
(src/flex_spmv_full_red.cu:391-427, main.cpp:126-176).  The generators here produce the matrices,
meshes and states the benchmark configurations describe; every one takes its size as a parameter so
the same code feeds small parity cases and the full-size benchmark.  All host generators use
``numpy.random.default_rng(seed)`` and return plain numpy arrays (identical arrays go to the CPU
oracle and to the GPU).  ``*_device`` variants build the two largest problems directly in GPU memory
with torch (same distributions, torch's generator) because shipping 2-15 GB from the host would
dominate a benchmark run.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np


@dataclass
class Problem:
    """Inputs of one operator call, in the reference IR's naming.

    ``values``  name -> array (num_edges, dim) or (num_vertices, dim) (dim==1 arrays are 1-D)
    ``indices`` selector target name -> int32 (num_edges,)
    ``row_offsets`` CSR offsets with the leading 0 (length num_rows+1), int32 or int64
    """
    graph: str
    values: Dict[str, np.ndarray]
    indices: Dict[str, np.ndarray]
    row_offsets: Optional[np.ndarray]
    num_rows: int
    num_cols: int
    meta: Dict[str, object] = field(default_factory=dict)

    @property
    def nnz(self) -> int:
        return int(next(iter(self.indices.values())).shape[0])


# ----------------------------------------------------------------------------------------------
# config 0 / config 4: Poisson stencils
# ----------------------------------------------------------------------------------------------

def poisson2d(n: int = 512, seed: int = 0, dtype=np.float64) -> Problem:
    """5-point Laplacian on an n x n grid, Dirichlet (out-of-grid neighbours dropped), CSR sorted,
    4.0 on the diagonal and -1.0 off it; x ~ U(-1,1)."""
    idx = np.arange(n * n, dtype=np.int64)
    i, j = idx // n, idx % n
    cand_col = np.stack([idx - n, idx - 1, idx, idx + 1, idx + n], axis=1)
    valid = np.stack([i > 0, j > 0, np.ones_like(i, bool), j < n - 1, i < n - 1], axis=1)
    cand_val = np.broadcast_to(np.array([-1.0, -1.0, 4.0, -1.0, -1.0]), cand_col.shape)
    counts = valid.sum(axis=1)
    ro = np.zeros(n * n + 1, dtype=np.int32)
    np.cumsum(counts, out=ro[1:])
    cols = cand_col[valid].astype(np.int32)
    vals = cand_val[valid].astype(dtype)
    x = np.random.default_rng(seed).uniform(-1.0, 1.0, n * n).astype(dtype)
    return Problem("spmv", {"vals": vals, "x": x}, {"selector": cols}, ro, n * n, n * n,
                   {"config": 0, "grid": n})


def poisson3d(n: int = 512, seed: int = 4, dtype=np.float64, offset_dtype=np.int64,
              z_begin: int = 0, z_end: Optional[int] = None, with_x: bool = True) -> Problem:
    """7-point Laplacian on an n^3 grid (x fastest), Dirichlet, 6.0 / -1.0, rows of z-planes
    [z_begin, z_end); column indices are global.  x ~ U(-1,1) over the whole grid."""
    z_end = n if z_end is None else z_end
    n2 = n * n
    idx = np.arange(z_begin * n2, z_end * n2, dtype=np.int64)
    k, r = idx // n2, idx % n2
    j, i = r // n, r % n
    cand_col = np.stack([idx - n2, idx - n, idx - 1, idx, idx + 1, idx + n, idx + n2], axis=1)
    valid = np.stack([k > 0, j > 0, i > 0, np.ones_like(i, bool), i < n - 1, j < n - 1, k < n - 1], axis=1)
    cand_val = np.broadcast_to(np.array([-1.0, -1.0, -1.0, 6.0, -1.0, -1.0, -1.0]), cand_col.shape)
    ro = np.zeros(idx.shape[0] + 1, dtype=offset_dtype)
    np.cumsum(valid.sum(axis=1), out=ro[1:])
    cols = cand_col[valid].astype(np.int32)
    vals = cand_val[valid].astype(dtype)
    x = np.random.default_rng(seed).uniform(-1.0, 1.0, n ** 3).astype(dtype) if with_x else np.zeros(0, dtype)
    return Problem("spmv", {"vals": vals, "x": x}, {"selector": cols}, ro, idx.shape[0], n ** 3,
                   {"config": 4, "grid": n, "z_begin": z_begin, "z_end": z_end})


def poisson3d_chunked(n: int = 512, seed: int = 4, dtype=np.float64, offset_dtype=np.int32) -> Problem:
    """The same matrix and vector as ``poisson3d(n)`` (all planes), assembled plane by plane into preallocated
    arrays from three plane templates (first, interior, last z-plane: every interior plane has the same
    pattern shifted by n^2 columns), so that the 512^3 problem (937,951,232 non-zeros) is built in seconds and
    needs little more host memory than its own 13 GB.  int32 offsets hold it (the reference's only offset
    width)."""
    if n < 3:
        p = poisson3d(n, seed, dtype, offset_dtype)
        return p
    n2, n3 = n * n, n ** 3
    nnz = 7 * n3 - 6 * n2
    assert np.dtype(offset_dtype).itemsize == 8 or nnz + n3 < 2 ** 31
    ro = np.zeros(n3 + 1, dtype=offset_dtype)
    cols = np.empty(nnz, dtype=np.int32)
    vals = np.empty(nnz, dtype=dtype)
    tmpl = {}
    for key, z in (("first", 0), ("mid", 1), ("last", n - 1)):
        part = poisson3d(n, seed, dtype, np.int64, z, z + 1, with_x=False)
        tmpl[key] = (part.indices["selector"].astype(np.int64) - z * n2, part.values["vals"], part.row_offsets[1:])
    e0 = 0
    for z in range(n):
        c, v, r = tmpl["first" if z == 0 else ("last" if z == n - 1 else "mid")]
        m = c.shape[0]
        np.add(c, z * n2, out=cols[e0:e0 + m], casting="unsafe")
        vals[e0:e0 + m] = v
        np.add(r, e0, out=ro[z * n2 + 1:(z + 1) * n2 + 1], casting="unsafe")
        e0 += m
    assert e0 == nnz
    x = np.random.default_rng(seed).uniform(-1.0, 1.0, n3).astype(dtype)
    return Problem("spmv", {"vals": vals, "x": x}, {"selector": cols}, ro, n3, n3, {"config": 4, "grid": n})


# ----------------------------------------------------------------------------------------------
# config 1: spring-mass lattice
# ----------------------------------------------------------------------------------------------

def spring_mass(n: int = 1024, seed: int = 1, dtype=np.float32) -> Problem:
    """n x n particle lattice, 8-neighbour directed edges stored CSR by source vertex.
    p = grid*h + U(-0.2h, 0.2h), h = 1/n; L_e = |p_i - p_j| * U(0.9, 1.1); k_e ~ U(0.5, 2.0)
    (rng draw order: jitter, L factors, k)."""
    rng = np.random.default_rng(seed)
    h = 1.0 / n
    idx = np.arange(n * n, dtype=np.int64)
    i, j = idx // n, idx % n
    p = np.stack([j * h, i * h], axis=1) + rng.uniform(-0.2 * h, 0.2 * h, (n * n, 2))
    p = p.astype(dtype)
    offs = [(-1, -1), (-1, 0), (-1, 1), (0, -1), (0, 1), (1, -1), (1, 0), (1, 1)]
    cand = np.stack([(i + di) * n + (j + dj) for di, dj in offs], axis=1)
    valid = np.stack([((i + di) >= 0) & ((i + di) < n) & ((j + dj) >= 0) & ((j + dj) < n) for di, dj in offs], axis=1)
    ro = np.zeros(n * n + 1, dtype=np.int32)
    np.cumsum(valid.sum(axis=1), out=ro[1:])
    dst = cand[valid].astype(np.int32)
    src = np.repeat(idx, valid.sum(axis=1)).astype(np.int32)
    d0 = p[dst].astype(np.float64) - p[src].astype(np.float64)
    L = (np.sqrt((d0 * d0).sum(axis=1)) * rng.uniform(0.9, 1.1, dst.shape[0])).astype(dtype)
    k = rng.uniform(0.5, 2.0, dst.shape[0]).astype(dtype)
    return Problem("spring_mass", {"L": L, "k": k, "p": p}, {"sel_src": src, "sel_dst": dst}, ro,
                   n * n, n * n, {"config": 1, "grid": n})


# ----------------------------------------------------------------------------------------------
# config 2: shallow water on a triangulated square
# ----------------------------------------------------------------------------------------------

def shallow_water(n: int = 1024, dtype=np.float64) -> Problem:
    """n x n unit squares each split along the (0,0)-(1,1) diagonal into a lower (L: corners
    (0,0),(1,0),(1,1)) and an upper (U: (0,0),(1,1),(0,1)) triangle -> 2 n^2 cells, 3 faces per cell.
    Cell id = 2*(iy*n+ix) + {0: L, 1: U}.  Boundary faces are kept as self-edges (neighbour = the
    cell itself), which for the zero-velocity initial state gives the reflective-wall flux.
    State U = (h, hu, hv), h = 1 + 0.1 exp(-((x-.5)^2 + (y-.5)^2)/0.01) at centroids, hu = hv = 0.
    Face data per edge: outward unit normal (nx, ny) and face length.  Deterministic (no rng)."""
    hs = 1.0 / n
    sq = np.arange(n * n, dtype=np.int64)
    iy, ix = sq // n, sq % n
    cl, cu = 2 * sq, 2 * sq + 1
    r2 = np.sqrt(0.5)
    # lower triangle faces: bottom (normal 0,-1) -> U of square below; right (1,0) -> U of square to
    # the right; diagonal (normal (-1,1)/sqrt2) -> U of same square
    nb_l = np.stack([np.where(iy > 0, 2 * (sq - n) + 1, cl), np.where(ix < n - 1, 2 * (sq + 1) + 1, cl), cu], axis=1)
    # upper triangle faces: diagonal (normal (1,-1)/sqrt2) -> L of same square; top (0,1) -> L of the
    # square above; left (-1,0) -> L of square to the left
    nb_u = np.stack([cl, np.where(iy < n - 1, 2 * (sq + n), cu), np.where(ix > 0, 2 * (sq - 1), cu)], axis=1)
    nbr = np.empty((2 * n * n, 3), dtype=np.int64)
    nbr[0::2], nbr[1::2] = nb_l, nb_u
    face_l = np.array([[0.0, -1.0, hs], [1.0, 0.0, hs], [-r2, r2, hs * np.sqrt(2.0)]])
    face_u = np.array([[r2, -r2, hs * np.sqrt(2.0)], [0.0, 1.0, hs], [-1.0, 0.0, hs]])
    face = np.empty((2 * n * n, 3, 3))
    face[0::2], face[1::2] = face_l, face_u
    cx = np.empty(2 * n * n)
    cy = np.empty(2 * n * n)
    cx[0::2], cy[0::2] = (ix + 2.0 / 3.0) * hs, (iy + 1.0 / 3.0) * hs
    cx[1::2], cy[1::2] = (ix + 1.0 / 3.0) * hs, (iy + 2.0 / 3.0) * hs
    hgt = 1.0 + 0.1 * np.exp(-((cx - 0.5) ** 2 + (cy - 0.5) ** 2) / 0.01)
    U = np.stack([hgt, np.zeros_like(hgt), np.zeros_like(hgt)], axis=1).astype(dtype)
    cells = 2 * n * n
    ro = (3 * np.arange(cells + 1, dtype=np.int64)).astype(np.int32)
    self_idx = np.repeat(np.arange(cells, dtype=np.int32), 3)
    return Problem("rusanov", {"face": face.reshape(-1, 3).astype(dtype), "U": U},
                   {"sel_self": self_idx, "sel_nbr": nbr.reshape(-1).astype(np.int32)}, ro, cells, cells,
                   {"config": 2, "grid": n})


def swe_mesh(n: int = 1024, dtype=np.float64) -> Problem:
    """Inputs of the reference shallow-water model's fused ``delta`` graph (graphs.swe_delta_graph) on the
    triangulated n x n square of ``shallow_water``: one directed edge per interior face and side (src =
    the neighbour, dst = the cell the flux is scattered to), sorted by dst, so boundary cells have 2
    edges (1 in two corners) and interior cells 3; face vectors (sx, sy) = the SOURCE cell's outward normal x length
    (it points into dst), the orientation the reference's assembler writes
    (shallow_water_equation/assemble_shallow_water.py:178-215), interpolation weight alpha = 0.5 (equal-size cells), h as in ``shallow_water`` and a smooth
    non-zero momentum field.  Deterministic (no rng).  The reference reads the same arrays from its HDF5
    mesh files (shallow_water_equation/swe_main.py:19-75)."""
    base = shallow_water(n, np.float64)
    cells = base.num_rows
    nbr = base.indices["sel_nbr"].astype(np.int64)
    dst = base.indices["sel_self"].astype(np.int64)
    keep = nbr != dst                       # boundary faces are self-edges there: the model treats them separately
    src, dst = nbr[keep], dst[keep]
    face = base.values["face"][keep]
    ro = np.zeros(cells + 1, dtype=np.int64)
    np.cumsum(np.bincount(dst, minlength=cells), out=ro[1:])
    hs = 1.0 / n
    sq = np.arange(n * n)
    iy, ix = sq // n, sq % n
    cx, cy = np.empty(cells), np.empty(cells)
    cx[0::2], cy[0::2] = (ix + 2.0 / 3.0) * hs, (iy + 1.0 / 3.0) * hs
    cx[1::2], cy[1::2] = (ix + 1.0 / 3.0) * hs, (iy + 2.0 / 3.0) * hs
    h = base.values["U"][:, 0]
    uh = 0.05 * h * np.sin(2 * np.pi * cx) * np.cos(2 * np.pi * cy)
    vh = -0.05 * h * np.cos(2 * np.pi * cx) * np.sin(2 * np.pi * cy)
    values = {"alpha": np.full(src.shape[0], 0.5), "sx": 0.0 - face[:, 0] * face[:, 2], "sy": 0.0 - face[:, 1] * face[:, 2],
              "h": h, "uh": uh, "vh": vh}
    return Problem("swe_delta", {k: np.ascontiguousarray(v.astype(dtype)) for k, v in values.items()},
                   {"gather_src": src.astype(np.int32), "gather_dst": dst.astype(np.int32)},
                   ro.astype(np.int32), cells, cells, {"grid": n})


def swe_init_mesh(n: int = 64, dtype=np.float64) -> Problem:
    """Inputs of the mesh assembler's per-edge graph (graphs.swe_init_edges_graph) for the triangulated n x n square of
    ``swe_mesh``: the (n + 1)^2 grid ``points``, and for every interior edge the three vertex ids of its source cell
    (src_p0..2) and of its destination cell (dst_p0..2), as the reference reads them from its mesh files
    (shallow_water_equation/assemble_shallow_water.py:94-110).  Square (ix, iy) holds cell 2 sq = (v00, v10, v11) and
    cell 2 sq + 1 = (v00, v11, v01).  sx / sy / alpha start at zero and are written by the graph."""
    mesh = swe_mesh(n, np.float64)
    src, dst = mesh.indices["gather_src"].astype(np.int64), mesh.indices["gather_dst"].astype(np.int64)
    hs = 1.0 / n
    g = np.arange(n + 1) * hs
    points = np.stack(np.meshgrid(g, g, indexing="xy"), axis=-1).reshape(-1, 2)      # point iy * (n + 1) + ix = (x, y)
    sq = np.arange(n * n)
    iy, ix = sq // n, sq % n
    v00 = iy * (n + 1) + ix
    v10, v01, v11 = v00 + 1, v00 + (n + 1), v00 + (n + 2)
    cells = np.empty((2 * n * n, 3), np.int64)
    cells[0::2] = np.stack([v00, v10, v11], axis=1)
    cells[1::2] = np.stack([v00, v11, v01], axis=1)
    e = src.shape[0]
    values = {"sx": np.zeros(e, dtype), "sy": np.zeros(e, dtype), "alpha": np.zeros(e, dtype), "points": points.astype(dtype)}
    indices = {}
    for i in range(3):
        indices[f"src_p{i}"] = cells[src, i].astype(np.int32)
        indices[f"dst_p{i}"] = cells[dst, i].astype(np.int32)
    indices = {k: indices[k] for k in [f"src_p{i}" for i in range(3)] + [f"dst_p{i}" for i in range(3)]}
    return Problem("swe_init_edges", values, indices, None, 0, points.shape[0], {"grid": n})


def swe_init_cells_mesh(n: int = 64, dtype=np.float64) -> Problem:
    """Inputs of the mesh assembler's per-cell graph (graphs.swe_init_cells_graph): ``points`` and the three vertex ids
    of every cell of the triangulated n x n square (the cell numbering of ``swe_init_mesh``); area / x / y / h start
    at zero and are written by the graph."""
    em = swe_init_mesh(n, dtype)
    sq = np.arange(n * n)
    iy, ix = sq // n, sq % n
    v00 = iy * (n + 1) + ix
    v10, v01, v11 = v00 + 1, v00 + (n + 1), v00 + (n + 2)
    cells = np.empty((2 * n * n, 3), np.int64)
    cells[0::2] = np.stack([v00, v10, v11], axis=1)
    cells[1::2] = np.stack([v00, v11, v01], axis=1)
    nc = cells.shape[0]
    values = {k: np.zeros(nc, dtype) for k in ("area", "x", "y", "h")}
    values["points"] = em.values["points"]
    indices = {f"cells_p{i}": cells[:, i].astype(np.int32) for i in range(3)}
    return Problem("swe_init_cells", values, indices, None, 0, em.values["points"].shape[0], {"grid": n})


def swe_init_boundary_mesh(n: int = 64, dtype=np.float64) -> Problem:
    """Inputs of the mesh assembler's boundary graph (graphs.swe_init_boundary_graph) for the triangulated n x n
    square: one record per wall face -- its two end points (bp0, bp1) and the cell it belongs to (bcells; a corner
    cell with two wall faces appears twice) -- plus ``points`` and the cell centroids the per-cell graph computes.
    bsx / bsy start at zero and are written by the graph."""
    cm = swe_init_cells_mesh(n, dtype)
    points = cm.values["points"]
    cells = np.stack([cm.indices[f"cells_p{i}"].astype(np.int64) for i in range(3)], axis=1)
    centroid = ((points[cells[:, 0]] + points[cells[:, 1]]) + points[cells[:, 2]]) / 3.0
    ix, iy = points[:, 0] * n, points[:, 1] * n
    on_wall = lambda a, b: (((ix[a] == 0) & (ix[b] == 0)) | ((ix[a] == n) & (ix[b] == n)) |
                            ((iy[a] == 0) & (iy[b] == 0)) | ((iy[a] == n) & (iy[b] == n)))
    recs = []
    for f in range(3):
        a, b = cells[:, f], cells[:, (f + 1) % 3]
        c = np.flatnonzero(on_wall(a, b))
        recs.append(np.stack([c, a[c], b[c]], axis=1))
    rec = np.concatenate(recs)
    rec = rec[np.argsort(rec[:, 0], kind="stable")]
    nb = rec.shape[0]
    values = {"bsx": np.zeros(nb, dtype), "bsy": np.zeros(nb, dtype), "points": points, "centroid": centroid.astype(dtype)}
    indices = {"bp0": rec[:, 1].astype(np.int32), "bp1": rec[:, 2].astype(np.int32), "bcells": rec[:, 0].astype(np.int32)}
    return Problem("swe_init_boundary", values, indices, None, 0, points.shape[0], {"grid": n})


def swe_raw_mesh(n: int = 64) -> Dict[str, np.ndarray]:
    """The arrays of the reference's MESH file (shallow_water_equation/assemble_shallow_water.py:14-31,85-112) for the
    triangulated n x n square of ``swe_mesh``: ``points`` (np, 2), ``cells`` (nc, 3), ``src`` / ``dst`` (edges sorted by
    dst), ``bcells`` and ``bpoints`` (one record per wall face; a corner cell with two wall faces appears twice)."""
    cm = swe_init_cells_mesh(n)
    em = swe_mesh(n)
    bm = swe_init_boundary_mesh(n)
    cells = np.stack([cm.indices[f"cells_p{i}"].astype(np.int64) for i in range(3)], axis=1)
    return {"points": cm.values["points"], "cells": cells,
            "src": em.indices["gather_src"].astype(np.int64), "dst": em.indices["gather_dst"].astype(np.int64),
            "bcells": bm.indices["bcells"].astype(np.int64),
            "bpoints": np.stack([bm.indices["bp0"], bm.indices["bp1"]], axis=1).astype(np.int64)}


def swe_components_mesh(n: int = 64, dtype=np.int64) -> Problem:
    """Inputs of the components-collector graph (graphs.swe_components_graph): ``cells`` and the edge lists of
    ``swe_raw_mesh``; the six per-edge outputs start at zero and are written by the graph."""
    raw = swe_raw_mesh(n)
    e = raw["src"].shape[0]
    values = {f"{side}_p{i}": np.zeros(e, dtype) for side in ("src", "dst") for i in range(3)}
    values = {k: values[k] for k in [f"src_p{i}" for i in range(3)] + [f"dst_p{i}" for i in range(3)]}
    values["cells"] = raw["cells"].astype(dtype)
    indices = {"selector_src": raw["src"].astype(np.int32), "selector_dst": raw["dst"].astype(np.int32)}
    return Problem("swe_components", values, indices, None, 0, raw["cells"].shape[0], {"grid": n})


def swe_model_inputs(n: int = 64, dtype=np.float64) -> Dict[str, np.ndarray]:
    """Every array the reference's ``ShallowWaterEquation`` module loads (shallow_water_equation/
    swe_main.py:19-81) for the triangulated n x n square: interior edges (src, dst sorted by dst, alpha,
    sx, sy) as in ``swe_mesh``; boundary cells ``bcells`` (sorted) with the summed face vector (bsx, bsy)
    of their wall faces, pointing INTO the domain as the reference's assembler writes it
    (shallow_water_equation/assemble_shallow_water.py:241-248); cell ``area``; initial h, uh, vh."""
    interior = swe_mesh(n, dtype)
    base = shallow_water(n, np.float64)
    nbr = base.indices["sel_nbr"].astype(np.int64)
    own = base.indices["sel_self"].astype(np.int64)
    wall = nbr == own
    face = base.values["face"][wall]
    cells = base.num_rows
    bx = np.bincount(own[wall], weights=face[:, 0] * face[:, 2], minlength=cells)
    by = np.bincount(own[wall], weights=face[:, 1] * face[:, 2], minlength=cells)
    bcells = np.flatnonzero(np.bincount(own[wall], minlength=cells))
    hs = 1.0 / n
    d = dict(interior.values)
    d.update({"src": interior.indices["gather_src"], "dst": interior.indices["gather_dst"],
              "row_offsets": interior.row_offsets, "bcells": bcells.astype(np.int32),
              "bsx": (0.0 - bx[bcells]).astype(dtype), "bsy": (0.0 - by[bcells]).astype(dtype),
              "area": np.full(cells, 0.5 * hs * hs, dtype=dtype)})
    return d


# ----------------------------------------------------------------------------------------------
# config 3: power-law CSR
# ----------------------------------------------------------------------------------------------

def powerlaw_row_lengths(n: int, rng, mean_len: float = 16.0, cap: int = 100_000) -> np.ndarray:
    """raw = min(floor(1/(1-u)), cap), u ~ U[0,1)  (discrete power law, exponent 2, min 1);
    len = clip(round(raw * mean_len / mean(raw)), 1, cap)."""
    u = rng.random(n)
    raw = np.minimum(np.floor(1.0 / (1.0 - u)), cap)
    ln = np.clip(np.rint(raw * (mean_len / raw.mean())), 1, cap).astype(np.int64)
    return ln


def powerlaw(n: int = 1 << 24, seed: int = 3, dtype=np.float32, mean_len: float = 16.0,
             cap: int = 100_000) -> Problem:
    """n x n CSR, power-law row lengths, uniform random columns sorted within each row, values
    N(0,1), x ~ U(-1,1) (rng draw order: lengths, columns, values, x)."""
    rng = np.random.default_rng(seed)
    ln = powerlaw_row_lengths(n, rng, mean_len, min(cap, n))
    ro = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(ln, out=ro[1:])
    m = int(ro[-1])
    cols = rng.integers(0, n, m, dtype=np.int64)
    rows = np.repeat(np.arange(n, dtype=np.int64), ln)
    key = np.sort((rows << 32) | cols)
    cols = (key & 0xFFFFFFFF).astype(np.int32)
    vals = rng.standard_normal(m).astype(dtype)
    x = rng.uniform(-1.0, 1.0, n).astype(dtype)
    assert m < 2 ** 31
    return Problem("spmv", {"vals": vals, "x": x}, {"selector": cols}, ro.astype(np.int32), n, n,
                   {"config": 3})


# ----------------------------------------------------------------------------------------------
# the reference harness' random problem (unit tests)
# ----------------------------------------------------------------------------------------------

def random_cut_csr(num_rows: int, nnz: int, rng) -> np.ndarray:
    """Row offsets = sorted random cut points, so empty rows and long rows both occur
    (the idea of src/flex_spmv_full_red.cu:391-427)."""
    cuts = np.sort(rng.integers(0, nnz + 1, max(num_rows - 1, 0)))
    ro = np.concatenate([[0], cuts, [nnz]]).astype(np.int32)
    return ro[: num_rows + 1] if num_rows > 0 else np.array([0], np.int32)


def random_problem(graph_ir, num_rows: int, num_vertices: int, nnz: int, seed: int, dtype,
                   integer_range: int = 7) -> Problem:
    """Random inputs for any graph IR: vertex tensors (num_vertices, dim), edge tensors (nnz, dim),
    selector indices uniform in [0, num_vertices), random cut-point CSR.  Row-identity selectors get
    the expanded row ids (and num_vertices is then forced to num_rows)."""
    from .graphs import dim_of
    rng = np.random.default_rng(seed)
    ro = random_cut_csr(num_rows, nnz, rng)
    is_int = np.issubdtype(np.dtype(dtype), np.integer)
    gather_src = {s["target"] for s in graph_ir.selector_register if s.get("selector") == 1}
    values, indices = {}, {}

    def draw(shape):
        if is_int:
            return rng.integers(-integer_range, integer_range + 1, shape).astype(dtype)
        a = rng.uniform(-1.0, 1.0, shape)
        a[rng.random(shape) < 0.02] = 0.0   # exact zeros exercise the guarded divide
        return a.astype(dtype)

    for inp in graph_ir.inputs:
        if inp["dtype"] == "int":
            continue
        d = dim_of(inp["shape"])
        rows = num_vertices if inp["name"] in gather_src else nnz
        a = draw((rows, d))
        values[inp["name"]] = a[:, 0].copy() if d == 1 else a
    if graph_ir.name == "rusanov":     # water depth must be positive for the flux to be defined
        values["U"][:, 0] = (np.abs(values["U"][:, 0]) + 0.5).astype(dtype)
    for s in graph_ir.selector_register:
        if s.get("selector") != 1 or s["selector_name"] in indices:
            continue
        if s.get("row_identity"):
            assert num_vertices == num_rows
            indices[s["selector_name"]] = np.repeat(np.arange(num_rows, dtype=np.int32), np.diff(ro))
        else:
            indices[s["selector_name"]] = rng.integers(0, num_vertices, nnz).astype(np.int32)
    return Problem(graph_ir.name, values, indices, ro if graph_ir.has_reducer else None, num_rows,
                   num_vertices, {"seed": seed})


# ----------------------------------------------------------------------------------------------
# algorithmic bytes
# ----------------------------------------------------------------------------------------------

def algorithmic_bytes(graph_ir, num_rows: int, nnz: int, num_vertices: int, value_bytes: int,
                      offset_bytes: int = 4) -> int:
    """Every compulsory array counted once (the reference's effective-bandwidth formula,
    src/flex_spmv_full_red.cu:347-359):  nnz*(4 per streamed index + V*sum(edge dims)) +
    (rows+1)*R + sum over gather sources V*dim*vertices + rows*V*sum(reducer dims) +
    nnz*V*dim per stored per-edge output.  A row-identity selector is derivable from the row
    offsets and is not counted."""
    from .graphs import dim_of
    b = 0
    seen_idx = set()
    for s in graph_ir.selector_register:
        if s.get("selector") == 1:
            if not s.get("row_identity") and s["selector_name"] not in seen_idx:
                b += 4 * nnz
                seen_idx.add(s["selector_name"])
        else:
            b += value_bytes * dim_of(s["shape"]) * nnz
    for src in {s["target"]: s for s in graph_ir.selector_register if s.get("selector") == 1}.values():
        b += value_bytes * dim_of(src["shape"]) * num_vertices
    if graph_ir.has_reducer:
        b += (num_rows + 1) * offset_bytes
    for o in graph_ir.outputs:
        d = dim_of(o["shape"])
        if str(o["target"]) == "reducer":
            b += value_bytes * d * num_rows
        elif "sum" in str(o["target"]):
            b += value_bytes * d
        else:
            b += value_bytes * d * nnz
    return b


# ----------------------------------------------------------------------------------------------
# device-side generators for the largest configuration (torch generator, same distributions)
# ----------------------------------------------------------------------------------------------

def powerlaw_device(n: int = 1 << 24, seed: int = 3, device="cuda", mean_len: float = 16.0, cap: int = 100_000):
    """Config 3 built directly in GPU memory: same construction as ``powerlaw`` (power-law lengths,
    uniform columns sorted within each row through the key row<<32|col, N(0,1) values, U(-1,1) x) but
    drawn from torch's device generator, so the arrays are not bit-identical to the numpy ones.
    Returns (row_offsets int32, cols int32, vals float32, x float32)."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    cap = min(cap, n)
    u = torch.rand(n, generator=g, device=device, dtype=torch.float64)
    raw = torch.clamp(torch.floor(1.0 / (1.0 - u)), max=float(cap))
    ln = torch.clamp(torch.round(raw * (mean_len / raw.mean())), 1, cap).to(torch.int64)
    del u, raw
    ro = torch.zeros(n + 1, dtype=torch.int64, device=device)
    torch.cumsum(ln, dim=0, out=ro[1:])
    m = int(ro[-1].item())
    assert m < 2 ** 31
    key = torch.repeat_interleave(torch.arange(n, dtype=torch.int64, device=device), ln)
    del ln
    key <<= 32
    key |= torch.randint(0, n, (m,), generator=g, device=device, dtype=torch.int64)
    key = torch.sort(key).values
    cols = (key & 0xFFFFFFFF).to(torch.int32)
    del key
    vals = torch.randn(m, generator=g, device=device, dtype=torch.float32)
    x = torch.rand(n, generator=g, device=device, dtype=torch.float32) * 2.0 - 1.0
    return ro.to(torch.int32), cols, vals, x
