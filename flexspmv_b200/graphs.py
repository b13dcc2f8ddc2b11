"""Fused-graph IR: the 6-tuple of dict lists that the reference's tracer hands to its code generators.

The reference's ``trace_graph`` (trace/graph_trace.py:32-328) returns
``(inputs, outputs, selector_register, map_operations, reducer_operations, aggregator_operations)``;
every emitter downstream (codegen/merged_gen_core.py, codegen/merged_gen_gpu.py,
codegen/merged_gen_binding.py) consumes only those lists.  ``easier`` (the package that produces the
FX graph) is a third-party dependency, so this module builds the same lists by hand for the graphs
the benchmark configurations need and for the unit-test graphs.  Dict keys follow
trace/graph_trace.py:133-157 (inputs), :179-205 (selector_register), :279-286 (map operations).

Two optional keys are an extension understood only by this package's CUDA emitter (the reference
emitters ignore unknown keys):

``row_identity`` (selector_register entry, selector == 1)
    the selector's index array equals the row id of every edge (``idx[e] == row(e)``), so the CUDA
    kernel derives it from the merge path instead of streaming the index array from HBM.  The array
    is still part of the operator signature.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Sequence, Tuple


class NodeRef:
    """Stand-in for a torch.fx Node: the binding generators only read ``args[0].name`` of a selector
    input (codegen/merged_gen_binding.py:46-48, codegen/merged_gen_binding_cpu.py:46-48)."""

    def __init__(self, name: str):
        self.name = name

    def __repr__(self) -> str:  # printed by the emitters when they str() an argument
        return self.name


@dataclass
class GraphIR:
    """One fused sub-graph in the reference's IR.  ``value_dtype`` is 'float32' | 'float64' | 'int64'
    for the instance that gets compiled (the reference dispatches float/double(/long) at run time,
    cuda_template/merged_binding_template.cu:55-69)."""

    name: str
    inputs: List[Dict[str, Any]]
    outputs: List[Dict[str, Any]]
    selector_register: List[Dict[str, Any]]
    map_operations: List[Dict[str, Any]]
    reducer_operations: List[Dict[str, Any]]
    aggregator_operations: List[Dict[str, Any]]
    doc: str = ""

    def as_tuple(self):
        return (self.inputs, self.outputs, self.selector_register, self.map_operations,
                self.reducer_operations, self.aggregator_operations)

    @property
    def has_reducer(self) -> bool:
        return len(self.reducer_operations) > 0

    def digest(self) -> str:
        def norm(o):
            if isinstance(o, dict):
                return {k: norm(v) for k, v in sorted(o.items()) if k != "dtype_data"}
            if isinstance(o, (list, tuple)):
                return [norm(v) for v in o]
            if isinstance(o, NodeRef):
                return o.name
            if isinstance(o, (int, float, str)) or o is None:
                return o
            return str(o)
        blob = json.dumps([norm(x) for x in self.as_tuple()], sort_keys=True)
        return hashlib.sha1(blob.encode()).hexdigest()[:12]


# ----------------------------------------------------------------------------------------------
# small helpers that produce dicts exactly in the tracer's shape
# ----------------------------------------------------------------------------------------------

def dim_of(shape: Sequence[int]) -> int:
    """Flattened per-element width (codegen/utils.py:5-12)."""
    d = 1
    for s in shape:
        d *= int(s)
    return d


def placeholder(name: str, shape: Tuple[int, ...]) -> Dict[str, Any]:
    return {"name": name, "target": name, "dtype": "scalar_t", "shape": tuple(shape),
            "op": "placeholder", "args": (), "dtype_data": None}


def selector_input(name: str, gather_src: str, shape: Tuple[int, ...], module: str | None = None) -> Dict[str, Any]:
    """A Selector module call; ``target`` names the index array (the Selector module: several calls of one
    module share it), args[0] is the gathered tensor."""
    return {"name": name, "target": module or name, "dtype": "int", "shape": tuple(shape),
            "op": "call_module", "args": (NodeRef(gather_src),), "dtype_data": None}


def edge_register(name: str, shape: Tuple[int, ...]) -> Dict[str, Any]:
    return {"name": name, "target": name, "dtype": "TensorT", "selector": 0,
            "selector_name": name, "shape": tuple(shape), "dtype_data": None}


def gather_register(name: str, gather_src: str, shape: Tuple[int, ...], row_identity: bool = False,
                    module: str | None = None) -> Dict[str, Any]:
    d = {"name": name, "target": gather_src, "dtype": "TensorKeyT", "selector": 1,
         "selector_name": module or name, "shape": tuple(shape), "dtype_data": None}
    if row_identity:
        d["row_identity"] = True
    return d


def mop(name: str, op: str, shape: Tuple[int, ...], *args) -> Dict[str, Any]:
    return {"name": name, "target": op, "op": op, "shape": tuple(shape), "dtype_data": None,
            "args": list(args)}


def out(name: str, target: Any, shape: Tuple[int, ...], args=()) -> Dict[str, Any]:
    return {"op": "call_module" if target == "reducer" else "call_function", "name": name,
            "target": target, "dtype": "ValueT", "shape": tuple(shape), "args": args,
            "dtype_data": None}


def _finish(name, inputs, outputs, selreg, mapops, doc="") -> GraphIR:
    reducers = [{k: v for k, v in m.items() if k != "target"} for m in mapops if m["op"] == "reducer"]
    aggs = [{k: v for k, v in m.items() if k != "target"} for m in mapops if m["op"] == "sum"]
    return GraphIR(name, inputs, outputs, selreg, mapops, reducers, aggs, doc)


# ----------------------------------------------------------------------------------------------
# the graphs
# ----------------------------------------------------------------------------------------------

def spmv_graph() -> GraphIR:
    """Plain y = A.x: ``mul(vals, x[col])`` then a dim-1 reducer.
    Operator: merged_spmv_launch(vals, x, selector_idx, row_end_offsets, num_rows, num_cols) -> (y,)"""
    inputs = [placeholder("vals", (1,)), placeholder("x", (1,)), selector_input("selector", "x", (1,))]
    selreg = [edge_register("vals", (1,)), gather_register("selector", "x", (1,))]
    mapops = [mop("mul", "mul", (1,), "vals", "selector"), mop("reducer", "reducer", (1,), "mul")]
    outputs = [out("reducer", "reducer", (1,))]
    return _finish("spmv", inputs, outputs, selreg, mapops, spmv_graph.__doc__)


def spring_mass_graph() -> GraphIR:
    """Spring-mass force: f = k (|d| - L) d/|d| with d = p[dst] - p[src], summed per source vertex.
    Operator: merged_spmv_launch(L, k, p, sel_src_idx, sel_dst_idx, row_end_offsets, N, N) -> (f,)
    ``sel_src`` is the row id of every edge (edges are stored CSR-by-source)."""
    inputs = [placeholder("L", (1,)), placeholder("k", (1,)), placeholder("p", (2,)),
              selector_input("sel_src", "p", (2,)), selector_input("sel_dst", "p", (2,))]
    selreg = [edge_register("L", (1,)), edge_register("k", (1,)),
              gather_register("sel_src", "p", (2,), row_identity=True),
              gather_register("sel_dst", "p", (2,))]
    mapops = [
        mop("d", "sub", (2,), "sel_dst", "sel_src"),
        mop("n", "norm", (1,), "d"),
        mop("s", "sub", (1,), "n", "L"),
        mop("ks", "mul", (1,), "k", "s"),
        mop("kd", "mul", (2,), "ks", "d"),
        mop("f", "truediv", (2,), "kd", "n"),
        mop("red", "reducer", (2,), "f"),
    ]
    outputs = [out("red", "reducer", (2,))]
    return _finish("spring_mass", inputs, outputs, selreg, mapops, spring_mass_graph.__doc__)


def rusanov_graph() -> GraphIR:
    """Shallow-water Rusanov / local Lax-Friedrichs face flux, g = 9.81, summed per cell.
    Per edge (cell i -> neighbour j) with face data (nx, ny, len) and state U = (h, hu, hv):
      un = (hu nx + hv ny)/h ;  F.n = (h un, hu un + g h^2 nx / 2, hv un + g h^2 ny / 2)
      lam = max(|un_i| + sqrt(g h_i), |un_j| + sqrt(g h_j))
      flux = (0.5 (F_i.n + F_j.n) - 0.5 lam (U_j - U_i)) len
    Written only with ops of the reference vocabulary (no sqrt/max: pow 0.5 and where(gt)); the three
    components are three dim-1 reducers because the vocabulary has no concat.
    Operator: merged_spmv_launch(face, U, sel_self_idx, sel_nbr_idx, row_end_offsets, n, n)
              -> (flux_h, flux_hu, flux_hv)"""
    S1 = (1,)
    inputs = [placeholder("face", (3,)), placeholder("U", (3,)),
              selector_input("sel_self", "U", (3,)), selector_input("sel_nbr", "U", (3,))]
    selreg = [edge_register("face", (3,)),
              gather_register("sel_self", "U", (3,), row_identity=True),
              gather_register("sel_nbr", "U", (3,))]
    m: List[Dict[str, Any]] = []

    def op(name, kind, *args):
        m.append(mop(name, kind, S1, *args))
        return name

    nx = op("nx", "getitem", "face", (None, 0))
    ny = op("ny", "getitem", "face", (None, 1))
    ln = op("ln", "getitem", "face", (None, 2))
    side = {}
    for s, sel in (("i", "sel_self"), ("j", "sel_nbr")):
        h = op(f"h{s}", "getitem", sel, (None, 0))
        hu = op(f"hu{s}", "getitem", sel, (None, 1))
        hv = op(f"hv{s}", "getitem", sel, (None, 2))
        a1 = op(f"a1{s}", "mul", hu, nx)
        a2 = op(f"a2{s}", "mul", hv, ny)
        a3 = op(f"a3{s}", "add", a1, a2)
        un = op(f"un{s}", "truediv", a3, h)
        h2 = op(f"h2{s}", "mul", h, h)
        p = op(f"p{s}", "mul", h2, 4.905)
        f0 = op(f"f0{s}", "mul", h, un)
        t1 = op(f"t1{s}", "mul", hu, un)
        t2 = op(f"t2{s}", "mul", p, nx)
        f1 = op(f"f1{s}", "add", t1, t2)
        t3 = op(f"t3{s}", "mul", hv, un)
        t4 = op(f"t4{s}", "mul", p, ny)
        f2 = op(f"f2{s}", "add", t3, t4)
        gh = op(f"gh{s}", "mul", h, 9.81)
        c = op(f"c{s}", "pow", gh, 0.5)
        au = op(f"au{s}", "abs", un)
        sp = op(f"sp{s}", "add", au, c)
        side[s] = dict(h=h, hu=hu, hv=hv, f=(f0, f1, f2), sp=sp)
    g = op("spgt", "gt", side["i"]["sp"], side["j"]["sp"])
    lam = op("lam", "where", g, side["i"]["sp"], side["j"]["sp"])
    hl = op("hl", "mul", lam, 0.5)
    reds = []
    for k, comp in enumerate(("h", "hu", "hv")):
        fs = op(f"fs{k}", "add", side["i"]["f"][k], side["j"]["f"][k])
        fa = op(f"fa{k}", "mul", fs, 0.5)
        du = op(f"du{k}", "sub", side["j"][comp], side["i"][comp])
        ds = op(f"ds{k}", "mul", hl, du)
        fx = op(f"fx{k}", "sub", fa, ds)
        fl = op(f"fl{k}", "mul", fx, ln)
        reds.append(op(f"flux_{comp}", "reducer", fl))
    outputs = [out(r, "reducer", S1) for r in reds]
    return _finish("rusanov", inputs, outputs, selreg, m, rusanov_graph.__doc__)


def swe_delta_graph() -> GraphIR:
    """The interior part of ``ShallowWaterEquation.delta`` of the reference's shallow-water model
    (shallow_water_equation/swe_main.py:86-119): face reconstruction of h, uh, vh from the two cells of
    every edge, ``phi_f = (1 - alpha) phi[src] + alpha phi[dst]``, face velocities ``uh_f / h_f`` and
    ``vh_f / h_f``, and the three ``scatter`` reducers over the destination cell:
      r_h  = sum uh_f sx + vh_f sy
      r_uh = sum (u_f uh_f + h_f^2/2) sx + u_f vh_f sy
      r_vh = sum v_f uh_f sx + (v_f vh_f + h_f^2/2) sy
    as a torch.fx trace of that method lists them: the ``gather_src`` / ``gather_dst`` Selector modules are
    called three times each (on h, uh, vh) and share one index array per module; edges are sorted by
    destination cell, so ``gather_dst`` is the row id.  The boundary reducers (``scatter_b``) and the
    ``-(...)/area`` update are separate, element-wise steps of the model.
    Operator: merged_spmv_launch(alpha, sx, sy, h, uh, vh, gather_src_idx, gather_dst_idx,
                                 row_end_offsets, nc, nc) -> (r_h, r_uh, r_vh)"""
    S1 = (1,)
    inputs = [placeholder("alpha", S1), placeholder("sx", S1), placeholder("sy", S1),
              placeholder("h", S1), placeholder("uh", S1), placeholder("vh", S1)]
    selreg = [edge_register("alpha", S1), edge_register("sx", S1), edge_register("sy", S1)]
    for i, phi in enumerate(("h", "uh", "vh")):
        sfx = "" if i == 0 else f"_{i}"
        inputs.append(selector_input("gather_src" + sfx, phi, S1, module="gather_src"))
        inputs.append(selector_input("gather_dst" + sfx, phi, S1, module="gather_dst"))
        selreg.append(gather_register("gather_src" + sfx, phi, S1, module="gather_src"))
        selreg.append(gather_register("gather_dst" + sfx, phi, S1, row_identity=True, module="gather_dst"))
    m: List[Dict[str, Any]] = []

    def op(name, kind, *args):
        m.append(mop(name, kind, S1, *args))
        return name

    face = {}
    for i, phi in enumerate(("h", "uh", "vh")):
        sfx = "" if i == 0 else f"_{i}"
        oma = op(f"oma_{phi}", "sub", 1.0, "alpha")          # traced once per face_reconstruct call
        a = op(f"a_{phi}", "mul", oma, "gather_src" + sfx)
        b = op(f"b_{phi}", "mul", "alpha", "gather_dst" + sfx)
        face[phi] = op(f"{phi}_f", "add", a, b)
    u_f = op("u_f", "truediv", face["uh"], face["h"])
    v_f = op("v_f", "truediv", face["vh"], face["h"])
    hh = op("hh", "mul", 0.5, face["h"])
    hsq = op("h_f_square", "mul", hh, face["h"])
    uhsx = op("uh_f_times_sx", "mul", face["uh"], "sx")
    vhsy = op("vh_f_times_sy", "mul", face["vh"], "sy")
    s_h = op("s_h", "add", uhsx, vhsy)
    r_h = op("r_h", "reducer", s_h)
    t1 = op("t1", "mul", u_f, face["uh"])
    t2 = op("t2", "add", t1, hsq)
    t3 = op("t3", "mul", t2, "sx")
    t4 = op("t4", "mul", u_f, vhsy)
    s_uh = op("s_uh", "add", t3, t4)
    r_uh = op("r_uh", "reducer", s_uh)
    t5 = op("t5", "mul", v_f, uhsx)
    t6 = op("t6", "mul", v_f, face["vh"])
    t7 = op("t7", "add", t6, hsq)
    t8 = op("t8", "mul", t7, "sy")
    s_vh = op("s_vh", "add", t5, t8)
    r_vh = op("r_vh", "reducer", s_vh)
    outputs = [out(r, "reducer", S1) for r in (r_h, r_uh, r_vh)]
    return _finish("swe_delta", inputs, outputs, selreg, m, swe_delta_graph.__doc__)


def swe_boundary_graph() -> GraphIR:
    """The boundary part of ``ShallowWaterEquation.delta`` (shallow_water_equation/swe_main.py:96-114):
    ``gather_b_h_square = 0.5 * gather_b(h)**2`` scattered with ``scatter_b`` once times ``bsx`` and once
    times ``bsy``.  One "edge" per boundary cell, sorted by cell; ``gather_b`` and ``scatter_b`` use the
    same index (``bcells``), so the selector is the row id.
    Operator: merged_spmv_launch(bsx, bsy, h, gather_b_idx, row_end_offsets, nc, nc) -> (rb_uh, rb_vh)"""
    S1 = (1,)
    inputs = [placeholder("bsx", S1), placeholder("bsy", S1), placeholder("h", S1),
              selector_input("gather_b", "h", S1)]
    selreg = [edge_register("bsx", S1), edge_register("bsy", S1),
              gather_register("gather_b", "h", S1, row_identity=True)]
    m = [
        mop("hb2", "pow", S1, "gather_b", 2),
        mop("gather_b_h_square", "mul", S1, 0.5, "hb2"),
        mop("bx", "mul", S1, "gather_b_h_square", "bsx"),
        mop("rb_uh", "reducer", S1, "bx"),
        mop("by", "mul", S1, "gather_b_h_square", "bsy"),
        mop("rb_vh", "reducer", S1, "by"),
    ]
    outputs = [out("rb_uh", "reducer", S1), out("rb_vh", "reducer", S1)]
    return _finish("swe_boundary", inputs, outputs, selreg, m, swe_boundary_graph.__doc__)


def swe_init_edges_graph() -> GraphIR:
    """The per-edge part of the reference's shallow-water mesh assembler (``ShallowWaterInitializer.forward``,
    shallow_water_equation/assemble_shallow_water.py:178-215): from the vertices of the two triangles of every
    edge (six Selector modules on ``points``) the face vector (sx, sy) of the face the two cells share, as seen from
    the source cell -- the one of the source's three faces whose outward normal points away from the destination's
    centroid side test -- and the interpolation weight ``alpha`` where the centroid line crosses that face, written
    in place into the model's sx / sy / alpha tensors (three rounds of ``where`` + ``setitem``).  Map-only graph:
    no reducer, no allocated output.
    Operator: merged_spmv_launch(sx, sy, alpha, points, src_p0_idx, src_p1_idx, src_p2_idx, dst_p0_idx, dst_p1_idx,
                                 dst_p2_idx, row_end_offsets(dummy), num_rows, num_cols) -> None"""
    S1, S2 = (1,), (2,)
    sels = [f"src_p{i}" for i in range(3)] + [f"dst_p{i}" for i in range(3)]
    inputs = [placeholder("sx", S1), placeholder("sy", S1), placeholder("alpha", S1), placeholder("points", S2)]
    inputs += [selector_input(n, "points", S2) for n in sels]
    selreg = [edge_register("sx", S1), edge_register("sy", S1), edge_register("alpha", S1)]
    selreg += [gather_register(n, "points", S2) for n in sels]
    m: List[Dict[str, Any]] = []
    count = [0]

    def op(kind, shape, *args, name=None):
        count[0] += 1
        nm = name or f"t{count[0]}_{kind}"
        m.append(mop(nm, kind, shape, *args))
        return nm

    def xy(pt):
        return op("getitem", S1, pt, (None, 0)), op("getitem", S1, pt, (None, 1))

    def centroid(a, b, c):
        return op("truediv", S2, op("add", S2, op("add", S2, a, b), c), 3.0)

    def face_norm(p0, p1, p2):      # get_face_norm(p0, p1, p2), :164-176
        a1, a2 = xy(p0)
        b1, b2 = xy(p1)
        c1, c2 = xy(p2)
        bc1, bc2 = op("sub", S1, b1, c1), op("sub", S1, b2, c2)
        ac1, ac2 = op("sub", S1, a1, c1), op("sub", S1, a2, c2)
        sg = op("sign", S1, op("sub", S1, op("mul", S1, bc1, ac2), op("mul", S1, bc2, ac1)))
        return op("mul", S1, sg, bc2), op("mul", S1, op("neg", S1, sg), bc1)

    def get_alpha(sc, dc, p0, p1):  # :141-162
        x1, y1 = xy(sc)
        x2, y2 = xy(dc)
        x3, y3 = xy(p0)
        x4, y4 = xy(p1)
        y21, y43, y31 = op("sub", S1, y2, y1), op("sub", S1, y4, y3), op("sub", S1, y3, y1)
        x31, x21, x43 = op("sub", S1, x3, x1), op("sub", S1, x2, x1), op("sub", S1, x4, x3)
        num = op("sub", S1, op("mul", S1, x31, y43), op("mul", S1, y31, x43))
        den = op("sub", S1, op("mul", S1, x21, y43), op("mul", S1, y21, x43))
        return op("truediv", S1, num, den)

    sp = ["src_p0", "src_p1", "src_p2"]
    src_cent = centroid(*sp)
    dst_cent = centroid("dst_p0", "dst_p1", "dst_p2")
    rounds = [((sp[2], sp[0], sp[1]), (sp[0], sp[1])), ((sp[0], sp[1], sp[2]), (sp[1], sp[2])), ((sp[1], sp[2], sp[0]), (sp[2], sp[0]))]
    normals = [face_norm(*own) for own, _ in rounds]                          # outward normals of the source's faces
    tests = [face_norm(dst_cent, *face) for _, face in rounds]                # the same faces seen from the destination's centroid
    for k, ((own, face), (nx, ny), (tx, ty)) in enumerate(zip(rounds, normals, tests)):
        cond = op("lt", S1, op("add", S1, op("mul", S1, nx, tx), op("mul", S1, ny, ty)), 0.0)
        al = get_alpha(src_cent, dst_cent, *face)
        prev = (0.0, 0.0, 0.0) if k == 0 else ("sx", "sy", "alpha")
        for tgt, val, old in (("sx", nx, prev[0]), ("sy", ny, prev[1]), ("alpha", al, prev[2])):
            w_ = op("where", S1, cond, val, old)
            op("setitem", S1, tgt, (None,), w_)
    return _finish("swe_init_edges", inputs, [], selreg, m, swe_init_edges_graph.__doc__)


def swe_init_cells_graph() -> GraphIR:
    """The per-cell part of the reference's mesh assembler (shallow_water_equation/assemble_shallow_water.py:217-239):
    from the three vertices of every cell (three Selector modules on ``points``) its area
    ``0.5 |x0 (y1 - y2) + x1 (y2 - y0) + x2 (y0 - y1)|``, its centroid (x, y) and the initial water height
    ``h = 1 + 0.1 exp(-100 (x^2 + y^2))``, written in place into the model's tensors (``setitem``).  Map-only graph
    whose "edges" are the cells.
    Operator: merged_spmv_launch(area, x, y, h, points, cells_p0_idx, cells_p1_idx, cells_p2_idx,
                                 row_end_offsets(dummy), num_rows, num_cols) -> None"""
    S1, S2 = (1,), (2,)
    sels = [f"cells_p{i}" for i in range(3)]
    inputs = [placeholder(n, S1) for n in ("area", "x", "y", "h")] + [placeholder("points", S2)]
    inputs += [selector_input(n, "points", S2) for n in sels]
    selreg = [edge_register(n, S1) for n in ("area", "x", "y", "h")] + [gather_register(n, "points", S2) for n in sels]
    m: List[Dict[str, Any]] = []

    def op(name, kind, shape, *args):
        m.append(mop(name, kind, shape, *args))
        return name

    xs, ys = [], []
    for i, sname in enumerate(sels):
        xs.append(op(f"x{i}", "getitem", S1, sname, (None, 0)))
        ys.append(op(f"y{i}", "getitem", S1, sname, (None, 1)))
    t0 = op("t0", "mul", S1, xs[0], op("d12", "sub", S1, ys[1], ys[2]))
    t1 = op("t1", "mul", S1, xs[1], op("d20", "sub", S1, ys[2], ys[0]))
    t2 = op("t2", "mul", S1, xs[2], op("d01", "sub", S1, ys[0], ys[1]))
    twice = op("twice", "add", S1, op("t01", "add", S1, t0, t1), t2)
    area = op("area_v", "mul", S1, 0.5, op("abs_twice", "abs", S1, twice))
    op("set_area", "setitem", S1, "area", (None,), area)
    cent = op("centroid", "truediv", S2, op("p012", "add", S2, op("p01", "add", S2, sels[0], sels[1]), sels[2]), 3.0)
    cx = op("cx", "getitem", S1, cent, (None, 0))
    cy = op("cy", "getitem", S1, cent, (None, 1))
    op("set_x", "setitem", S1, "x", (None,), cx)
    op("set_y", "setitem", S1, "y", (None,), cy)
    # the tracer records the assignments above; the height then reads the tensors just written (self.x, self.y)
    dx2 = op("dx2", "pow", S1, op("dx", "sub", S1, "x", 0.0), 2)
    dy2 = op("dy2", "pow", S1, op("dy", "sub", S1, "y", 0.0), 2)
    ex = op("ex", "exp", S1, op("arg", "mul", S1, -100.0, op("r2", "add", S1, dx2, dy2)))
    hv = op("h_v", "add", S1, 1.0, op("bump", "mul", S1, 0.1, ex))
    op("set_h", "setitem", S1, "h", (None,), hv)
    return _finish("swe_init_cells", inputs, [], selreg, m, swe_init_cells_graph.__doc__)


def swe_init_boundary_graph() -> GraphIR:
    """The boundary part of the reference's mesh assembler (shallow_water_equation/assemble_shallow_water.py:241-248):
    for every boundary face the two end points (Selector modules ``bp0`` / ``bp1`` on ``points``) and the centroid of
    the cell the face belongs to (Selector ``bcells`` on the centroids computed by the per-cell part), giving the face
    vector that points out of the domain, ``(bsx, bsy) = -get_face_norm(centroid, p0, p1)``, written in place
    (``setitem``).  Map-only graph whose "edges" are the boundary faces; two gather sources of different lengths.
    Operator: merged_spmv_launch(bsx, bsy, points, centroid, bp0_idx, bp1_idx, bcells_idx,
                                 row_end_offsets(dummy), num_rows, num_cols) -> None"""
    S1, S2 = (1,), (2,)
    inputs = [placeholder("bsx", S1), placeholder("bsy", S1), placeholder("points", S2), placeholder("centroid", S2),
              selector_input("bp0", "points", S2), selector_input("bp1", "points", S2),
              selector_input("bcells", "centroid", S2)]
    selreg = [edge_register("bsx", S1), edge_register("bsy", S1), gather_register("bp0", "points", S2),
              gather_register("bp1", "points", S2), gather_register("bcells", "centroid", S2)]
    m: List[Dict[str, Any]] = []

    def op(name, kind, shape, *args):
        m.append(mop(name, kind, shape, *args))
        return name

    # get_face_norm(p0 = centroid, p1 = b_p0, p2 = b_p1), :164-176
    a1, a2 = op("a1", "getitem", S1, "bcells", (None, 0)), op("a2", "getitem", S1, "bcells", (None, 1))
    b1, b2 = op("b1", "getitem", S1, "bp0", (None, 0)), op("b2", "getitem", S1, "bp0", (None, 1))
    c1, c2 = op("c1", "getitem", S1, "bp1", (None, 0)), op("c2", "getitem", S1, "bp1", (None, 1))
    bc1, bc2 = op("bc1", "sub", S1, b1, c1), op("bc2", "sub", S1, b2, c2)
    ac1, ac2 = op("ac1", "sub", S1, a1, c1), op("ac2", "sub", S1, a2, c2)
    sg = op("sg", "sign", S1, op("cross", "sub", S1, op("m0", "mul", S1, bc1, ac2), op("m1", "mul", S1, bc2, ac1)))
    nx = op("nx", "mul", S1, sg, bc2)
    ny = op("ny", "mul", S1, op("nsg", "neg", S1, sg), bc1)
    op("set_bsx", "setitem", S1, "bsx", (None,), op("neg_nx", "neg", S1, nx))
    op("set_bsy", "setitem", S1, "bsy", (None,), op("neg_ny", "neg", S1, ny))
    return _finish("swe_init_boundary", inputs, [], selreg, m, swe_init_boundary_graph.__doc__)


def swe_components_graph() -> GraphIR:
    """The gathering part of the reference's mesh-components collector (``ShallowWaterMeshComponentsCollector.forward``,
    shallow_water_equation/assemble_shallow_water.py:62-72): for every edge the three vertex ids of its source cell and
    of its destination cell (two Selector modules on the (nc, 3) ``cells`` tensor), column by column into six
    per-edge tensors (``getitem`` / ``clone`` / ``copy_``).  Integer map-only graph; the per-cell and per-boundary
    columns the same module copies (:74-78) are slices of its inputs and need no gather.
    Operator: merged_spmv_launch(src_p0, src_p1, src_p2, dst_p0, dst_p1, dst_p2, cells, src_idx, dst_idx,
                                 row_end_offsets(dummy), num_rows, num_cols) -> None"""
    S1, S3 = (1,), (3,)
    outs = [f"src_p{i}" for i in range(3)] + [f"dst_p{i}" for i in range(3)]
    inputs = [placeholder(n, S1) for n in outs] + [placeholder("cells", S3)]
    inputs += [selector_input("selector_src", "cells", S3), selector_input("selector_dst", "cells", S3)]
    selreg = [edge_register(n, S1) for n in outs]
    selreg += [gather_register("selector_src", "cells", S3), gather_register("selector_dst", "cells", S3)]
    m: List[Dict[str, Any]] = []
    for i in range(3):
        for side in ("src", "dst"):
            m.append(mop(f"{side}_col{i}", "getitem", S1, f"selector_{side}", (None, i)))
            m.append(mop(f"{side}_clone{i}", "clone", S1, f"{side}_col{i}"))
            m.append(mop(f"{side}_copy{i}", "copy_", S1, f"{side}_p{i}", f"{side}_clone{i}"))
    return _finish("swe_components", inputs, [], selreg, m, swe_components_graph.__doc__)


def mixed_dims_graph() -> GraphIR:
    """Unit-test graph shaped like the reference's demo model (easier_spmv.py:17-69, generated
    instance include/merged_agent_spmv.cuh:124-149): two selectors on one dim-2 vertex tensor, edge
    tensors of dim 2 and 6, modulo broadcasting 2 -> 6, a dim-2 and a dim-6 reducer, one per-edge
    map output.  Exercises empty rows, multi-reducer accumulation and mixed widths."""
    inputs = [placeholder("ea", (2,)), placeholder("eb", (6,)), placeholder("vx", (2,)),
              selector_input("s0", "vx", (2,)), selector_input("s1", "vx", (2,))]
    selreg = [edge_register("ea", (2,)), edge_register("eb", (6,)),
              gather_register("s0", "vx", (2,)), gather_register("s1", "vx", (2,))]
    m = [
        mop("t0", "add", (2,), "s0", "s1"),
        mop("t1", "mul", (2,), "t0", "ea"),
        mop("t2", "mul", (6,), "eb", "t1"),          # 6 x 2 modulo broadcast
        mop("t3", "sub", (6,), "t2", 0.25),
        mop("t4", "neg", (2,), "t1"),
        mop("r2", "reducer", (2,), "t4"),
        mop("r6", "reducer", (6,), "t3"),
    ]
    outputs = [out("r2", "reducer", (2,)), out("r6", "reducer", (6,)), out("t1", "mul", (2,))]
    return _finish("mixed_dims", inputs, outputs, selreg, m, mixed_dims_graph.__doc__)


def ops_zoo_graph() -> GraphIR:
    """Unit-test graph touching the rest of the map vocabulary (trace/graph_trace.py:229-276):
    truediv with a zero divisor (guarded: result 0, data_struct_shared.cuh:194-200), scalar / tensor,
    pow, exp, abs, sign, lt, gt, where, getitem, clone, norm."""
    inputs = [placeholder("w", (2,)), placeholder("v", (2,)), selector_input("sel", "v", (2,))]
    selreg = [edge_register("w", (2,)), gather_register("sel", "v", (2,))]
    m = [
        mop("q", "truediv", (2,), "w", "sel"),       # same dims: guarded divide
        mop("iq", "truediv", (2,), 1.5, "sel"),      # scalar / tensor: guarded
        mop("aw", "abs", (2,), "w"),
        mop("pw", "pow", (2,), "aw", 1.5),
        mop("sw", "mul", (2,), "w", -0.125),
        mop("ex", "exp", (2,), "sw"),
        mop("sg", "sign", (2,), "w"),
        mop("lt0", "lt", (2,), "w", 0.25),
        mop("g0", "gt", (2,), "sel", "w"),
        mop("wh", "where", (2,), "lt0", "pw", "ex"),
        mop("w0", "getitem", (1,), "w", (None, 0)),
        mop("cl", "clone", (2,), "sg"),
        mop("nn", "norm", (1,), "sel"),
        mop("a0", "add", (2,), "q", "iq"),
        mop("a1", "add", (2,), "a0", "wh"),
        mop("a2", "mul", (2,), "a1", "w0"),          # 2 x 1 broadcast
        mop("a3", "add", (2,), "a2", "cl"),
        mop("a4", "add", (2,), "a3", "g0"),
        mop("a5", "truediv", (2,), "a4", "nn"),      # tensor / scalar: unguarded
        mop("red", "reducer", (2,), "a5"),
    ]
    outputs = [out("red", "reducer", (2,))]
    return _finish("ops_zoo", inputs, outputs, selreg, m, ops_zoo_graph.__doc__)


def edge_sum_graph() -> GraphIR:
    """Aggregator flavour (no reducer, cuda_template/aggregator/*): per-edge product stored as a map
    output plus a global ``sum`` of it.  Operator:
    merged_spmv_launch(ew, vx, sel_idx, row_end_offsets(dummy), num_rows, num_cols) -> (prod, total)"""
    inputs = [placeholder("ew", (2,)), placeholder("vx", (2,)), selector_input("sel", "vx", (2,))]
    selreg = [edge_register("ew", (2,)), gather_register("sel", "vx", (2,))]
    m = [mop("prod", "mul", (2,), "ew", "sel"), mop("total", "sum", (2,), "prod")]
    outputs = [out("prod", "mul", (2,)), out("total", "sum", (2,))]
    return _finish("edge_sum", inputs, outputs, selreg, m, edge_sum_graph.__doc__)


def edge_copy_graph() -> GraphIR:
    """Map-only flavour with in-place writes, the shape of the reference's checked-in CPU instance
    (merged_spmv.h:92-151: getitem / clone / copy_ on boundary points): gathers a vertex tensor and
    writes it through an input pointer (copy_), no allocated output.  Valid for integer ValueT."""
    inputs = [placeholder("dst", (2,)), placeholder("src", (2,)), selector_input("sel", "src", (2,))]
    selreg = [edge_register("dst", (2,)), gather_register("sel", "src", (2,))]
    m = [mop("c", "clone", (2,), "sel"), mop("cp", "copy_", (2,), "dst", "c")]
    return _finish("edge_copy", inputs, [], selreg, m, edge_copy_graph.__doc__)


ALL_GRAPHS = {
    "spmv": spmv_graph,
    "spring_mass": spring_mass_graph,
    "rusanov": rusanov_graph,
    "swe_delta": swe_delta_graph,
    "swe_boundary": swe_boundary_graph,
    "swe_components": swe_components_graph,
    "swe_init_edges": swe_init_edges_graph,
    "swe_init_cells": swe_init_cells_graph,
    "swe_init_boundary": swe_init_boundary_graph,
    "mixed_dims": mixed_dims_graph,
    "ops_zoo": ops_zoo_graph,
    "edge_sum": edge_sum_graph,
    "edge_copy": edge_copy_graph,
}

# value types each graph is compiled for (one C-ABI symbol per pair)
GRAPH_DTYPES = {
    "spmv": ("float32", "float64", "int64"),
    "spring_mass": ("float32", "float64"),
    "rusanov": ("float64", "float32"),
    "swe_delta": ("float64", "float32"),
    "swe_boundary": ("float64", "float32"),
    "swe_components": ("int64",),
    "swe_init_edges": ("float64",),
    "swe_init_cells": ("float64",),
    "swe_init_boundary": ("float64",),
    "mixed_dims": ("float32", "float64", "int64"),
    "ops_zoo": ("float32", "float64"),
    "edge_sum": ("float32", "float64", "int64"),
    "edge_copy": ("float32", "float64", "int64"),
}


def operator_signature(ir: GraphIR):
    """Positional argument order of the operator, as the reference's binding generator derives it
    (codegen/merged_gen_binding.py:27-78): non-gather value inputs, gather value inputs (first-use
    order, de-duplicated), one index tensor per distinct selector target, then row_end_offsets,
    num_rows, num_cols.  Returns (value_names, gather_names, index_names)."""
    gather_targets = {s["target"] for s in ir.selector_register if s.get("selector") == 1}
    value_inputs = [i for i in ir.inputs if i["dtype"] != "int"]
    seen, sel_inputs = set(), []
    for i in ir.inputs:
        if i["dtype"] == "int" and i["target"] not in seen:
            sel_inputs.append(i)
            seen.add(i["target"])
    non_gather = [i["name"] for i in value_inputs if i["name"] not in gather_targets]
    gathers, seen_g = [], set()
    for i in ir.inputs:
        if i["op"] == "call_module" and i["args"][0].name in gather_targets and i["args"][0].name not in seen_g:
            gathers.append(i["args"][0].name)
            seen_g.add(i["args"][0].name)
    return non_gather, gathers, [s["target"] for s in sel_inputs]
