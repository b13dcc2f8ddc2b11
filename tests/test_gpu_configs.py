"""The five benchmark configurations on the GPU: against the CPU oracle at sizes the oracle finishes in
seconds (identical numpy inputs on both sides), against the committed golden fixtures, and at full
size through size-independent properties (checksum against an independent torch reduction, linearity,
agreement with torch's own CSR product, run-to-run determinism)."""
import os

import numpy as np
import pytest
import torch

from flexspmv_b200 import graphs, multi_gpu, problems
from flexspmv_b200.binding import GraphExtension
from golden_io import golden_files, load
from oracle import ir_eval
from parity import TOL, assert_outputs_match, row_error
from test_gpu_parity import run_gpu

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,make", [
    ("config0 poisson2d 128", lambda: ("spmv", problems.poisson2d(128))),
    ("config0 poisson2d 512 (full size)", lambda: ("spmv", problems.poisson2d(512))),
    ("config1 spring-mass 160", lambda: ("spring_mass", problems.spring_mass(160))),
    ("config1 spring-mass 1024 (full size)", lambda: ("spring_mass", problems.spring_mass(1024))),
    ("config2 shallow-water 1024 (full size)", lambda: ("rusanov", problems.shallow_water(1024))),
    ("config2 shallow-water 96", lambda: ("rusanov", problems.shallow_water(96))),
    ("reference shallow-water model, fused delta graph, mesh 96", lambda: ("swe_delta", problems.swe_mesh(96))),
    ("config3 power-law 2^16", lambda: ("spmv", problems.powerlaw(1 << 16, cap=20000))),
    ("config4 poisson3d 40, int64 offsets", lambda: ("spmv", problems.poisson3d(40))),
], ids=lambda v: v if isinstance(v, str) else "")
def test_config_matches_oracle(name, make):
    gname, prob = make()
    ir = graphs.ALL_GRAPHS[gname]()
    dt = next(iter(prob.values.values())).dtype
    ref, _, sums = ir_eval.run_graph(ir, prob, dt, num_threads=8, want_abs_sums=True)
    got, _ = run_gpu(GraphExtension(ir), ir, prob, dt)
    assert_outputs_match(ir, got, ref, sums, dt, what=name)


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: os.path.basename(p)[:-4])
def test_gpu_matches_golden_fixture(path):
    """The fixtures were produced by the reference's own generated CPU operator."""
    prob, dt, threads, outs, written = load(path)
    ir = graphs.ALL_GRAPHS[prob.graph]()
    _, _, sums = ir_eval.run_graph(ir, prob, dt, num_threads=threads, want_abs_sums=True)
    got, got_written = run_gpu(GraphExtension(ir), ir, prob, dt)
    assert_outputs_match(ir, got, outs, sums, dt, what=os.path.basename(path))
    for k, r in written.items():
        g = got_written[k].reshape(r.shape)
        if prob.graph == "swe_init_cells":           # exp / pow: the CPU's math library against CUDA's
            assert np.allclose(g, r, rtol=1e-13, atol=0), f"in-place input {k}"
        elif np.dtype(dt).kind == "i" or prob.graph != "ops_zoo":
            assert np.array_equal(g, r), f"in-place input {k}"


def _spmv(ext, vals, x, cols, ro, n):
    y = torch.empty(n, dtype=vals.dtype, device=vals.device)
    ext.launch_into([vals, x], [cols], ro, [y], n, cols.numel(), x.numel())
    return y


def test_config3_full_size_properties():
    """16.8 M rows, ~260 M non-zeros, rows up to 100 000 long, built on the device."""
    dev = torch.device("cuda:0")
    ro, cols, vals, x = problems.powerlaw_device(1 << 24, 3, dev)
    n = x.numel()
    ext = GraphExtension(graphs.spmv_graph())
    y = _spmv(ext, vals, x, cols, ro, n)
    # checksum of checksums: sum(y) == sum over edges of val * x[col] (independent fp64 reduction)
    terms = vals.double() * x[cols.long()].double()
    assert abs(float(y.double().sum()) - float(terms.sum())) <= 1e-5 * float(terms.abs().sum())
    # per-row agreement with torch's CSR product on the same device arrays
    A = torch.sparse_csr_tensor(ro.long(), cols.long(), vals.double(), size=(n, n))
    y_ref = (A @ x.double().unsqueeze(1)).squeeze(1)
    rid = torch.repeat_interleave(torch.arange(n, device=dev), (ro[1:] - ro[:-1]).long())
    abs_sum = torch.zeros(n, dtype=torch.float64, device=dev).index_add_(0, rid, terms.abs())
    err = ((y.double() - y_ref).abs() / abs_sum.clamp_min(1e-300)).max()
    assert float(err) <= TOL[np.dtype(np.float32)]
    # the reference's own generated CPU operator on the same full-size arrays (rows of up to 100 000 edges included)
    from oracle import ref_run
    if ref_run.available("spmv"):
        prob = problems.Problem("spmv", {"vals": vals.cpu().numpy(), "x": x.cpu().numpy()}, {"selector": cols.cpu().numpy()},
                                ro.cpu().numpy(), n, n, {"config": 3})
        call = ref_run.PreparedCall(graphs.spmv_graph(), prob, np.float32, num_threads=min(os.cpu_count() or 8, 64), copy_inputs=False)
        (y_cpu,) = call.run()
        assert row_error(y.cpu().numpy(), y_cpu, abs_sum.cpu().numpy()) <= TOL[np.dtype(np.float32)]
        del prob, call, y_cpu
    # linearity: A(2x) == 2 A x exactly in binary floating point, and determinism
    y2 = _spmv(ext, vals, x * 2.0, cols, ro, n)
    assert torch.equal(y2, y * 2.0)
    assert torch.equal(_spmv(ext, vals, x, cols, ro, n), y)


def test_config4_slab_properties_int64_offsets():
    """A 512 x 512 x 24 slab of the 512^3 problem (same plane size and row structure), int64 offsets,
    built on the device exactly as the benchmark builds each rank's block."""
    dev = torch.device("cuda:0")
    n, planes = 512, 24
    ro, cols, vals = multi_gpu.poisson3d_planes_device(n, 1, 1 + planes, dev, col_shift=0)
    rows = planes * n * n
    x = torch.rand((planes + 2) * n * n, dtype=torch.float64, device=dev) * 2 - 1
    ext = GraphExtension(graphs.spmv_graph())
    y = _spmv(ext, vals, x, cols, ro, rows)
    # the 7-point stencil applied with torch slicing on the (z, y, x) grid
    X = x.view(planes + 2, n, n)
    C = X[1:-1]
    ref = 6.0 * C - X[:-2] - X[2:]
    ref[:, 1:, :] -= C[:, :-1, :]
    ref[:, :-1, :] -= C[:, 1:, :]
    ref[:, :, 1:] -= C[:, :, :-1]
    ref[:, :, :-1] -= C[:, :, 1:]
    err = (y.view(planes, n, n) - ref).abs().max() / 12.0      # sum |terms| <= 12 for |x| <= 1
    assert float(err) <= 1e-12
    ones = torch.ones_like(x)
    y1 = _spmv(ext, vals, ones, cols, ro, rows)                 # row sums of the Laplacian: 0 inside, >0 on faces
    assert float(y1.view(planes, n, n)[:, 1:-1, 1:-1].abs().max()) == 0.0
    assert torch.equal(_spmv(ext, vals, x, cols, ro, rows), y)


def test_operator_reuses_and_invalidates_its_plan():
    """The shim caches the partition per row-offset tensor; a different matrix of the same size must not
    be served from the old plan."""
    ir = graphs.spmv_graph()
    ext = GraphExtension(ir)
    a = problems.random_problem(ir, 3000, 3000, 50000, seed=1, dtype=np.float64)
    b = problems.random_problem(ir, 3000, 3000, 50000, seed=2, dtype=np.float64)
    for prob in (a, b, a):
        ref, _, sums = ir_eval.run_graph(ir, prob, np.float64, num_threads=8, want_abs_sums=True)
        got, _ = run_gpu(ext, ir, prob, np.float64)
        assert row_error(got[0], ref[0], sums[0]) <= 1e-12
    # in-place edit of the same offsets tensor bumps its version and forces a re-plan
    dev = torch.device("cuda:0")
    ro = torch.from_numpy(a.row_offsets).to(dev)
    vals = torch.from_numpy(a.values["vals"]).to(dev)
    x = torch.from_numpy(a.values["x"]).to(dev)
    cols = torch.from_numpy(a.indices["selector"]).to(dev)
    (y0,) = ext.merged_spmv_launch(vals, x, cols, ro, a.num_rows, a.num_cols)
    ro.copy_(torch.from_numpy(b.row_offsets).to(dev))
    (y1,) = ext.merged_spmv_launch(torch.from_numpy(b.values["vals"]).to(dev), torch.from_numpy(b.values["x"]).to(dev),
                                   torch.from_numpy(b.indices["selector"]).to(dev), ro, b.num_rows, b.num_cols)
    refb, _, sumsb = ir_eval.run_graph(ir, b, np.float64, num_threads=8, want_abs_sums=True)
    assert row_error(y1.cpu().numpy(), refb[0], sumsb[0]) <= 1e-12


def test_prepared_launch_matches_operator_and_orders_after_its_plan():
    """`prepare` binds tensors once; its launches must equal the operator's result, also when the first
    launch happens on a stream other than the one the plan ran on."""
    ir = graphs.spmv_graph()
    ext = GraphExtension(ir)
    prob = problems.random_problem(ir, 20000, 20000, 300000, seed=21, dtype=np.float64)
    dev = torch.device("cuda:0")
    vals = torch.from_numpy(prob.values["vals"]).to(dev)
    x = torch.from_numpy(prob.values["x"]).to(dev)
    cols = torch.from_numpy(prob.indices["selector"]).to(dev)
    ro = torch.from_numpy(prob.row_offsets).to(dev)
    (want,) = ext.merged_spmv_launch(vals, x, cols, ro, prob.num_rows, prob.num_cols)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        y = torch.full((prob.num_rows,), float("nan"), dtype=torch.float64, device=dev)
    side.synchronize()
    other = GraphExtension(ir)                       # fresh plan cache: prepare() plans on the default stream
    prepared = other.prepare([vals, x], [cols], ro, [y], prob.num_rows, prob.nnz, prob.num_cols)
    with torch.cuda.stream(side):
        prepared.launch()
        prepared.launch()
    side.synchronize()
    assert torch.equal(y, want)
    x.mul_(2.0)                                      # tensors may be rewritten in place between launches
    prepared.launch()
    torch.cuda.synchronize()
    assert torch.equal(y, want * 2.0)


def test_shallow_water_model_step_matches_model_oracle():
    """Three Runge-Kutta steps of the reference's shallow-water model on the fused operators (eager, then
    the same from a captured CUDA graph) against the numpy restatement of the model."""
    from flexspmv_b200.shallow_water import ShallowWaterStep
    from oracle import swe_model
    dev = torch.device("cuda:0")
    m = problems.swe_model_inputs(48)
    h, uh, vh = m["h"], m["uh"], m["vh"]
    for _ in range(3):
        h, uh, vh = swe_model.forward(m, h, uh, vh, dt=0.005)
    for use_graph in (False, True):
        mesh = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in m.items() if k != "row_offsets"}
        step = ShallowWaterStep(mesh, dt=0.005)
        if use_graph:
            step.capture()
        for _ in range(3):
            step.replay() if use_graph else step.forward()
        torch.cuda.synchronize()
        for name, want in (("h", h), ("uh", uh), ("vh", vh)):
            got = mesh[name].cpu().numpy()
            scale = max(float(np.abs(want).max()), 1e-300)
            assert float(np.abs(got - want).max()) <= 1e-12 * scale, (name, use_graph)


def test_mesh_assembler_edge_graph_reproduces_the_model_mesh():
    """The per-edge part of the reference's mesh assembler as a fused map-only graph (graphs.swe_init_edges_graph):
    bit-identical to the CPU oracle, and equal to the closed-form face vectors / weights of the synthetic mesh the
    model tests use."""
    ir = graphs.swe_init_edges_graph()
    prob = problems.swe_init_mesh(96)
    _, want, _ = ir_eval.run_graph(ir, prob, np.float64, num_threads=8, want_abs_sums=True)
    outs, written = run_gpu(GraphExtension(ir), ir, prob, np.float64)
    assert outs == []
    mesh = problems.swe_mesh(96)
    for k in ("sx", "sy", "alpha"):
        assert np.array_equal(written[k].reshape(-1), want[k].reshape(-1)), k
    assert np.abs(written["sx"].reshape(-1) - mesh.values["sx"]).max() <= 1e-15
    assert np.abs(written["sy"].reshape(-1) - mesh.values["sy"]).max() <= 1e-15
    assert np.abs(written["alpha"].reshape(-1) - 0.5).max() <= 1e-12


def test_mesh_assembler_boundary_graph_reproduces_the_model_boundary():
    """The boundary part of the reference's mesh assembler (graphs.swe_init_boundary_graph; two gather sources of
    different lengths): bit-identical to the CPU oracle, and its face vectors, summed per boundary cell, are the
    bsx / bsy the model tests use."""
    ir = graphs.swe_init_boundary_graph()
    prob = problems.swe_init_boundary_mesh(96)
    _, want, _ = ir_eval.run_graph(ir, prob, np.float64, num_threads=8, want_abs_sums=True)
    outs, written = run_gpu(GraphExtension(ir), ir, prob, np.float64)
    assert outs == []
    for k in ("bsx", "bsy"):
        assert np.array_equal(written[k].reshape(-1), want[k].reshape(-1)), k
    m = problems.swe_model_inputs(96)
    cells = 2 * 96 * 96
    for k in ("bsx", "bsy"):
        per_cell = np.bincount(prob.indices["bcells"], weights=written[k].reshape(-1), minlength=cells)
        assert np.abs(per_cell[m["bcells"]] - m[k]).max() <= 1e-15, k
    assert np.array_equal(np.unique(prob.indices["bcells"]), m["bcells"])


def test_mesh_assembler_end_to_end_feeds_the_model():
    """The reference's whole ``assemble_shallow_water`` flow (components collector + initializer) as four launches
    (flexspmv_b200.shallow_water.assemble_shallow_water) from the raw mesh arrays: every saved data set equals the
    synthetic mesh the model tests use, and three model steps from the assembled mesh match the model oracle."""
    from flexspmv_b200.shallow_water import ShallowWaterStep, assemble_shallow_water
    from oracle import swe_model
    dev = torch.device("cuda:0")
    n = 48
    raw = problems.swe_raw_mesh(n)
    sw = assemble_shallow_water({k: torch.from_numpy(v).to(dev) for k, v in raw.items()})
    torch.cuda.synchronize()
    edges, cellsp, bnd = problems.swe_init_mesh(n), problems.swe_init_cells_mesh(n), problems.swe_init_boundary_mesh(n)
    for k, v in list(edges.indices.items()) + list(cellsp.indices.items()) + [(k, bnd.indices[k]) for k in ("bp0", "bp1")]:
        assert np.array_equal(sw[k].cpu().numpy(), v.astype(np.int64)), k
    m = problems.swe_model_inputs(n)
    for k, tol in (("sx", 1e-15), ("sy", 1e-15), ("area", 1e-15), ("alpha", 1e-12)):   # alpha is a quotient of differences
        assert np.abs(sw[k].cpu().numpy() - m[k]).max() <= tol, k
    hs = 1.0 / n
    assert np.abs(sw["x"].cpu().numpy()[0::2] - (np.arange(n * n) % n + 2.0 / 3.0) * hs).max() <= 1e-15
    # the model on the assembled mesh: one boundary record per wall face (a corner cell twice), momentum as in the model tests
    host = {k: v.cpu().numpy() for k, v in sw.items()}
    mm = {"src": raw["src"].astype(np.int32), "dst": raw["dst"].astype(np.int32), "bcells": raw["bcells"].astype(np.int32),
          "uh": m["uh"], "vh": m["vh"]}
    mm.update({k: host[k] for k in ("alpha", "sx", "sy", "bsx", "bsy", "area", "h")})
    h, uh, vh = mm["h"], mm["uh"], mm["vh"]
    for _ in range(3):
        h, uh, vh = swe_model.forward(mm, h, uh, vh, dt=0.005)
    mesh = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in mm.items()}
    step = ShallowWaterStep(mesh, dt=0.005)
    for _ in range(3):
        step.forward()
    torch.cuda.synchronize()
    for name, want in (("h", h), ("uh", uh), ("vh", vh)):
        got = mesh[name].cpu().numpy()
        assert float(np.abs(got - want).max()) <= 1e-12 * max(float(np.abs(want).max()), 1e-300), name


def test_more_than_two_to_the_31_nonzeros():
    """A 688^3 7-point Laplacian has 2.27e9 non-zeros: edge positions no longer fit 32 bits (the reference's
    OffsetT is int only).  Checked against the stencil applied with torch slicing."""
    dev = torch.device("cuda:0")
    if torch.cuda.get_device_properties(dev).total_memory < 120 * 2 ** 30:
        pytest.skip("needs a 180 GB device")
    n = 688
    ro, cols, vals = multi_gpu.poisson3d_planes_device(n, 0, n, dev)
    assert int(ro[-1]) > 2 ** 31 and ro.dtype == torch.int64
    rows = n ** 3
    x = torch.rand(rows, dtype=torch.float64, device=dev) * 2 - 1
    ext = GraphExtension(graphs.spmv_graph())
    y = _spmv(ext, vals, x, cols, ro, rows)
    del vals, cols, ro
    X = x.view(n, n, n)
    ref = 6.0 * X
    ref[1:] -= X[:-1]
    ref[:-1] -= X[1:]
    ref[:, 1:] -= X[:, :-1]
    ref[:, :-1] -= X[:, 1:]
    ref[:, :, 1:] -= X[:, :, :-1]
    ref[:, :, :-1] -= X[:, :, 1:]
    err = float((y.view(n, n, n) - ref).abs().max()) / 12.0
    assert err <= 1e-12
    assert ext.device_status(torch.float64) == 0
    del x, y, ref, X
    torch.cuda.empty_cache()
