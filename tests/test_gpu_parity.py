"""GPU parity: the CUDA path, called through the operator shim and the C ABI, against the CPU oracle
on identical seeded inputs.  Shapes follow the reference's self-checking harnesses
(src/flex_spmv_full_red.cu:391-427,624-635; main.cpp:413-415): sorted random cut points so empty rows
and rows spanning many tiles both occur, dims 1/2/6 mixed in one graph, exact equality for int64."""
import ctypes

import numpy as np
import pytest
import torch

from flexspmv_b200 import graphs, problems
from flexspmv_b200.binding import Desc, GraphExtension, load_library
from oracle import ir_eval
from parity import assert_outputs_match

pytestmark = pytest.mark.gpu

NP2T = {np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64, np.dtype(np.int64): torch.int64}


def run_gpu(ext: GraphExtension, ir, prob, dtype, offsets_dtype=None):
    dev = torch.device("cuda:0")
    non_gather, gathers, index_names = graphs.operator_signature(ir)
    vals = [torch.from_numpy(np.ascontiguousarray(prob.values[n].astype(dtype))).to(dev) for n in non_gather + gathers]
    idxs = [torch.from_numpy(np.ascontiguousarray(prob.indices[n])).to(dev) for n in index_names]
    if prob.row_offsets is not None:
        ro = prob.row_offsets.astype(offsets_dtype) if offsets_dtype is not None else prob.row_offsets
        ro_t = torch.from_numpy(np.ascontiguousarray(ro)).to(dev)
    else:
        ro_t = torch.tensor([42], dtype=torch.int32, device=dev)
    outs = ext.merged_spmv_launch(*vals, *idxs, ro_t, prob.num_rows, prob.num_cols)
    torch.cuda.synchronize()
    outs = [] if outs is None else [o.cpu().numpy() for o in outs]
    written = {n: v.cpu().numpy() for n, v in zip(non_gather + gathers, vals)}
    return outs, written


SHAPES = [
    # rows, vertices, nnz
    (1, 1, 1),
    (37, 37, 211),
    (500, 500, 40),          # mostly empty rows
    (3, 3, 5000),            # rows spanning several tiles
    (1543, 1543, 12313),
    (12314, 12314, 123134),  # the reference harness' default shape
    (9000, 9000, 0x3ffff),
]

CASES = [(g, dt) for g in graphs.ALL_GRAPHS for dt in graphs.GRAPH_DTYPES[g]]
LIBM_GRAPHS = {"swe_init_cells"}      # graphs whose in-place results pass through pow / exp


@pytest.mark.parametrize("gname,dt", CASES)
def test_graph_matches_oracle(gname, dt):
    ir = graphs.ALL_GRAPHS[gname]()
    ext = GraphExtension(ir)
    dtype = np.dtype(dt)
    for (nr, nv, nnz) in SHAPES:
        prob = problems.random_problem(ir, nr, nv, nnz, seed=1000 + nr + nnz, dtype=dtype)
        ref, ref_written, sums = ir_eval.run_graph(ir, prob, dtype, num_threads=8, want_abs_sums=True)
        got, got_written = run_gpu(ext, ir, prob, dtype)
        assert_outputs_match(ir, got, ref, sums, dtype, what=f"{gname}/{dt}/{nr}x{nnz}")
        for name, arr in ref_written.items():     # in-place map ops write through input pointers
            g = got_written[name].reshape(arr.shape)
            if gname in LIBM_GRAPHS:               # pow / exp come from two different math libraries
                assert np.allclose(g, arr, rtol=1e-5 if dtype == np.float32 else 1e-13, atol=0, equal_nan=True), f"{gname}: in-place input {name}"
            else:
                assert np.array_equal(g, arr), f"{gname}: in-place input {name} differs"


@pytest.mark.parametrize("tile_items", [1, 7, 320, 896, 1000])
def test_small_tiles_and_few_ctas(tile_items):
    """Odd tile sizes (incl. the reference's 320 / 896) and a grid of 3 CTAs force long carry chains
    across tiles and across CTAs."""
    ir = graphs.spmv_graph()
    for dt in ("float64", "int64"):
        dtype = np.dtype(dt)
        probe = GraphExtension(ir)
        cap = probe.symbols(NP2T[dtype]).graph_info.default_tile_items      # a tile cannot exceed the compiled carve-up
        ext = GraphExtension(ir, tile_items=min(tile_items, cap), max_ctas=3)
        nnz = 2000 if tile_items < 10 else 60000
        prob = problems.random_problem(ir, 97, 97, nnz, seed=5, dtype=dtype)
        ref, _, sums = ir_eval.run_graph(ir, prob, dtype, num_threads=4, want_abs_sums=True)
        got, _ = run_gpu(ext, ir, prob, dtype)
        assert_outputs_match(ir, got, ref, sums, dtype, what=f"tile {tile_items}")


def test_int64_row_offsets_match_int32():
    ir = graphs.spmv_graph()
    ext = GraphExtension(ir)
    prob = problems.random_problem(ir, 4000, 4000, 70000, seed=11, dtype=np.float64)
    a, _ = run_gpu(ext, ir, prob, np.float64)
    b, _ = run_gpu(ext, ir, prob, np.float64, offsets_dtype=np.int64)
    assert np.array_equal(a[0], b[0])


def test_run_to_run_deterministic():
    ir = graphs.spmv_graph()
    ext = GraphExtension(ir)
    prob = problems.random_problem(ir, 5000, 5000, 400000, seed=3, dtype=np.float32)
    a, _ = run_gpu(ext, ir, prob, np.float32)
    for _ in range(3):
        b, _ = run_gpu(ext, ir, prob, np.float32)
        assert np.array_equal(a[0], b[0])


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("tile_items", [320, 896, 1792, 5])
def test_partition_coordinates_bit_exact(bits, tile_items):
    lib = load_library()
    rng = np.random.default_rng(9)
    for (nr, nnz) in [(1, 0), (0, 0), (12314, 123134), (50, 100000), (100000, 50)]:
        ro = problems.random_cut_csr(nr, nnz, rng).astype(np.int32 if bits == 32 else np.int64)
        ref = ir_eval.tile_coordinates(ro, tile_items)
        ro_t = torch.from_numpy(ro).cuda()
        nbytes = ctypes.c_size_t()
        assert lib.flexspmv_partition_bytes(ctypes.c_int64(nr), ctypes.c_int64(nnz), bits, tile_items, ctypes.byref(nbytes)) == 0
        out = torch.empty(nbytes.value // (bits // 8), dtype=torch.int32 if bits == 32 else torch.int64, device="cuda")
        st = lib.flexspmv_partition(ctypes.c_void_p(ro_t.data_ptr()), bits, ctypes.c_int64(nr), ctypes.c_int64(nnz),
                                    tile_items, ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(0))
        assert st == 0
        torch.cuda.synchronize()
        got = out.cpu().numpy().reshape(-1, 2)
        assert np.array_equal(got, ref)
        # and against the reference header's own MergePathSearch, called in the compiled reference object
        from oracle import ref_run
        if ref_run.available("spmv") and got.shape[0] <= 4000:
            diagonals = np.minimum(np.arange(got.shape[0], dtype=np.int64) * tile_items, nr + nnz)
            assert np.array_equal(got, ref_run.reference_merge_path_search(ro, diagonals))


def test_row_blocks_bit_exact():
    lib = load_library()
    rng = np.random.default_rng(2)
    ro = problems.random_cut_csr(5000, 777777, rng).astype(np.int64)
    ro_t = torch.from_numpy(ro).cuda()
    for parts, snap in [(1, 1), (2, 1), (8, 1), (8, 64), (3, 1000)]:
        out = torch.empty(parts + 1, dtype=torch.int64, device="cuda")
        assert lib.flexspmv_row_blocks(ctypes.c_void_p(ro_t.data_ptr()), 64, ctypes.c_int64(5000), parts,
                                       ctypes.c_int64(snap), ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(0)) == 0
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), ir_eval.nnz_balanced_row_blocks(ro, parts, snap))


def test_errors_are_loud():
    ir = graphs.spmv_graph()
    ext = GraphExtension(ir)
    prob = problems.random_problem(ir, 10, 10, 50, seed=1, dtype=np.float32)
    vals = torch.from_numpy(prob.values["vals"]).cuda()
    x = torch.from_numpy(prob.values["x"]).cuda()
    idx = torch.from_numpy(prob.indices["selector"]).cuda()
    ro = torch.from_numpy(prob.row_offsets).cuda()
    with pytest.raises(RuntimeError):
        ext.merged_spmv_launch(vals.cpu(), x, idx, ro, 10, 10)            # CPU tensor
    with pytest.raises(RuntimeError):
        ext.merged_spmv_launch(vals.half(), x.half(), idx, ro, 10, 10)    # unsupported dtype
    with pytest.raises(RuntimeError):
        ext.merged_spmv_launch(vals, x.double(), idx, ro, 10, 10)         # dtype mismatch
    with pytest.raises(RuntimeError):
        ext.merged_spmv_launch(vals, x, idx.long(), ro, 10, 10)           # index dtype
    with pytest.raises(RuntimeError):
        ext.merged_spmv_launch(vals[1:], x, idx, ro, 10, 10)              # misaligned streamed array (and short)
    lib = load_library()
    assert lib.flexspmv_partition(None, 32, ctypes.c_int64(1), ctypes.c_int64(1), 4, None, None) != 0


def test_c_abi_edge_cases_empty_matrices():
    """Below the operator's own `ne > 0` check the C ABI accepts matrices without edges (every row sums to
    0) and without rows (nothing to do)."""
    ir = graphs.spmv_graph()
    ext = GraphExtension(ir)
    dev = torch.device("cuda:0")
    x = torch.ones(64, dtype=torch.float64, device=dev)
    vals = torch.zeros(16, dtype=torch.float64, device=dev)       # valid, aligned pointers; no element is read
    cols = torch.zeros(16, dtype=torch.int32, device=dev)
    for rows in (1, 37, 5000):
        ro = torch.zeros(rows + 1, dtype=torch.int32, device=dev)
        y = torch.full((rows,), float("nan"), dtype=torch.float64, device=dev)
        ext.launch_into([vals, x], [cols], ro, [y], rows, 0, 64)
        torch.cuda.synchronize()
        assert float(y.abs().max()) == 0.0
    ro = torch.zeros(1, dtype=torch.int32, device=dev)
    y = torch.full((4,), 7.0, dtype=torch.float64, device=dev)
    ext.launch_into([vals, x], [cols], ro, [y], 0, 0, 64)          # zero rows, zero edges: no launch at all
    torch.cuda.synchronize()
    assert float(y.min()) == 7.0
    assert ext.device_status(torch.float64) == 0


def test_coo_rows_to_csr_bit_exact_and_checked():
    """Device COO -> CSR offsets against numpy (int32 and int64 ids, empty rows, empty input); unsorted ids
    and ids outside [0, rows) are reported, not silently mis-converted."""
    from flexspmv_b200.python_wrapper.dynamic_replace_submodule import coo_rows_to_csr_ptr
    rng = np.random.default_rng(4)
    for rows, edges in [(1, 1), (1000, 0), (5000, 123457), (17, 100000), (300000, 4000)]:
        ids = np.sort(rng.integers(0, rows, edges))
        want = np.searchsorted(ids, np.arange(rows + 1), side="left").astype(np.int64)
        for dt in (np.int32, np.int64):
            got = coo_rows_to_csr_ptr(torch.from_numpy(ids.astype(dt)).cuda(), rows)
            assert got.dtype == torch.int64 and np.array_equal(got.cpu().numpy(), want)
    bad = torch.tensor([0, 2, 1, 3], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError):
        coo_rows_to_csr_ptr(bad, 4)
    with pytest.raises(RuntimeError):
        coo_rows_to_csr_ptr(torch.tensor([0, 1, 9], dtype=torch.int64, device="cuda"), 4)


@pytest.mark.parametrize("gname,dt", [("spmv", "float64"), ("spmv", "float32"), ("spmv", "int64"), ("ops_zoo", "float64")])
def test_gather_windows_are_bit_identical_to_global_gathers(gname, dt):
    """Banded matrices (every tile gets windows), random columns (no tile does), and a mix; int32 and int64
    offsets; gathered arrays whose length is not a multiple of 16 bytes."""
    ir = graphs.ALL_GRAPHS[gname]()
    dtype = np.dtype(dt)
    # same tile size and CTA count on both sides: which partial sums meet at a tile or CTA boundary is part of
    # the rounding, and the two kernels have different numbers of resident CTAs
    plain = GraphExtension(ir, gather_windows=False, max_ctas=296)
    win = GraphExtension(ir, gather_windows=True, max_ctas=296)
    assert win._flags(win.symbols(NP2T[dtype])) == 1
    probs = []
    if gname == "spmv":
        for mk in (lambda: problems.poisson2d(97), lambda: problems.poisson3d(23), lambda: problems.poisson3d(31, offset_dtype=np.int32)):
            p = mk()
            p.values = {k: (v * 3).astype(dtype) if dtype.kind == "i" else v.astype(dtype) for k, v in p.values.items()}
            probs.append(p)
    rng = np.random.default_rng(17)
    for nr, nnz, band in [(4001, 60000, 40), (4001, 60000, 0), (777, 30011, 3), (50, 20000, 0)]:
        p = problems.random_problem(ir, nr, nr, nnz, seed=nr + nnz + band, dtype=dtype)
        if band:       # columns within +-band of the row, plus a second band far away for every third edge
            rows = np.repeat(np.arange(nr), np.diff(p.row_offsets))
            off = rng.integers(-band, band + 1, nnz)
            far = (np.arange(nnz) % 3 == 0) * (nr // 2)
            key = next(iter(p.indices))
            p.indices[key] = np.clip(rows + off + far, 0, nr - 1).astype(np.int32)
        probs.append(p)
    for p in probs:
        a, _ = run_gpu(plain, ir, p, dtype)
        b, _ = run_gpu(win, ir, p, dtype)
        for x, y in zip(a, b):
            assert np.array_equal(x, y, equal_nan=True)
    assert win.device_status(NP2T[dtype]) == 0


def test_gather_window_plan_bit_exact():
    """The per-tile segment table and the per-edge 16-bit positions against their numpy restatement."""
    from flexspmv_b200.binding import Desc
    lib = load_library()
    for prob, bits in ((problems.poisson3d(23, offset_dtype=np.int32), 32), (problems.poisson3d(17), 64),
                       (problems.random_problem(graphs.spmv_graph(), 300, 300, 9000, 5, np.float64), 32)):
        ro = prob.row_offsets.astype(np.int32 if bits == 32 else np.int64)
        cols = prob.indices["selector"]
        desc = Desc(prob.num_rows, prob.nnz, prob.num_cols, bits, 0, 0, 1)
        nbytes = ctypes.c_size_t()
        for f in (lib.flexspmv_spmv_f64_workspace_bytes, lib.flexspmv_spmv_f64_plan, lib.flexspmv_spmv_f64_plan_windows):
            f.restype = ctypes.c_int
        assert lib.flexspmv_spmv_f64_workspace_bytes(ctypes.byref(desc), ctypes.byref(nbytes)) == 0
        ws = torch.zeros(nbytes.value, dtype=torch.uint8, device="cuda")
        ro_t, cols_t = torch.from_numpy(ro).cuda(), torch.from_numpy(cols).cuda()
        assert lib.flexspmv_spmv_f64_plan(ctypes.byref(desc), ctypes.c_void_p(ro_t.data_ptr()), ctypes.c_void_p(ws.data_ptr()),
                                          ctypes.c_size_t(nbytes.value), None) == 0
        ip = (ctypes.c_void_p * 1)(cols_t.data_ptr())
        assert lib.flexspmv_spmv_f64_plan_windows(ctypes.byref(desc), ip, ctypes.c_void_p(ws.data_ptr()),
                                                  ctypes.c_size_t(nbytes.value), None) == 0
        torch.cuda.synchronize()
        raw = ws.cpu().numpy()
        # workspace header: tile_items is the int32 at byte 40, the window table / index offsets the int64 at 112 / 120
        tile_items = int(raw[:256].view(np.int32)[10])
        coords = ir_eval.tile_coordinates(ro, tile_items)
        tiles = coords.shape[0] - 1
        # the plan moves the boundaries between the CTAs of its grid onto row ends where it can (int32 at byte 132: that
        # grid, 0 when it could not): the coordinates in the workspace against the restatement of that step
        snapped_grid = int(raw[:256].view(np.int32)[33])
        if snapped_grid:
            coords, ok = ir_eval.snap_cta_boundaries(coords, ro, snapped_grid)
            assert ok
        got_coords = raw[256:256 + coords.nbytes].view(coords.dtype).reshape(coords.shape)
        assert np.array_equal(got_coords, coords)
        t_off, i_off = (int(v) for v in raw[112:128].view(np.int64))
        table = raw[t_off:t_off + tiles * 112].view(np.int32).reshape(tiles, 28)[:, :26]
        pos = raw[i_off:i_off + 2 * prob.nnz].view(np.uint16)
        want_table, want_pos = ir_eval.gather_window_plan(coords, cols, 8, 8192)
        assert np.array_equal(table, want_table)
        assert np.array_equal(pos, want_pos)


def test_bounded_wait_runs_out_and_the_context_stays_usable():
    """A stage that is never filled (testing aid flexspmv_debug_withhold_stage) makes the consumers' one-second
    wait run out: the launch returns, the workspace status says FLEXSPMV_ERR_TIMEOUT, rows of the tiles before
    the withheld one are correct, and after a fresh plan the same workspace gives the full result again."""
    from flexspmv_b200.binding import Desc
    lib = load_library()
    ir = graphs.spmv_graph()
    prob = problems.random_problem(ir, 4000, 4000, 60000, seed=77, dtype=np.float64)
    ref, _, sums = ir_eval.run_graph(ir, prob, np.float64, num_threads=4, want_abs_sums=True)
    dev = torch.device("cuda:0")
    vals, x = (torch.from_numpy(prob.values[k]).to(dev) for k in ("vals", "x"))
    cols = torch.from_numpy(prob.indices["selector"]).to(dev)
    ro = torch.from_numpy(prob.row_offsets).to(dev)
    y = torch.full((prob.num_rows,), float("nan"), dtype=torch.float64, device=dev)
    desc = Desc(prob.num_rows, prob.nnz, prob.num_cols, 32, 0, 0, 0)
    nbytes = ctypes.c_size_t()
    for name in ("workspace_bytes", "plan", "launch", "device_status"):
        getattr(lib, f"flexspmv_spmv_f64_{name}").restype = ctypes.c_int
    lib.flexspmv_debug_withhold_stage.restype = ctypes.c_int
    assert lib.flexspmv_spmv_f64_workspace_bytes(ctypes.byref(desc), ctypes.byref(nbytes)) == 0
    ws = torch.zeros(nbytes.value, dtype=torch.uint8, device=dev)
    wsp, nb = ctypes.c_void_p(ws.data_ptr()), ctypes.c_size_t(nbytes.value)
    vp = (ctypes.c_void_p * 2)(vals.data_ptr(), x.data_ptr())
    ip = (ctypes.c_void_p * 1)(cols.data_ptr())
    op = (ctypes.c_void_p * 1)(y.data_ptr())
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def plan_and_launch(withhold):
        assert lib.flexspmv_spmv_f64_plan(ctypes.byref(desc), ctypes.c_void_p(ro.data_ptr()), wsp, nb, None) == 0
        if withhold:
            assert lib.flexspmv_debug_withhold_stage(wsp, ctypes.c_uint32(withhold), None) == 0
        assert lib.flexspmv_spmv_f64_launch(ctypes.byref(desc), vp, ip, ctypes.c_void_p(ro.data_ptr()), op, wsp, nb, None) == 0
        assert lib.flexspmv_spmv_f64_device_status(wsp, ctypes.c_void_p(status.data_ptr()), None) == 0
        torch.cuda.synchronize()
        return int(status.item())

    tile_items = 1280
    tiles = (prob.num_rows + prob.nnz + tile_items - 1) // tile_items
    assert tiles >= 20
    first_withheld = 11                                   # 1-based: tiles 0..9 are staged, 10.. never
    assert plan_and_launch(first_withheld) == -6          # FLEXSPMV_ERR_TIMEOUT
    coords = ir_eval.tile_coordinates(prob.row_offsets, tile_items)
    done_rows = int(coords[first_withheld - 1, 0])        # rows that end inside the staged tiles
    got = y.cpu().numpy()
    from parity import row_error
    assert row_error(got[:done_rows], ref[0][:done_rows], sums[0][:done_rows]) <= 1e-12
    y.fill_(float("nan"))
    assert plan_and_launch(0) == 0                        # plan resets the status and the aid
    assert row_error(y.cpu().numpy(), ref[0], sums[0]) <= 1e-12


def test_row_aligned_plan_serves_launches_of_any_grid():
    """The plan moves the boundaries between the CTAs of ITS grid onto row ends (workspace header, int32 at byte 132);
    a launch of that grid hands no carries over, a launch of another grid (descriptor with another max_ctas) finds
    boundaries of its own that cut rows and must hand them over as before.  Both give the oracle's rows."""
    from flexspmv_b200.binding import Desc
    from parity import row_error
    lib = load_library()
    ir = graphs.spmv_graph()
    prob = problems.poisson2d(150)
    ref, _, sums = ir_eval.run_graph(ir, prob, np.float64, num_threads=4, want_abs_sums=True)
    dev = torch.device("cuda:0")
    vals, x = (torch.from_numpy(prob.values[k]).to(dev) for k in ("vals", "x"))
    cols = torch.from_numpy(prob.indices["selector"]).to(dev)
    ro = torch.from_numpy(prob.row_offsets).to(dev)
    y = torch.empty(prob.num_rows, dtype=torch.float64, device=dev)
    for name in ("workspace_bytes", "plan", "launch", "device_status"):
        getattr(lib, f"flexspmv_spmv_f64_{name}").restype = ctypes.c_int
    desc = Desc(prob.num_rows, prob.nnz, prob.num_cols, 32, 0, 0, 0)
    nbytes = ctypes.c_size_t()
    assert lib.flexspmv_spmv_f64_workspace_bytes(ctypes.byref(desc), ctypes.byref(nbytes)) == 0
    ws = torch.zeros(nbytes.value, dtype=torch.uint8, device=dev)
    wsp, nb = ctypes.c_void_p(ws.data_ptr()), ctypes.c_size_t(nbytes.value)
    assert lib.flexspmv_spmv_f64_plan(ctypes.byref(desc), ctypes.c_void_p(ro.data_ptr()), wsp, nb, None) == 0
    torch.cuda.synchronize()
    tiles = (prob.num_rows + prob.nnz + 1279) // 1280
    assert int(ws[:256].cpu().numpy().view(np.int32)[33]) == tiles        # fewer tiles than CTA slots: one tile per CTA
    vp = (ctypes.c_void_p * 2)(vals.data_ptr(), x.data_ptr())
    ip = (ctypes.c_void_p * 1)(cols.data_ptr())
    op = (ctypes.c_void_p * 1)(y.data_ptr())
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for max_ctas in (0, 7, 1, 50):
        launch_desc = Desc(prob.num_rows, prob.nnz, prob.num_cols, 32, 0, max_ctas, 0)
        y.fill_(float("nan"))
        assert lib.flexspmv_spmv_f64_launch(ctypes.byref(launch_desc), vp, ip, ctypes.c_void_p(ro.data_ptr()), op, wsp, nb, None) == 0
        assert lib.flexspmv_spmv_f64_device_status(wsp, ctypes.c_void_p(status.data_ptr()), None) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert row_error(y.cpu().numpy(), ref[0], sums[0]) <= 1e-12, max_ctas


def test_failed_launch_reaches_the_host_without_a_status_copy():
    """The operator registers a page-locked int with every workspace it plans; a kernel that gives up stores its
    status there.  `ext.check()` and the next call on that workspace raise; nothing on the launch path
    synchronises.  A fresh plan (new row-offset tensor) works again."""
    from flexspmv_b200.binding import FlexSpmvError
    lib = load_library()
    lib.flexspmv_debug_withhold_stage.restype = ctypes.c_int
    ir = graphs.spmv_graph()
    ext = GraphExtension(ir)
    prob = problems.random_problem(ir, 4000, 4000, 60000, seed=78, dtype=np.float64)
    dev = torch.device("cuda:0")
    vals, x = (torch.from_numpy(prob.values[k]).to(dev) for k in ("vals", "x"))
    cols = torch.from_numpy(prob.indices["selector"]).to(dev)
    ro = torch.from_numpy(prob.row_offsets).to(dev)
    (want,) = ext.merged_spmv_launch(vals, x, cols, ro, prob.num_rows, prob.num_cols)
    ext.check()                                            # nothing failed so far
    plan = next(reversed(ext._plans.values()))
    assert plan.status() == 0
    assert lib.flexspmv_debug_withhold_stage(ctypes.c_void_p(plan.ws.data_ptr()), ctypes.c_uint32(5), None) == 0
    ext.merged_spmv_launch(vals, x, cols, ro, prob.num_rows, prob.num_cols)     # enqueues; the wait runs out on the device
    with pytest.raises(FlexSpmvError, match="bounded device-side wait"):
        ext.check()
    with pytest.raises(FlexSpmvError, match="outputs are undefined"):
        ext.merged_spmv_launch(vals, x, cols, ro, prob.num_rows, prob.num_cols)
    assert ext.device_status(torch.float64) == -6
    ro2 = ro.clone()                                       # another tensor: another plan, another workspace
    (again,) = ext.merged_spmv_launch(vals, x, cols, ro2, prob.num_rows, prob.num_cols)
    torch.cuda.synchronize()
    assert torch.equal(again, want)


def test_edge_kernel_refuses_a_workspace_that_was_never_planned():
    """The aggregator / map-only kernel checks the header like the tile kernel: on a zero-filled workspace it
    raises FLEXSPMV_ERR_NOT_PLANNED, writes no output, and a planned workspace of another problem size is
    refused the same way."""
    lib = load_library()
    for name in ("workspace_bytes", "plan", "launch", "device_status"):
        getattr(lib, f"flexspmv_edge_sum_f32_{name}").restype = ctypes.c_int
    dev = torch.device("cuda:0")
    E, NV = 5000, 300
    g = torch.Generator(device="cpu")
    g.manual_seed(5)
    ew = torch.rand(E, 2, generator=g).to(dev)
    vx = torch.rand(NV, 2, generator=g).to(dev)
    sel = torch.randint(0, NV, (E,), generator=g, dtype=torch.int32).to(dev)
    prod = torch.full((E, 2), float("nan"), device=dev)
    total = torch.full((2,), float("nan"), device=dev)
    desc = Desc(0, E, NV, 32, 0, 0, 0)
    nbytes = ctypes.c_size_t()
    assert lib.flexspmv_edge_sum_f32_workspace_bytes(ctypes.byref(desc), ctypes.byref(nbytes)) == 0
    ws = torch.zeros(nbytes.value, dtype=torch.uint8, device=dev)
    wsp, nb = ctypes.c_void_p(ws.data_ptr()), ctypes.c_size_t(nbytes.value)
    vp = (ctypes.c_void_p * 2)(ew.data_ptr(), vx.data_ptr())
    ip = (ctypes.c_void_p * 1)(sel.data_ptr())
    op = (ctypes.c_void_p * 2)(prod.data_ptr(), total.data_ptr())
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def launch(d):
        assert lib.flexspmv_edge_sum_f32_launch(ctypes.byref(d), vp, ip, None, op, wsp, nb, None) == 0
        assert lib.flexspmv_edge_sum_f32_device_status(wsp, ctypes.c_void_p(status.data_ptr()), None) == 0
        torch.cuda.synchronize()
        return int(status.item())

    assert launch(desc) == -7                              # FLEXSPMV_ERR_NOT_PLANNED
    assert torch.isnan(prod).all() and torch.isnan(total).all()
    assert lib.flexspmv_edge_sum_f32_plan(ctypes.byref(desc), None, wsp, nb, None) == 0
    assert launch(desc) == 0
    want = ew * vx[sel.long()]
    assert torch.equal(prod, want)
    assert torch.allclose(total, want.sum(dim=0), rtol=1e-5)
    smaller = Desc(0, E - 1, NV, 32, 0, 0, 0)              # planned for E edges, launched for E - 1
    prod.fill_(float("nan"))
    assert launch(smaller) == -7
    assert torch.isnan(prod).all()


@pytest.mark.parametrize("dt", ["float32", "float64", "int64"])
def test_warp_kernel_for_random_columns_matches_oracle(dt):
    """The kernel without staging (FLEXSPMV_FLAG_RANDOM_GATHER): same shapes as the plain path (empty rows, rows
    spanning many chunks, one row, no rows), odd chunk sizes and few CTAs (long carry chains across warps),
    int64 bit-exact, run-to-run deterministic."""
    ir = graphs.spmv_graph()
    dtype = np.dtype(dt)
    ext = GraphExtension(ir, random_gather=True)
    assert ext.symbols(NP2T[dtype]).graph_info.reserved & 2
    shapes = SHAPES + [(2, 5000, 300000), (40000, 40000, 40)]
    for (nr, nv, nnz) in shapes:
        prob = problems.random_problem(ir, nr, nv, nnz, seed=2000 + nr + nnz, dtype=dtype)
        ref, _, sums = ir_eval.run_graph(ir, prob, dtype, num_threads=8, want_abs_sums=True)
        got, _ = run_gpu(ext, ir, prob, dtype)
        assert_outputs_match(ir, got, ref, sums, dtype, what=f"warp kernel {dt} {nr}x{nnz}")
        again, _ = run_gpu(ext, ir, prob, dtype)
        assert np.array_equal(got[0], again[0])
    prob = problems.random_problem(ir, 97, 97, 60000, seed=6, dtype=dtype)
    ref, _, sums = ir_eval.run_graph(ir, prob, dtype, num_threads=4, want_abs_sums=True)
    for tile_items, max_ctas in ((1, 2), (7, 3), (33, 1), (160, 3), (159, 0)):
        small = GraphExtension(ir, random_gather=True, tile_items=tile_items, max_ctas=max_ctas)
        sub = prob if tile_items > 7 else problems.random_problem(ir, 97, 97, 3000, seed=6, dtype=dtype)
        r2, _, s2 = (ref, None, sums) if sub is prob else ir_eval.run_graph(ir, sub, dtype, num_threads=4, want_abs_sums=True)
        got, _ = run_gpu(small, ir, sub, dtype, offsets_dtype=np.int64 if tile_items == 33 else None)
        assert_outputs_match(ir, got, r2, s2, dtype, what=f"warp kernel {dt} chunk {tile_items} ctas {max_ctas}")
        assert small.device_status(NP2T[dtype]) == 0


def test_random_gather_is_detected_per_matrix():
    """Left to itself the operator samples the index array once per matrix: a power-law matrix with random columns
    takes the warp kernel, a stencil matrix the staged kernel; both agree with the oracle."""
    ir = graphs.spmv_graph()
    ext = GraphExtension(ir)
    for prob, expect in ((problems.powerlaw(1 << 17, cap=20000), 2), (problems.poisson2d(512), 0)):
        ref, _, sums = ir_eval.run_graph(ir, prob, prob.values["vals"].dtype, num_threads=8, want_abs_sums=True)
        got, _ = run_gpu(ext, ir, prob, prob.values["vals"].dtype)
        assert_outputs_match(ir, got, ref, sums, prob.values["vals"].dtype, what="auto-detected kernel")
        key = next(reversed(ext._plans))
        assert key[6] == expect          # the flags the plan was made with


def test_rows_spanning_every_cta():
    """Two rows of 1.5 M edges each: every CTA contributes a carry to the same row and the last CTA folds
    hundreds of them (exact for int64, tolerance for fp64)."""
    ir = graphs.spmv_graph()
    ext = GraphExtension(ir)
    for dt in (np.int64, np.float64):
        prob = problems.random_problem(ir, 2, 5000, 3_000_000, seed=41, dtype=dt)
        prob.row_offsets = np.array([0, 1_500_000, 3_000_000], dtype=np.int32)
        ref, _, sums = ir_eval.run_graph(ir, prob, dt, num_threads=8, want_abs_sums=True)
        got, _ = run_gpu(ext, ir, prob, dt)
        assert_outputs_match(ir, got, ref, sums, np.dtype(dt), what=f"two long rows {np.dtype(dt).name}")
