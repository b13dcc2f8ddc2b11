"""The CPU oracle against (1) the committed golden fixtures, which were produced by the reference's
own generated CPU operator, (2) that operator itself when oracle/_ref is present, and (3) the
properties the reference's harnesses check (naive gold loop, src/flex_spmv_full_red.cu:74-133)."""
import os

import numpy as np
import pytest

from flexspmv_b200 import graphs, problems
from golden_io import golden_files, load
from oracle import ir_eval, ref_run

EXACT_GRAPHS = {"spmv", "spring_mass", "rusanov", "mixed_dims", "edge_sum", "edge_copy"}   # only exactly rounded ops


def _close(a, b, exact, dt):
    if exact or np.dtype(dt).kind == "i":
        return np.array_equal(a, b, equal_nan=True)
    tol = 1e-5 if np.dtype(dt) == np.float32 else 1e-12
    with np.errstate(invalid="ignore"):
        ok = np.isclose(a, b, rtol=tol, atol=tol * max(1.0, float(np.nanmax(np.abs(b))) if b.size else 1.0), equal_nan=True)
    return bool(ok.all())


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: os.path.basename(p)[:-4])
def test_oracle_matches_golden(path):
    prob, dt, threads, outs, written = load(path)
    ir = graphs.ALL_GRAPHS[prob.graph]()
    got, got_written = ir_eval.run_graph(ir, prob, dt, num_threads=threads)
    exact = prob.graph in EXACT_GRAPHS
    assert len(got) == len(outs)
    for g, r in zip(got, outs):
        assert g.shape == r.shape and g.dtype == r.dtype
        assert _close(g, r, exact, dt)
    for k, r in written.items():     # every value input after the call; untouched ones must be unchanged
        mine = got_written[k] if k in got_written else prob.values[k]
        assert _close(mine.reshape(r.shape), r, exact, dt)


def test_golden_set_is_complete():
    names = {os.path.basename(p) for p in golden_files()}
    assert len(names) >= 11
    for g in graphs.ALL_GRAPHS:
        assert any(n.startswith(g) for n in names), f"no golden fixture for graph {g}"


@pytest.mark.skipif(not ref_run.available(), reason="oracle/_ref not built (reference tree absent)")
@pytest.mark.parametrize("gname", list(graphs.ALL_GRAPHS))
def test_oracle_matches_compiled_reference(gname):
    ir = graphs.ALL_GRAPHS[gname]()
    for dt in graphs.GRAPH_DTYPES[gname]:
        for (nr, nv, nnz, T) in [(37, 37, 211, 3), (1231, 1231, 12313, 8), (500, 500, 40, 7), (3, 3, 5000, 16), (12, 12, 12, 256)]:
            prob = problems.random_problem(ir, nr, nv, nnz, seed=nr + nnz, dtype=np.dtype(dt))
            a, wa = ir_eval.run_graph(ir, prob, dt, num_threads=T)
            b, wb = ref_run.run_graph(ir, prob, dt, num_threads=T)
            for x, y in zip(a, b):
                assert _close(x, y, gname in EXACT_GRAPHS, dt), (gname, dt, nr, nnz)
            for k in wa:
                assert _close(wa[k].reshape(wb[k].shape), wb[k], gname in EXACT_GRAPHS, dt)


@pytest.mark.skipif(not ref_run.available("spmv"), reason="oracle/_ref not built")
def test_reference_configs_small():
    """Configs 0, 1, 2, 4 at reduced size: restatement == compiled reference, bit for bit."""
    cases = [("spmv", problems.poisson2d(48)), ("spring_mass", problems.spring_mass(40)),
             ("rusanov", problems.shallow_water(24)), ("spmv", problems.poisson3d(12, offset_dtype=np.int32)),
             ("spmv", problems.powerlaw(4096, cap=500))]
    for gname, prob in cases:
        ir = graphs.ALL_GRAPHS[gname]()
        a, _ = ir_eval.run_graph(ir, prob, num_threads=8)
        b, _ = ref_run.run_graph(ir, prob, num_threads=8)
        for x, y in zip(a, b):
            assert np.array_equal(x, y)


def test_spmv_oracle_against_naive_gold():
    ir = graphs.spmv_graph()
    prob = problems.random_problem(ir, 300, 300, 4000, 5, np.float64)
    (y,), _ = ir_eval.run_graph(ir, prob, num_threads=1)      # one thread: plain left-to-right row sums
    ro = prob.row_offsets
    gold = np.zeros(300)
    for r in range(300):
        s = 0.0
        for e in range(ro[r], ro[r + 1]):
            s += prob.values["vals"][e] * prob.values["x"][prob.indices["selector"][e]]
        gold[r] = s
    assert np.array_equal(y, gold)


def test_merge_path_search_properties():
    rng = np.random.default_rng(0)
    for nr, nnz in [(0, 0), (1, 0), (5, 0), (0, 7), (40, 200), (200, 40), (1000, 5000)]:
        ro = problems.random_cut_csr(nr, nnz, rng) if nr else np.array([0], np.int32)
        if nr == 0:
            continue
        prev = (0, 0)
        for d in range(0, nr + nnz + 1):
            x, y = ir_eval.merge_path_search(d, ro)
            assert x + y == d and 0 <= x <= nr and 0 <= y <= nnz
            assert x >= prev[0] and y >= prev[1]            # monotone path
            if x > 0:
                assert ro[x] <= y                            # rows consumed have ended at or before edge y
            if x < nr and y > 0:
                assert ro[x + 1] > y - 1                     # the current row has not ended before the last consumed edge
            prev = (x, y)
        assert ir_eval.merge_path_search(nr + nnz, ro) == (nr, nnz)
        x64 = ir_eval.merge_path_search(nr + nnz, ro.astype(np.int64))
        assert x64 == (nr, nnz)


def test_tile_coordinates_and_row_blocks():
    rng = np.random.default_rng(1)
    ro = problems.random_cut_csr(3000, 70000, rng)
    for t in (320, 896, 1280):
        c32 = ir_eval.tile_coordinates(ro, t)
        c64 = ir_eval.tile_coordinates(ro.astype(np.int64), t)
        assert np.array_equal(c32, c64)
        assert tuple(c32[0]) == (0, 0) and tuple(c32[-1]) == (3000, 70000)
        assert (np.diff(c32.sum(axis=1))[:-1] == t).all()
    fb = ir_eval.nnz_balanced_row_blocks(ro, 8)
    assert fb[0] == 0 and fb[-1] == 3000 and (np.diff(fb) >= 0).all()
    per = np.diff(ro.astype(np.int64)[fb])
    assert per.max() - per.min() <= 2 * np.diff(ro).max()      # balanced up to one row


def test_restated_search_equals_the_reference_headers_own_search():
    """The tile coordinates of the restatement against the reference's free function MergePathSearch
    (cpu_template/merged_spmv_template_reducer.h:27-51), called through the compiled reference object, for every
    tile diagonal of several matrices (empty rows, rows spanning tiles, no rows, no edges)."""
    from oracle import ref_run
    if not ref_run.available("spmv"):
        pytest.skip("oracle/_ref not built")
    rng = np.random.default_rng(11)
    for nr, nnz in ((1, 0), (1, 5), (37, 211), (500, 40), (3, 5000), (12314, 123134)):
        ro = problems.random_cut_csr(nr, nnz, rng)
        for tile in (5, 320, 896, 1280):
            if (nr + nnz) // tile > 3000:
                continue
            ours = ir_eval.tile_coordinates(ro, tile)
            diagonals = np.minimum(np.arange(ours.shape[0], dtype=np.int64) * tile, nr + nnz)
            theirs = ref_run.reference_merge_path_search(ro, diagonals)
            assert np.array_equal(ours, theirs), (nr, nnz, tile)


def test_tensor_semantics_corner_cases():
    """guarded divide returns 0 on a zero divisor for equal widths and scalar/tensor, but the
    mixed-width broadcast and tensor/scalar divides are plain IEEE (data_struct_shared.cuh)."""
    ev = ir_eval.IREvaluator(graphs.ops_zoo_graph(), np.float64)
    a = np.array([[1.0, 2.0]])
    z = np.array([[0.0, 4.0]])
    assert np.array_equal(ev._binary("truediv", a, z), [[0.0, 0.5]])
    assert np.array_equal(ev._binary("truediv", np.float64(3.0), z), [[0.0, 0.75]])
    with np.errstate(divide="ignore"):
        r = ev._binary("truediv", a, np.array([[0.0]]))
    assert np.isinf(r).all()
    r = ev._binary("mul", np.array([[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]), np.array([[10.0, 100.0]]))
    assert np.array_equal(r, [[10.0, 200.0, 30.0, 400.0, 50.0, 600.0]])          # index-modulo broadcast
    evi = ir_eval.IREvaluator(graphs.mixed_dims_graph(), np.int64)
    assert np.array_equal(evi._binary("truediv", np.array([[-7, 7]]), np.array([[2, -2]])), [[-3, -3]])   # C++ truncation


def test_snapped_cta_boundaries_keep_every_tile_within_its_capacity():
    """The restatement of the plan step that moves the boundaries between CTAs onto row ends: afterwards every CTA
    starts at the first edge of a row, no tile holds more edges than a tile has items, and boundaries stay ordered;
    a matrix whose rows are longer than a tile is left alone."""
    from flexspmv_b200 import problems
    prob = problems.poisson2d(40)
    ro = prob.row_offsets
    tile = 256
    coords = ir_eval.tile_coordinates(ro, tile)
    tiles = coords.shape[0] - 1
    for grid in (2, 7, tiles):
        snapped, ok = ir_eval.snap_cta_boundaries(coords, ro, grid)
        assert ok
        q, r = divmod(tiles, grid)
        for c in range(1, grid):
            t = c * q + min(c, r)
            assert snapped[t, 1] == ro[snapped[t, 0]]
        assert np.all(np.diff(snapped[:, 1]) >= 0) and np.all(np.diff(snapped[:, 1]) <= tile)
        assert np.array_equal(snapped[:, 0], coords[:, 0])
    long_rows = np.array([0, 5000, 5001, 9000], dtype=np.int32)
    c2 = ir_eval.tile_coordinates(long_rows, tile)
    same, ok = ir_eval.snap_cta_boundaries(c2, long_rows, 4)
    assert not ok and same is c2
