"""Host-side logic that needs no GPU: IR -> operator signature, the CUDA emitter, tile configuration,
problem generators and the algorithmic-bytes figures of the benchmark configurations."""
import numpy as np
import pytest

from flexspmv_b200 import graphs, problems
from flexspmv_b200.codegen import emit_cuda


def test_operator_signature_follows_reference_binding_order():
    # non-gather values, gather values, one index tensor per selector target (codegen/merged_gen_binding.py:65-78)
    assert graphs.operator_signature(graphs.spmv_graph()) == (["vals"], ["x"], ["selector"])
    assert graphs.operator_signature(graphs.spring_mass_graph()) == (["L", "k"], ["p"], ["sel_src", "sel_dst"])
    assert graphs.operator_signature(graphs.rusanov_graph()) == (["face"], ["U"], ["sel_self", "sel_nbr"])
    assert graphs.operator_signature(graphs.mixed_dims_graph()) == (["ea", "eb"], ["vx"], ["s0", "s1"])


def test_binding_argument_names_without_gpu():
    from flexspmv_b200.binding import GraphExtension
    ext = GraphExtension(graphs.spring_mass_graph())
    assert ext.arg_names == ["L", "k", "p", "sel_src_idx", "sel_dst_idx", "row_end_offsets", "num_rows", "num_cols"]
    with pytest.raises(TypeError):
        ext.merged_spmv_launch(1, 2, 3)                  # missing arguments
    import torch
    t = torch.zeros(4)
    with pytest.raises(RuntimeError):                    # CPU tensors are refused: there is no CPU path
        ext.merged_spmv_launch(t, t, t.reshape(2, 2), t.int(), t.int(), t.int(), 3, 3)


def test_emitter_is_deterministic_and_resolves_overloads():
    ir = graphs.ops_zoo_graph()
    a = emit_cuda.emit_graph(ir, "float32")
    assert a == emit_cuda.emit_graph(graphs.ops_zoo_graph(), "float32")
    assert "fx::zip(w, sel, fx::DivGuard{})" in a              # equal widths: guarded member operator/
    assert "fx::zip_sv(V(1.5), sel, fx::DivGuard{})" in a      # scalar / tensor: guarded
    assert "fx::zip_vs(a4, nn, fx::Div{})" in a                # tensor / scalar: plain IEEE divide
    assert "FLEXSPMV_DEFINE_GRAPH(ops_zoo_f32, gen_ops_zoo_f32::Graph, gen_ops_zoo_f32::Cfg, gen_ops_zoo_f32::CfgWin, gen_ops_zoo_f32::CfgLean)" in a
    r = emit_cuda.emit_graph(graphs.rusanov_graph(), "float64")
    assert "fx::PowHalf{}" in r and "kGatherNeedsRow = true" in r and "kNumReducers = 3, kAccDim = 3" in r
    s = emit_cuda.emit_graph(graphs.spring_mass_graph(), "float32")
    assert "kNumStreams = 1" in s        # only the sel_dst index array is staged: sel_src is the row id, L and k are read directly
    assert "r.L = fx::ldg_vec<V, 1>(p.L + e * 1);" in s
    assert "kNumStreams = 2" in emit_cuda.emit_graph(graphs.spmv_graph(), "float64")    # two-phase graphs stage values too
    body = s.split("struct GRow")[1]
    assert "sel_src_idx" not in body and "idx_sel_src" not in body      # the row-identity index array is never read
    assert "g.sel_src = fx::ldg_vec<V, 2>(p.p + row * 2);" in body      # it is the row the merge path already knows
    assert "int idx_sel_dst;" in body
    m = emit_cuda.emit_graph(graphs.mixed_dims_graph(), "int64")
    assert "fx::st_vec(p.out_t1 + (long long)e * 2, t1)" in m  # per-edge map output


def test_emitter_rejects_what_the_reference_cannot_express():
    ir = graphs.spmv_graph()
    ir.map_operations.insert(0, graphs.mop("bad", "gt", (1,), 0.5, "vals"))
    with pytest.raises(ValueError):
        emit_cuda.emit_graph(ir, "float32")
    ir2 = graphs.spmv_graph()
    ir2.map_operations.insert(0, graphs.mop("u", "cosh", (1,), "vals"))
    with pytest.raises(ValueError):
        emit_cuda.emit_graph(ir2, "float32")


def test_tile_configs_fit_shared_memory():
    for g, make in graphs.ALL_GRAPHS.items():
        ir = make()
        if not ir.has_reducer:
            continue
        for dt in graphs.GRAPH_DTYPES[g]:
            block, ipt, stages, ctas = emit_cuda.choose_config(ir, dt)
            assert block % 32 == 0 and ipt % 2 == 1 and block * ipt <= 65535
            assert emit_cuda.smem_bytes(ir, dt, block, ipt, stages) * ctas <= 227 * 1024 + 1024 * ctas


def test_algorithmic_bytes_of_the_benchmark_configs():
    p0 = problems.poisson2d(512)
    assert (p0.num_rows, p0.nnz) == (262144, 1308672)
    assert problems.algorithmic_bytes(graphs.spmv_graph(), p0.num_rows, p0.nnz, p0.num_cols, 8, 4) == 20946948
    p1 = problems.spring_mass(64)
    assert p1.nnz == 8 * 64 * 64 - 6 * 64 * 2 + 4 - 0 or p1.nnz == int(p1.row_offsets[-1])
    n = 1024
    e1 = 8 * n * n - 12 * n + 4
    assert e1 == 8376324
    assert problems.algorithmic_bytes(graphs.spring_mass_graph(), n * n, e1, n * n, 4, 4) == 121487412
    assert problems.algorithmic_bytes(graphs.rusanov_graph(), 2 * n * n, 6 * n * n, 2 * n * n, 8, 4) == 285212676
    n3 = 512 ** 3
    nnz4 = 7 * n3 - 6 * 512 * 512
    assert nnz4 == 937951232
    assert problems.algorithmic_bytes(graphs.spmv_graph(), n3, nnz4, n3, 8, 8) == 14476640264


def test_generators_are_valid_csr():
    for prob in (problems.poisson2d(16), problems.poisson3d(6), problems.spring_mass(12), problems.shallow_water(8),
                 problems.powerlaw(2000, cap=300)):
        ro = prob.row_offsets
        assert ro[0] == 0 and (np.diff(ro) >= 0).all() and ro[-1] == prob.nnz and ro.shape[0] == prob.num_rows + 1
        for idx in prob.indices.values():
            assert idx.dtype == np.int32 and idx.min() >= 0 and idx.max() < prob.num_cols
    sm = problems.spring_mass(12)
    assert np.array_equal(sm.indices["sel_src"], np.repeat(np.arange(144), np.diff(sm.row_offsets)))
    sw = problems.shallow_water(8)
    nbr = sw.indices["sel_nbr"].reshape(-1, 3)
    own = np.arange(128)[:, None]
    back = nbr[nbr]                                   # neighbour relation is symmetric (or a boundary self-edge)
    assert ((back == own[:, None, :].repeat(3, axis=1).reshape(128, 3, 1)).any(axis=2) | (nbr == own)).all()
    face = sw.values["face"].reshape(-1, 3, 3)
    assert np.allclose((face[:, :, :2] * face[:, :, 2:3]).sum(axis=1), 0.0, atol=1e-15)   # closed cells: sum n*len = 0
    pl = problems.powerlaw(5000, cap=400)
    r = np.repeat(np.arange(5000), np.diff(pl.row_offsets))
    k = r.astype(np.int64) * (1 << 32) + pl.indices["selector"]
    assert (np.diff(k) >= 0).all()                    # columns sorted within each row


def test_warp_kernel_configuration_follows_the_value_width():
    """The emitter gives the random-column kernel 1024-thread CTAs for 4-byte values and 768-thread CTAs for 8-byte
    values (which need more than the 64 registers a 1024-thread CTA leaves a thread)."""
    from flexspmv_b200 import graphs
    from flexspmv_b200.codegen.emit_cuda import emit_graph
    ir = graphs.spmv_graph()
    assert "using CfgLean = flex::WarpCfg<1024, 5, 1>;" in emit_graph(ir, "float32", "spmv_f32")
    for dt, sym in (("float64", "spmv_f64"), ("int64", "spmv_i64")):
        assert "using CfgLean = flex::WarpCfg<768, 5, 1>;" in emit_graph(ir, dt, sym)
