"""Front-end pieces that sit above the operator: the tracer equivalent (driven with stand-ins for the
absent ``easier`` package), the reference-named codegen entry points and the runtime wrapper."""
import operator
import os

import numpy as np
import pytest
import torch
import torch.fx
import torch.nn as nn

from flexspmv_b200 import graphs
from flexspmv_b200.codegen import emit_cuda, merged_gen_binding, merged_gen_gpu
from flexspmv_b200.python_wrapper.dynamic_replace_submodule import (DynamicCudaWrapper, coo_rows_to_csr_ptr,
                                                                    dynamic_replace_submodule)
from flexspmv_b200.trace.graph_trace import classify_op, trace_graph


class Selector(nn.Module):
    def __init__(self, idx):
        super().__init__()
        self.idx = idx

    def forward(self, t):
        return t[self.idx]


class Reducer(nn.Module):
    def __init__(self, idx, n):
        super().__init__()
        self.idx, self.n = idx, n

    def forward(self, t):
        out = torch.zeros((self.n,) + t.shape[1:], dtype=t.dtype)
        return out.index_add_(0, self.idx, t)


class SpmvModel(nn.Module):
    def __init__(self, rows, cols, n):
        super().__init__()
        self.selector = Selector(cols)
        self.reducer = Reducer(rows, n)

    def forward(self, vals, x):
        return [self.reducer(vals * self.selector(x))]


class LeafTracer(torch.fx.Tracer):
    def is_leaf_module(self, m, qualname):
        return isinstance(m, (Selector, Reducer))


def _traced():
    rows = torch.tensor([0, 0, 1, 3, 3, 3])
    cols = torch.tensor([1, 2, 0, 3, 1, 2])
    model = SpmvModel(rows, cols, 4)
    gm = torch.fx.GraphModule(model, LeafTracer().trace(model))
    return model, gm


def test_trace_graph_reproduces_the_spmv_ir():
    model, gm = _traced()
    mods = dict(gm.named_modules())
    six = trace_graph(gm, None,
                      is_selector=lambda n: n.op == "call_module" and isinstance(mods[n.target], Selector),
                      is_reducer=lambda n: n.op == "call_module" and isinstance(mods[n.target], Reducer),
                      node_meta=lambda n: ((), torch.float32))
    ir = graphs.GraphIR("traced_spmv", *six)
    ref = graphs.spmv_graph()
    assert graphs.operator_signature(ir) == graphs.operator_signature(ref)
    assert [m["op"] for m in ir.map_operations] == ["mul", "reducer"]
    assert [o["target"] for o in ir.outputs] == ["reducer"]
    # the emitter accepts the traced IR and produces the same kernel body as the hand-built one
    a = emit_cuda.emit_graph(ir, "float32", "x")
    b = emit_cuda.emit_graph(ref, "float32", "x")
    assert a.split("\n", 1)[1] == b.split("\n", 1)[1]


def test_classify_op_follows_the_reference_table():
    assert classify_op(operator.add) == "add" and classify_op(operator.truediv) == "truediv"
    assert classify_op(operator.lt) == "lt" and classify_op(operator.getitem) == "getitem"
    assert classify_op("add_") == "add_" and classify_op("<built-in method where of type>") == "where"
    with pytest.raises(ValueError):
        classify_op("cosh")


def test_generate_sources_from_ir(tmp_path):
    paths = merged_gen_gpu.generate_cuda_code_from_ir(graphs.spring_mass_graph(), ("float32",), str(tmp_path))
    text = open(paths[0]).read()
    assert "FLEXSPMV_DEFINE_GRAPH(spring_mass_f32, gen_spring_mass_f32::Graph," in text and "kGatherNeedsRow = true" in text


def test_coo_rows_to_csr_ptr():
    assert coo_rows_to_csr_ptr(torch.tensor([0, 0, 1, 3, 3, 3]), 5).tolist() == [0, 2, 3, 3, 6, 6]
    with pytest.raises(ValueError):
        coo_rows_to_csr_ptr(torch.tensor([0, 2, 1]), 3)


class FakeExt:
    def __init__(self):
        self.calls = []

    def merged_spmv_launch(self, *a):
        self.calls.append(a)
        return (torch.zeros(a[-2]),)


def test_wrapper_marshals_arguments_in_operator_order():
    model, gm = _traced()

    class Eqn(nn.Module):
        def __init__(self):
            super().__init__()
            self.fused = gm
            self.jit_engine = type("E", (), {})()
            g = torch.fx.Graph()
            a, b = g.placeholder("vals"), g.placeholder("x")
            g.output(g.call_module("fused", (a, b)))
            self.jit_engine.graph = g

    eqn = Eqn()
    ext = FakeExt()
    node_name = [n.name for n in eqn.jit_engine.graph.nodes if n.op == "call_module"][0]
    assert dynamic_replace_submodule(eqn, ext, node_name)
    w = getattr(eqn, node_name)
    assert isinstance(w, DynamicCudaWrapper)
    vals, x = torch.arange(6.0), torch.arange(4.0)
    out = w(vals, x)
    assert isinstance(out, list) and out[0].shape == (4,)
    (a_vals, a_x, a_idx, a_ro, n_rows, n_cols), = ext.calls
    assert a_vals is vals and a_x is x                     # no copies of contiguous inputs
    assert a_idx.dtype == torch.int32 and a_idx.tolist() == [1, 2, 0, 3, 1, 2]
    assert a_ro.dtype == torch.int32 and a_ro.tolist() == [0, 2, 3, 3, 6]
    assert (n_rows, n_cols) == (4, 4)
    assert not dynamic_replace_submodule(eqn, ext, "no_such_node")


def test_generated_binding_source_follows_the_reference_contract(tmp_path):
    """No GPU work: the emitted text has the operator's positional order and keyword names, the output shapes of
    every output kind, and no per-call allocation of scratch."""
    ir = graphs.mixed_dims_graph()
    path = merged_gen_binding.generate_binding_code(str(tmp_path), ir.inputs, ir.outputs, ir.selector_register,
                                                    ir.map_operations, ir.reducer_operations, ir.aggregator_operations,
                                                    name=ir.name, dtypes=("float32", "int64"))
    text = open(path).read()
    order = [text.index(f'py::arg("{n}")') for n in ("ea", "eb", "vx", "s0_idx", "s1_idx", "row_end_offsets", "num_rows", "num_cols")]
    assert order == sorted(order)
    assert "torch::empty({num_rows, 2}" in text and "torch::empty({num_rows, 6}" in text and "torch::empty({ne, 2}" in text
    assert "case torch::kLong" in text and "case torch::kDouble" not in text
    assert "cudaMalloc" not in text and "cudaFree" not in text
    for f in ("flexspmv.h", "flex_tile_kernel.cuh", "merged_graph_merged_mixed_dims_f32.cuh", "merged_graph_merged_mixed_dims_i64.cuh"):
        assert os.path.exists(os.path.join(str(tmp_path), "include", f))
