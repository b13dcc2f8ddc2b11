"""Unsorted reducers: the device's stable radix sort of row ids (``flexspmv_sort_rows``) against
``numpy.argsort(kind="stable")``, bit for bit, and the runtime wrapper on a Reducer whose ids are not ascending
(the reference's wrapper assumes they are: python_wrapper/dynamic_replace_submodule.py:20-41)."""
import numpy as np
import pytest
import torch
import torch.fx
import torch.nn as nn

from flexspmv_b200.python_wrapper.dynamic_replace_submodule import (DynamicCudaWrapper, dynamic_replace_submodule,
                                                                    permute_edges, sort_edges_by_row)

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,rows,dtype", [(1, 1, np.int32), (5, 3, np.int64), (2048, 16, np.int32), (2049, 17, np.int32),
                                          (100_000, 1, np.int32), (300_000, 70_000, np.int64), (1_000_003, 2_000_000, np.int32)])
def test_sort_rows_equals_stable_argsort(n, rows, dtype):
    rng = np.random.default_rng(n + rows)
    ids = rng.integers(0, rows, n).astype(dtype)
    if n > 1000:
        ids[: n // 3] = np.sort(ids[: n // 3])           # a partly sorted prefix
    perm, crow = sort_edges_by_row(torch.from_numpy(ids).cuda(), rows)
    torch.cuda.synchronize()
    want = np.argsort(ids, kind="stable")
    assert np.array_equal(perm.cpu().numpy(), want.astype(np.int32))
    counts = np.bincount(ids, minlength=rows)
    assert np.array_equal(crow.cpu().numpy(), np.concatenate([[0], np.cumsum(counts)]))
    vals = rng.random((n, 3))
    got = permute_edges(torch.from_numpy(vals).cuda(), perm)
    assert np.array_equal(got.cpu().numpy(), vals[want])


def test_sort_rows_flags_ids_out_of_range():
    from flexspmv_b200.binding import FlexSpmvError
    ids = torch.tensor([0, 5, 2], dtype=torch.int32).cuda()
    with pytest.raises(FlexSpmvError):
        sort_edges_by_row(ids, 4)


class Selector(nn.Module):
    def __init__(self, idx):
        super().__init__()
        self.register_buffer("idx", idx)

    def forward(self, t):
        return t[self.idx]


class Reducer(nn.Module):
    def __init__(self, idx, n):
        super().__init__()
        self.register_buffer("idx", idx)
        self.n = n

    def forward(self, t):
        out = torch.zeros((self.n,) + t.shape[1:], dtype=t.dtype, device=t.device)
        return out.index_add_(0, self.idx, t)


class Spmv(nn.Module):
    def __init__(self, rows, cols, n):
        super().__init__()
        self.selector = Selector(cols)
        self.reducer = Reducer(rows, n)

    def forward(self, vals, x):
        return [self.reducer(vals * self.selector(x))]


class LeafTracer(torch.fx.Tracer):
    def is_leaf_module(self, m, qualname):
        return isinstance(m, (Selector, Reducer))


def test_wrapper_accepts_an_unsorted_reducer():
    from flexspmv_b200.binding import load_builtin
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(12)
    n, e = 5000, 60000
    rows = torch.from_numpy(rng.integers(0, n, e)).to(dev)          # COO order, not sorted by row
    cols = torch.from_numpy(rng.integers(0, n, e)).to(dev)
    vals = torch.from_numpy(rng.uniform(-1, 1, e)).to(dev)
    x = torch.from_numpy(rng.uniform(-1, 1, n)).to(dev)
    model = Spmv(rows, cols, n).to(dev)
    gm = torch.fx.GraphModule(model, LeafTracer().trace(model))

    class Eqn(nn.Module):
        def __init__(self):
            super().__init__()
            self.fused = gm
            self.jit_engine = type("E", (), {})()
            g = torch.fx.Graph()
            args = [g.placeholder(nm) for nm in ("vals", "x")]
            g.output(g.call_module("fused", tuple(args)))
            self.jit_engine.graph = g

    eqn = Eqn()
    want = gm(vals, x)[0]
    name = [nd.name for nd in eqn.jit_engine.graph.nodes if nd.op == "call_module"][0]
    assert dynamic_replace_submodule(eqn, load_builtin("spmv"), name)
    wrapper = getattr(eqn, name)
    assert isinstance(wrapper, DynamicCudaWrapper) and wrapper._perm is not None
    got = wrapper(vals, x)[0]
    torch.cuda.synchronize()
    assert float((got - want).abs().max()) <= 1e-12 * 40
