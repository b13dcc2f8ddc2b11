"""The reference's whole flow on the GPU, with stand-ins for the absent ``easier`` package: an FX-traced
module built from Selector / Reducer modules -> ``trace_graph`` -> generated CUDA source -> nvcc (JIT) ->
``dynamic_replace_submodule`` -> the wrapper's call, compared with the eager module
(test_full/easier_full.py:300-420 is the reference driver this mirrors)."""
import shutil

import numpy as np
import pytest
import torch
import torch.fx
import torch.nn as nn
from torch.fx.passes.shape_prop import ShapeProp

from flexspmv_b200 import graphs
from flexspmv_b200.codegen import merged_gen_gpu
from flexspmv_b200.python_wrapper.dynamic_replace_submodule import DynamicCudaWrapper, dynamic_replace_submodule
from flexspmv_b200.trace.graph_trace import trace_graph

pytestmark = pytest.mark.gpu


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


class SpringForces(nn.Module):
    """f_i = sum over edges (i -> j) of k (|d| - L) d / |d|, d = p_j - p_i  (the reference's spring-mass map)."""

    def __init__(self, src, dst, n):
        super().__init__()
        self.sel_src, self.sel_dst = Selector(src), Selector(dst)
        self.reducer = Reducer(src, n)

    def forward(self, L, k, p):
        d = self.sel_dst(p) - self.sel_src(p)
        n = torch.norm(d, dim=1, keepdim=True)
        f = (k * (n - L)) * d / n
        return [self.reducer(f)]


class LeafTracer(torch.fx.Tracer):
    def is_leaf_module(self, m, qualname):
        return isinstance(m, (Selector, Reducer))


@pytest.mark.parametrize("dt", [torch.float64, torch.float32])
def test_traced_module_runs_through_generated_operator(dt):
    if shutil.which("nvcc") is None and not __import__("os").path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("needs nvcc to build the generated operator")
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(5)
    n, deg = 3000, 6
    src = np.repeat(np.arange(n), deg)
    dst = (src + rng.integers(1, 40, src.shape[0])) % n
    e = src.shape[0]
    src_t, dst_t = torch.from_numpy(src).to(dev), torch.from_numpy(dst).to(dev)
    p = torch.from_numpy(rng.random((n, 2))).to(dev, dt)
    L = torch.from_numpy(rng.uniform(0.1, 0.5, (e, 1))).to(dev, dt)
    k = torch.from_numpy(rng.uniform(0.5, 2.0, (e, 1))).to(dev, dt)

    model = SpringForces(src_t, dst_t, n).to(dev)
    gm = torch.fx.GraphModule(model, LeafTracer().trace(model))
    ShapeProp(gm).propagate(L, k, p)
    mods = dict(gm.named_modules())
    six = trace_graph(gm, None,
                      is_selector=lambda nd: nd.op == "call_module" and isinstance(mods[nd.target], Selector),
                      is_reducer=lambda nd: nd.op == "call_module" and isinstance(mods[nd.target], Reducer),
                      node_meta=lambda nd: (tuple(nd.meta["tensor_meta"].shape[1:]), nd.meta["tensor_meta"].dtype))
    ir = graphs.GraphIR("traced_spring", *six)
    assert [m["op"] for m in ir.map_operations] == ["sub", "norm", "sub", "mul", "mul", "truediv", "reducer"]
    ext = merged_gen_gpu.build_extension(ir, ("float32", "float64"))

    class Eqn(nn.Module):           # the shape of the reference's compiled module: a graph with one call_module node
        def __init__(self):
            super().__init__()
            self.fused = gm
            self.jit_engine = type("E", (), {})()
            g = torch.fx.Graph()
            args = [g.placeholder(nm) for nm in ("L", "k", "p")]
            g.output(g.call_module("fused", tuple(args)))
            self.jit_engine.graph = g

    eqn = Eqn()
    want = gm(L, k, p)[0]
    node_name = [nd.name for nd in eqn.jit_engine.graph.nodes if nd.op == "call_module"][0]
    assert dynamic_replace_submodule(eqn, ext, node_name)
    wrapper = getattr(eqn, node_name)
    assert isinstance(wrapper, DynamicCudaWrapper)
    got = wrapper(L, k, p)[0]
    torch.cuda.synchronize()
    assert got.shape == want.shape and got.dtype == dt
    scale = float(want.abs().max())
    tol = 1e-12 if dt == torch.float64 else 1e-5
    assert float((got - want).abs().max()) <= tol * scale * 8      # 6 terms per row, magnitudes up to `scale`
