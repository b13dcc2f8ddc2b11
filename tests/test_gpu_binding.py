"""The generated torch-extension shim (``merged_binding.cu``, flexspmv_b200/codegen/merged_gen_binding.py) built the
way the reference's driver builds its own (``torch.utils.cpp_extension.load`` on the one generated source,
test_full/easier_full.py:359-373) and called as the runtime wrapper calls it: positionally and by keyword.  Results
are compared with the CPU oracle and, bit for bit, with the ctypes operator of the built-in library (same kernels,
same tile configuration)."""
import os
import shutil

import numpy as np
import pytest
import torch

from flexspmv_b200 import graphs, problems
from flexspmv_b200.binding import GraphExtension
from flexspmv_b200.codegen import merged_gen_binding
from oracle import ir_eval
from parity import assert_outputs_match

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _device_args(ir, prob, dt):
    dev = torch.device("cuda:0")
    non_gather, gathers, index_names = graphs.operator_signature(ir)
    vals = [torch.from_numpy(np.ascontiguousarray(prob.values[n].astype(dt))).to(dev) for n in non_gather + gathers]
    idxs = [torch.from_numpy(np.ascontiguousarray(prob.indices[n])).to(dev) for n in index_names]
    ro = torch.from_numpy(np.ascontiguousarray(prob.row_offsets)).to(dev)
    names = non_gather + gathers + [n + "_idx" for n in index_names] + ["row_end_offsets", "num_rows", "num_cols"]
    return vals, idxs, ro, names


@pytest.mark.parametrize("gname,dt,make", [
    ("spmv", "float64", lambda ir: problems.random_problem(ir, 12314, 12314, 123134, seed=3, dtype=np.float64)),
    ("spring_mass", "float32", lambda ir: problems.spring_mass(96)),
], ids=["spmv-f64", "spring_mass-f32"])
def test_generated_binding_builds_and_matches(gname, dt, make):
    if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("needs nvcc to build the generated extension")
    ir = graphs.ALL_GRAPHS[gname]()
    project_root = os.path.join(ROOT, "build", "jit", f"binding_{gname}_{dt}")
    os.makedirs(project_root, exist_ok=True)
    ext = merged_gen_binding.load_binding(ir, project_root, dtypes=(dt,))
    prob = make(ir)
    dtype = np.dtype(dt)
    vals, idxs, ro, names = _device_args(ir, prob, dtype)
    outs = ext.merged_spmv_launch(*vals, *idxs, ro, prob.num_rows, prob.num_cols)             # positional, as the wrapper calls it
    kw = dict(zip(names, vals + idxs + [ro, prob.num_rows, prob.num_cols]))
    outs_kw = ext.merged_spmv_launch(**kw)                                                     # the generated py::arg names
    torch.cuda.synchronize()
    assert isinstance(outs, tuple) and len(outs) == len(ir.outputs)
    ref, _, sums = ir_eval.run_graph(ir, prob, dtype, num_threads=8, want_abs_sums=True)
    assert_outputs_match(ir, [o.cpu().numpy() for o in outs], ref, sums, dtype, what=f"binding {gname}")
    same = GraphExtension(ir).merged_spmv_launch(*vals, *idxs, ro, prob.num_rows, prob.num_cols)
    torch.cuda.synchronize()
    for a, b, c in zip(outs, outs_kw, same):
        assert torch.equal(a, b) and torch.equal(a, c)
    assert ext.device_status() == 0
    # int64 row offsets are taken as they are; the plan cache must not serve the int32 plan for them
    outs64 = ext.merged_spmv_launch(*vals, *idxs, ro.long(), prob.num_rows, prob.num_cols)
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(outs, outs64))
    # the checks of the reference binding, and the dtype that is not compiled raises instead of falling through
    with pytest.raises(RuntimeError, match="CUDA device required"):
        ext.merged_spmv_launch(vals[0].cpu(), *vals[1:], *idxs, ro, prob.num_rows, prob.num_cols)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ext.merged_spmv_launch(*vals[:-1], vals[-1].cpu(), *idxs, ro, prob.num_rows, prob.num_cols)
    with pytest.raises(RuntimeError, match="dtype mismatch"):
        ext.merged_spmv_launch(*vals, *[i.long() for i in idxs], ro, prob.num_rows, prob.num_cols)
    other = torch.float32 if dt == "float64" else torch.float64
    with pytest.raises(RuntimeError, match="Unsupported dtype"):
        ext.merged_spmv_launch(*[v.to(other) for v in vals], *idxs, ro, prob.num_rows, prob.num_cols)
