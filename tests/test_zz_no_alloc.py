"""The allocation-free entry point ``flexspmv_spmv_f64_launch_static``.

It exists for hosts of the library that are not allowed to allocate device memory while they run (a
pipeline whose memory was fixed at start-up, a plug-in that only receives pointers, a real-time loop
that may not take the allocator's locks): the kernels' scratch lives in a 2 MiB device array compiled
into the library instead of a caller-provided workspace.  The test calls it through the C ABI twice in
a row, on two different problems (the array still holds the first call's contents during the second),
and requires the result of each call to be bit-identical to the workspace-based entry points, which
run the same deterministic kernels.  It also checks that an oversized problem is refused.

Collected last on purpose (file name), and independent of every other test: it passes alone in a fresh
process and after the rest of the suite.
"""
import ctypes

import numpy as np
import pytest
import torch

from flexspmv_b200 import graphs, problems
from flexspmv_b200.binding import Desc, load_library

pytestmark = pytest.mark.gpu

ERR_STATIC_SCRATCH = -8


def _device_problem(prob, offsets_dtype):
    dev = torch.device("cuda:0")
    vals = torch.from_numpy(prob.values["vals"]).to(dev)
    x = torch.from_numpy(prob.values["x"]).to(dev)
    cols = torch.from_numpy(prob.indices["selector"]).to(dev)
    ro = torch.from_numpy(prob.row_offsets.astype(offsets_dtype)).to(dev)
    return vals, x, cols, ro


def _ptrs(*tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _workspace_result(lib, desc, vals, x, cols, ro):
    nbytes = ctypes.c_size_t()
    assert lib.flexspmv_spmv_f64_workspace_bytes(ctypes.byref(desc), ctypes.byref(nbytes)) == 0
    ws = torch.empty(nbytes.value, dtype=torch.uint8, device=vals.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.flexspmv_spmv_f64_plan(ctypes.byref(desc), ctypes.c_void_p(ro.data_ptr()), ctypes.c_void_p(ws.data_ptr()),
                                      ctypes.c_size_t(nbytes.value), stream) == 0
    y = torch.full((desc.num_rows,), float("nan"), dtype=torch.float64, device=vals.device)
    assert lib.flexspmv_spmv_f64_launch(ctypes.byref(desc), _ptrs(vals, x), _ptrs(cols), ctypes.c_void_p(ro.data_ptr()),
                                        _ptrs(y), ctypes.c_void_p(ws.data_ptr()), ctypes.c_size_t(nbytes.value), stream) == 0
    torch.cuda.synchronize()
    return y


def _static_result(lib, desc, vals, x, cols, ro):
    y = torch.full((desc.num_rows,), float("nan"), dtype=torch.float64, device=vals.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = lib.flexspmv_spmv_f64_launch_static(ctypes.byref(desc), _ptrs(vals, x), _ptrs(cols),
                                             ctypes.c_void_p(ro.data_ptr()), _ptrs(y), stream)
    assert st == 0, lib.flexspmv_error_string(st).decode()
    # the error channel of this entry point: the status word of the built-in array
    status = torch.full((1,), 99, dtype=torch.int32, device=vals.device)
    assert lib.flexspmv_spmv_f64_static_device_status(ctypes.c_void_p(status.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return y


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    lib = load_library()
    lib.flexspmv_spmv_f64_launch_static.restype = ctypes.c_int
    lib.flexspmv_spmv_f64_static_device_status.restype = ctypes.c_int
    ir = graphs.spmv_graph()
    first = problems.random_problem(ir, 20000, 20000, 300000, seed=21, dtype=np.float64)   # long and empty rows
    second = problems.poisson2d(96)                                                         # short rows, other size
    for prob, offsets_dtype in ((first, np.int32), (second, np.int64)):
        vals, x, cols, ro = _device_problem(prob, offsets_dtype)
        desc = Desc(prob.num_rows, prob.nnz, prob.num_cols, 64 if offsets_dtype == np.int64 else 32, 0, 0, 0)
        expect = _workspace_result(lib, desc, vals, x, cols, ro)
        got = _static_result(lib, desc, vals, x, cols, ro)
        assert not torch.isnan(got).any()
        assert torch.equal(got, expect)
        flagged = Desc(prob.num_rows, prob.nnz, prob.num_cols, desc.offset_bits, 0, 0, 1)   # gather-window flag: ignored here
        assert torch.equal(_static_result(lib, flagged, vals, x, cols, ro), expect)


def test_static_scratch_entry_refuses_oversized_problems():
    lib = load_library()
    lib.flexspmv_spmv_f64_launch_static.restype = ctypes.c_int
    dummy = torch.zeros(16, dtype=torch.float64, device="cuda:0")
    desc = Desc(1 << 28, 1 << 30, 1 << 28, 64, 0, 0, 0)    # needs far more than 2 MiB of tile coordinates
    st = lib.flexspmv_spmv_f64_launch_static(ctypes.byref(desc), _ptrs(dummy, dummy), _ptrs(dummy),
                                             ctypes.c_void_p(dummy.data_ptr()), _ptrs(dummy), ctypes.c_void_p(0))
    assert st == ERR_STATIC_SCRATCH
    assert b"static scratch" in lib.flexspmv_error_string(st)
