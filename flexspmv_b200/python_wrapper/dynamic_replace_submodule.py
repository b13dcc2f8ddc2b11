"""Swaps a fused FX sub-module for the CUDA operator.  Same contract as the reference's
``dynamic_replace_submodule(compiled_eqn, ext, submodule_name)``
(python_wrapper/dynamic_replace_submodule.py:202-258): find the ``call_module`` node, collect the Selector
index tensors and the Reducer's row ids from the sub-module, turn the row ids into CSR offsets, and
install a wrapper whose ``__call__`` marshals the placeholders into the operator's positional order
(:180-193) and returns the outputs as a list.

What the reference's wrapper does on every call and this one does once: ``.contiguous()`` copies
(:147-149; here only non-contiguous arguments are copied), device moves of the index buffers, and the
int64 -> int32 cast of the row offsets (kept int64 when they do not fit int32: the kernels take both).
What the reference never checks and this one does once at construction: whether the Reducer's row ids are
sorted ascending (its ``_coo_rows_to_csr_ptr`` silently assumes it, :20-41).  Ids on the device that are not
sorted are sorted here, once, by the library's stable radix sort (``flexspmv_sort_rows``); the wrapper then
permutes the selector index arrays once and the per-edge value inputs on every call
(``flexspmv_permute_edges``), and scatters per-edge outputs back into the caller's edge order.

Selector / Reducer modules are recognised by duck typing (an ``idx`` tensor; a Reducer also has ``n``), so
the module works with ``easier``'s classes without importing them.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn


def coo_rows_to_csr_ptr(row_ids: torch.Tensor, num_rows: Optional[int] = None) -> torch.Tensor:
    """Sorted COO row ids -> CSR offsets with the leading 0 (int64).  CUDA ids are converted by the
    library's ``flexspmv_coo_rows_to_csr`` (one launch, checks that the ids are ascending and in range);
    ids on the host go through bincount + cumsum as in the reference (:20-41), with the same check."""
    if row_ids.dtype not in (torch.int32, torch.int64):
        row_ids = row_ids.to(torch.int64)
    if num_rows is None:
        if row_ids.numel() == 0:
            raise RuntimeError("row_ids is empty; cannot infer num_rows")
        num_rows = int(row_ids.max().item()) + 1
    if row_ids.is_cuda:
        import ctypes
        from ..binding import check, load_library
        lib = load_library()
        ids = row_ids.contiguous()
        crow = torch.empty(num_rows + 1, dtype=torch.int64, device=ids.device)
        status = torch.empty(1, dtype=torch.int32, device=ids.device)
        with torch.cuda.device(ids.device):
            lib.flexspmv_coo_rows_to_csr.restype = ctypes.c_int
            st = lib.flexspmv_coo_rows_to_csr(ctypes.c_void_p(ids.data_ptr()), 64 if ids.dtype == torch.int64 else 32,
                                              ctypes.c_int64(ids.numel()), ctypes.c_int64(num_rows),
                                              ctypes.c_void_p(crow.data_ptr()), 64, ctypes.c_void_p(status.data_ptr()),
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        check(lib, st, "coo_rows_to_csr")
        code = int(status.item())
        if code == -5:      # FLEXSPMV_ERR_BAD_CSR
            raise ValueError("Reducer row ids must be sorted ascending (edges stored CSR-by-row)")
        check(lib, code, "coo_rows_to_csr")
        return crow
    row_ids = row_ids.to(torch.int64)
    if row_ids.numel() > 1 and bool((row_ids[1:] < row_ids[:-1]).any()):
        raise ValueError("Reducer row ids must be sorted ascending (edges stored CSR-by-row)")
    counts = torch.bincount(row_ids, minlength=num_rows)
    crow = torch.zeros(num_rows + 1, dtype=torch.int64, device=row_ids.device)
    torch.cumsum(counts, dim=0, out=crow[1:])
    return crow


def sort_edges_by_row(row_ids: torch.Tensor, num_rows: int):
    """Stable sort of CUDA row ids on the device: returns (perm int32, CSR offsets int64) with
    ``row_ids[perm]`` ascending and equal ids in their input order."""
    import ctypes
    from ..binding import check, load_library
    lib = load_library()
    ids = row_ids.contiguous()
    if ids.dtype not in (torch.int32, torch.int64):
        ids = ids.to(torch.int64)
    n = ids.numel()
    nbytes = ctypes.c_size_t()
    lib.flexspmv_sort_rows_bytes.restype = ctypes.c_int
    lib.flexspmv_sort_rows.restype = ctypes.c_int
    check(lib, lib.flexspmv_sort_rows_bytes(ctypes.c_int64(n), ctypes.byref(nbytes)), "sort_rows_bytes")
    dev = ids.device
    scratch = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
    perm = torch.empty(n, dtype=torch.int32, device=dev)
    crow = torch.empty(num_rows + 1, dtype=torch.int64, device=dev)
    status = torch.empty(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        st = lib.flexspmv_sort_rows(ctypes.c_void_p(ids.data_ptr()), 64 if ids.dtype == torch.int64 else 32, ctypes.c_int64(n),
                                    ctypes.c_int64(num_rows), ctypes.c_void_p(perm.data_ptr()), ctypes.c_void_p(crow.data_ptr()), 64,
                                    ctypes.c_void_p(scratch.data_ptr()), ctypes.c_size_t(nbytes.value),
                                    ctypes.c_void_p(status.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    check(lib, st, "sort_rows")
    check(lib, int(status.item()), "sort_rows (row ids)")
    return perm, crow


def permute_edges(src: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    """dst[k] = src[perm[k]] along the first dimension (records of 4-byte multiples), by the library's kernel."""
    import ctypes
    from ..binding import check, load_library
    lib = load_library()
    src = src.contiguous()
    rec = src.element_size() * (src.numel() // max(src.shape[0], 1))
    dst = torch.empty_like(src)
    with torch.cuda.device(src.device):
        lib.flexspmv_permute_edges.restype = ctypes.c_int
        st = lib.flexspmv_permute_edges(ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(dst.data_ptr()), ctypes.c_void_p(perm.data_ptr()),
                                        ctypes.c_int64(src.shape[0]), ctypes.c_int32(rec),
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    check(lib, st, "permute_edges")
    return dst


def _is_selector(m) -> bool:
    return hasattr(m, "idx") and not hasattr(m, "n")


def _is_reducer(m) -> bool:
    return hasattr(m, "idx") and hasattr(m, "n")


class DynamicCudaWrapper(nn.Module):
    def __init__(self, ext, input_param_names: Sequence[str], non_gather_value_inputs: Sequence[str],
                 gather_value_inputs: Sequence[str], selector_idx_tensors: Sequence[torch.Tensor],
                 row_end_offsets: Optional[torch.Tensor], edge_perm: Optional[torch.Tensor] = None):
        """``edge_perm``: permutation that sorts the edges by row (None: they already are); the CSR offsets and
        kernels work in the sorted order."""
        super().__init__()
        self._ext = ext
        self._perm = edge_perm
        if edge_perm is not None:
            selector_idx_tensors = [permute_edges(t.to(edge_perm.device), edge_perm) for t in selector_idx_tensors]
        self._names = list(input_param_names)
        self._non_gather, self._gather = list(non_gather_value_inputs), list(gather_value_inputs)
        self._sel_names: List[str] = []
        for i, t in enumerate(selector_idx_tensors):
            t = t.contiguous()
            if t.dtype != torch.int32:
                if t.numel() and int(t.max()) >= 2 ** 31:
                    raise ValueError("selector indices beyond int32 are not supported")
                t = t.to(torch.int32)
            self.register_buffer(f"selector_{i}_idx", t, persistent=False)
            self._sel_names.append(f"selector_{i}_idx")
        if row_end_offsets is not None:
            ro = row_end_offsets.contiguous()
            if int(ro[-1]) < 2 ** 31 and ro.dtype != torch.int32:
                ro = ro.to(torch.int32)
        else:
            ro = None
        self.register_buffer("row_end_offsets", ro, persistent=False)
        self._moved_to = None

    def _buffers_on(self, device):
        if self._moved_to != device:
            for n in self._sel_names + (["row_end_offsets"] if self.row_end_offsets is not None else []):
                setattr(self, n, getattr(self, n).to(device))
            self._moved_to = device

    def __call__(self, *args):
        amap: Dict[str, torch.Tensor] = {n: (a if a.is_contiguous() else a.contiguous()) for n, a in zip(self._names, args)}
        device = next(iter(amap.values())).device
        self._buffers_on(device)
        ro = self.row_end_offsets
        gv = self._gather[0] if self._gather else self._non_gather[0]
        num_cols = int(amap[gv].shape[0])
        if ro is None:     # map-only graph: the operator still takes a (dummy) offsets tensor
            ro = torch.tensor([42], dtype=torch.int32, device=device)
            num_rows = num_cols
        else:
            num_rows = int(ro.numel() - 1)
        if self._perm is not None:      # per-edge inputs into the sorted edge order
            ne = int(self._perm.numel())
            for n in self._non_gather:
                if amap[n].dim() >= 1 and amap[n].shape[0] == ne:
                    amap[n] = permute_edges(amap[n], self._perm)
        call_args = [amap[n] for n in self._non_gather] + [amap[n] for n in self._gather] + \
                    [getattr(self, n) for n in self._sel_names] + [ro, num_rows, num_cols]
        outs = self._ext.merged_spmv_launch(*call_args)
        if outs is None:
            return []
        outs = list(outs) if isinstance(outs, tuple) else [outs]
        if self._perm is not None:      # per-edge outputs back into the caller's edge order
            ne = int(self._perm.numel())
            for i, o in enumerate(outs):
                if o.dim() >= 1 and o.shape[0] == ne and o.shape[0] != num_rows:
                    back = torch.empty_like(o)
                    back[self._perm.long()] = o
                    outs[i] = back
        return outs


def dynamic_replace_submodule(compiled_eqn: nn.Module, ext, submodule_name: str) -> bool:
    graph = compiled_eqn.jit_engine.graph
    for node in graph.nodes:
        if node.op != "call_module" or node.name != submodule_name:
            continue
        gm = compiled_eqn.get_submodule(node.target)
        names = [n.name for n in gm.graph.nodes if n.op == "placeholder"]
        selectors, reducer = [], None
        for qn, m in gm.named_modules():
            if qn == "":
                continue
            if _is_reducer(m):
                reducer = m
                break                      # the first Reducer's row ids define the CSR of the whole sub-module
            if _is_selector(m):
                selectors.append((qn, m))
        sel_q = {q for q, _ in selectors}
        gathers: List[str] = []
        for n in gm.graph.nodes:
            if n.op == "call_module" and n.target in sel_q:
                for a in n.args:
                    if hasattr(a, "op") and a.op == "placeholder" and a.name not in gathers:
                        gathers.append(a.name)
        ro, perm = None, None
        if reducer is not None:
            try:
                ro = coo_rows_to_csr_ptr(reducer.idx, int(reducer.n))
            except ValueError:
                if not reducer.idx.is_cuda:
                    raise
                perm, ro = sort_edges_by_row(reducer.idx, int(reducer.n))      # unsorted ids: sorted once, on the device
        wrapper = DynamicCudaWrapper(ext, names, [n for n in names if n not in gathers], gathers,
                                     [m.idx for _, m in selectors], ro, perm)
        setattr(compiled_eqn, submodule_name, wrapper)
        return True
    return False
