"""The operator the reference's runtime wrapper calls: ``ext.merged_spmv_launch(*args)``.

The reference JIT-builds one pybind11 torch extension per fused graph whose single function
``merged_spmv_launch`` (cuda_template/merged_binding_template.cu:73-80) takes, positionally
(codegen/merged_gen_binding.py:65-78): the non-gather value inputs, the gather value inputs, one int32
index tensor per selector target, ``row_end_offsets`` (leading 0 included), ``num_rows``,
``num_cols`` -- and returns a tuple of freshly allocated outputs (or None when the graph has none).
``GraphExtension`` is that object for this library: same function name, argument order, keyword
names, checks and return convention; behind it a ctypes call into the C ABI of
libflexspmv_b200.so (include/flexspmv.h) on torch's current CUDA stream.  PyTorch provides device
memory and the stream, nothing else.

Differences from the reference binding, all on the host side of the same contract:
  * outputs are ``torch.empty`` (the kernels write every element; the reference needs torch::zeros
    because it accumulates with atomicAdd), scratch comes from torch's caching allocator instead of a
    per-call cudaMalloc/cudaFree (cuda_template/merged_binding_template.cu:42-49);
  * the merge-path partition is planned once per (row_end_offsets tensor, version, stream) and cached;
  * int64 ``row_end_offsets`` are accepted as they are (the reference casts to int32);
  * an unsupported dtype raises (the reference prints to stderr and falls off the end of a non-void
    function, cuda_template/merged_binding_template.cu:65-68);
  * a kernel that gives up (a bounded device-side wait ran out, or the workspace was not planned for the
    problem) stores its status in a page-locked host int registered with the workspace: the next call on
    that workspace, or ``ext.check()``, raises FlexSpmvError.  The launch path itself never synchronises;
    FLEXSPMV_CHECK_STATUS=1 makes every call synchronise and check.  After such an error the outputs of the
    failed launch are undefined.

There is no CPU path: a missing library or a CPU tensor is an error.
"""
from __future__ import annotations

import ctypes
import os
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .graphs import GraphIR, dim_of, operator_signature

_PKG = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIB = os.path.join(_PKG, "lib", "libflexspmv_b200.so")

_SFX = {torch.float32: "f32", torch.float64: "f64", torch.int64: "i64"}


class Desc(ctypes.Structure):
    _fields_ = [("num_rows", ctypes.c_int64), ("num_edges", ctypes.c_int64), ("num_vertices", ctypes.c_int64),
                ("offset_bits", ctypes.c_int32), ("tile_items", ctypes.c_int32), ("max_ctas", ctypes.c_int32),
                ("reserved", ctypes.c_int32)]


class GraphInfo(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in
                ("num_values", "num_indices", "num_outputs", "has_reducer", "value_bytes", "default_tile_items",
                 "block_threads", "items_per_thread", "stages", "smem_bytes", "acc_dim", "reserved")]


class FlexSpmvError(RuntimeError):
    pass


_libs: Dict[str, ctypes.CDLL] = {}


def load_library(path: Optional[str] = None) -> ctypes.CDLL:
    """dlopen the C-ABI library; raises when it is missing (no fallback of any kind)."""
    path = os.path.abspath(path or os.environ.get("FLEXSPMV_LIB", DEFAULT_LIB))
    if path not in _libs:
        if not os.path.exists(path):
            raise FlexSpmvError(f"{path} not found: build it with `python -m flexspmv_b200.build` "
                                "(there is no CPU or eager fallback)")
        lib = ctypes.CDLL(path)
        lib.flexspmv_error_string.restype = ctypes.c_char_p
        lib.flexspmv_error_string.argtypes = [ctypes.c_int]
        _libs[path] = lib
    return _libs[path]


def check(lib, status: int, what: str):
    if status != 0:
        raise FlexSpmvError(f"{what} failed: {lib.flexspmv_error_string(status).decode()} (status {status})")


_CHECK_EVERY_CALL = os.environ.get("FLEXSPMV_CHECK_STATUS", "0") == "1"


class _Plan:
    """One planned workspace: the scratch tensor, its size, the tensors whose addresses it depends on, and
    the page-locked int the kernels copy their error status to."""
    __slots__ = ("ws", "nbytes", "keep", "flag", "_flag_view")

    def __init__(self, ws, nbytes, keep):
        self.ws, self.nbytes, self.keep = ws, nbytes, keep
        self.flag = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._flag_view = self.flag.numpy()

    def status(self) -> int:
        return int(self._flag_view[0])


def _raise_if_failed(lib, plan: "_Plan", what: str):
    st = plan.status()
    if st != 0:
        raise FlexSpmvError(f"{what}: an earlier launch on this workspace failed on the device: "
                            f"{lib.flexspmv_error_string(st).decode()} (status {st}); its outputs are undefined")


def _stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class _Symbols:
    def __init__(self, lib, sym: str):
        def fn(name):
            try:
                f = getattr(lib, f"flexspmv_{sym}_{name}")
            except AttributeError as e:
                raise FlexSpmvError(f"library has no graph '{sym}' (symbol flexspmv_{sym}_{name})") from e
            f.restype = ctypes.c_int
            return f
        self.info, self.workspace_bytes, self.plan = fn("info"), fn("workspace_bytes"), fn("plan")
        self.plan_windows = fn("plan_windows")
        self.launch, self.device_status = fn("launch"), fn("device_status")
        gi = GraphInfo()
        check(lib, self.info(ctypes.byref(gi)), f"{sym}_info")
        self.graph_info = gi


class GraphExtension:
    """Drop-in for the module object ``torch.utils.cpp_extension.load`` returns in the reference flow
    (test_full/easier_full.py:359-373): exposes ``merged_spmv_launch``."""

    PLAN_CACHE_ENTRIES = 8

    def __init__(self, ir: GraphIR, lib_path: Optional[str] = None, symbol_prefix: Optional[str] = None,
                 tile_items: int = 0, max_ctas: int = 0, gather_windows: Optional[bool] = None,
                 random_gather: Optional[bool] = None):
        """``random_gather``: run the kernel for matrices whose columns have no locality (include/flexspmv.h,
        FLEXSPMV_FLAG_RANDOM_GATHER), for graphs built with it.  None = decide per matrix the first time it is
        planned, from a sample of its index array (one device-to-host read, at plan time only): the flag is set
        when 32 consecutive edges gather from more than 16 different cache lines on average.  The environment
        variable FLEXSPMV_RANDOM_GATHER=0/1 overrides None.

        ``gather_windows``: plan column segments per tile so that the kernel gathers from shared memory
        (include/flexspmv.h, FLEXSPMV_FLAG_GATHER_WINDOWS), for graphs that support it; None = off unless the
        environment variable FLEXSPMV_GATHER_WINDOWS is 1.  Costs 2 bytes of workspace per edge and a longer
        first call per matrix; results are bit-identical for equal tile size and CTA count.  Measured on B200:
        faster on small stencil matrices that are latency-bound (2-D Poisson 512^2: 14.4 us against 16.5 us per
        launch), slower on large ones
        (3-D Poisson: 62 % against 71 % of the HBM peak -- the kernel is bound by shared-memory / L1 data-pipe
        wavefronts there, and a gather from shared memory costs more of them than an L1-cached global gather)."""
        self.ir = ir
        if gather_windows is None:
            gather_windows = os.environ.get("FLEXSPMV_GATHER_WINDOWS", "0") == "1"
        self.gather_windows = bool(gather_windows)
        if random_gather is None and os.environ.get("FLEXSPMV_RANDOM_GATHER") in ("0", "1"):
            random_gather = os.environ["FLEXSPMV_RANDOM_GATHER"] == "1"
        self.random_gather = random_gather
        self._locality: Dict[tuple, bool] = {}
        edge_sel = [s_ for s_ in ir.selector_register if s_.get("selector") == 1 and not s_.get("row_identity")]
        self._gather_dim = dim_of(edge_sel[0]["shape"]) if edge_sel else 1
        self.lib = load_library(lib_path)
        self._lib_path = lib_path
        self.prefix = symbol_prefix or ir.name
        self.tile_items, self.max_ctas = int(tile_items), int(max_ctas)
        self.non_gather, self.gathers, self.index_names = operator_signature(ir)
        self.value_names = self.non_gather + self.gathers
        self.arg_names = self.value_names + [n + "_idx" for n in self.index_names] + \
            ["row_end_offsets", "num_rows", "num_cols"]
        self._syms: Dict[str, _Symbols] = {}
        self._plans: "OrderedDict[tuple, tuple]" = OrderedDict()
        self.launches = 0    # kernels this object enqueued (plan kernels included)

    # -- helpers ----------------------------------------------------------------------------------
    def symbols(self, dtype: torch.dtype) -> _Symbols:
        if dtype not in _SFX:
            raise FlexSpmvError(f"Unsupported dtype for ValueT: {dtype}. Use float32, float64 or int64.")
        sfx = _SFX[dtype]
        if sfx not in self._syms:
            self._syms[sfx] = _Symbols(self.lib, f"{self.prefix}_{sfx}")
        return self._syms[sfx]

    def _bind(self, args, kwargs) -> list:
        if len(args) > len(self.arg_names):
            raise TypeError(f"merged_spmv_launch() takes {len(self.arg_names)} arguments ({len(args)} given)")
        vals = list(args)
        for n in self.arg_names[len(args):]:
            if n not in kwargs:
                raise TypeError(f"merged_spmv_launch() missing argument '{n}'")
            vals.append(kwargs[n])
        extra = set(kwargs) - set(self.arg_names[len(args):])
        if extra:
            raise TypeError(f"merged_spmv_launch() got unexpected keyword arguments {sorted(extra)}")
        return vals

    def _looks_random(self, idx: torch.Tensor, record_bytes: int) -> bool:
        """Whether 32 consecutive edges of a sample from the middle of the index array gather from more than 16
        different 128-byte cache lines on average.  Small matrices never qualify: they are latency-bound and the
        staged kernel serves them."""
        n = idx.numel()
        if n < (1 << 20):
            return False
        key = (idx.data_ptr(), idx._version, n)
        hit = self._locality.get(key)
        if hit is None:
            m = min(n, 1 << 18) // 32 * 32
            start = (n - m) // 2 // 32 * 32
            lines = (idx[start:start + m].view(-1, 32).long() * record_bytes) >> 7
            lines = lines.sort(dim=1).values
            distinct = 1 + (lines[:, 1:] != lines[:, :-1]).sum(dim=1)
            hit = bool(float(distinct.float().mean().item()) > 16.0)
            if len(self._locality) > 64:
                self._locality.clear()
            self._locality[key] = hit
        return hit

    def _flags(self, syms: _Symbols, values=(), indices=()) -> int:
        flags = 1 if (self.gather_windows and (syms.graph_info.reserved & 1)) else 0
        if (syms.graph_info.reserved & 2) and self.random_gather is not False and len(indices):
            if self.random_gather or self._looks_random(indices[0], self._gather_dim * values[0].element_size()):
                flags = 2
        return flags

    def _desc(self, syms: _Symbols, values, row_end_offsets, num_rows: int, num_edges: int, num_cols: int,
              indices=()) -> Desc:
        has_red = self.ir.has_reducer
        flags = self._flags(syms, values, indices)
        if flags & 1:      # the windows are bounded by the gathered array's length: take it from the tensor itself
            num_cols = int(values[len(self.non_gather)].shape[0])
        return Desc(num_rows if has_red else 0, num_edges, num_cols,
                    64 if (has_red and row_end_offsets.dtype == torch.int64) else 32,
                    self.tile_items, self.max_ctas, flags)

    def _workspace(self, syms: _Symbols, desc: Desc, ro: Optional[torch.Tensor], device,
                   indices: Sequence[torch.Tensor] = ()) -> "_Plan":
        # a workspace holds per-launch state (ticket, carries): launches that may overlap on the GPU must not
        # share one, so the plan is cached per stream as well as per matrix
        key = (id(syms), desc.num_rows, desc.num_edges, desc.offset_bits, desc.tile_items, desc.max_ctas, desc.reserved,
               (ro.data_ptr(), ro._version) if ro is not None else None, device.index,
               torch.cuda.current_stream(device).cuda_stream,
               tuple((t.data_ptr(), t._version) for t in indices) if (desc.reserved & 1) else None)
        hit = self._plans.get(key)
        if hit is not None:
            self._plans.move_to_end(key)
            return hit
        nbytes = ctypes.c_size_t()
        check(self.lib, syms.workspace_bytes(ctypes.byref(desc), ctypes.byref(nbytes)), "workspace_bytes")
        ws = torch.empty(nbytes.value, dtype=torch.uint8, device=device)
        check(self.lib, syms.plan(ctypes.byref(desc), ctypes.c_void_p(ro.data_ptr() if ro is not None else 0),
                                  ctypes.c_void_p(ws.data_ptr()), ctypes.c_size_t(nbytes.value), _stream_ptr()),
              "plan")
        if desc.reserved & 1:      # gather windows: the second planning step reads the index array
            ip = (ctypes.c_void_p * max(len(indices), 1))(*[t.data_ptr() for t in indices])
            check(self.lib, syms.plan_windows(ctypes.byref(desc), ip, ctypes.c_void_p(ws.data_ptr()),
                                              ctypes.c_size_t(nbytes.value), _stream_ptr()), "plan_windows")
            self.launches += 2
        self.launches += 2 if ro is not None else 1
        # keep the row-offset tensor alive so its address cannot be recycled under a cached plan
        plan = _Plan(ws, nbytes.value, (ro, tuple(indices) if (desc.reserved & 1) else None))
        check(self.lib, self.lib.flexspmv_workspace_status_mirror(ctypes.c_void_p(ws.data_ptr()),
                                                                  ctypes.c_void_p(plan.flag.data_ptr()), _stream_ptr()),
              "workspace_status_mirror")
        self.launches += 1
        self._plans[key] = plan
        while len(self._plans) > self.PLAN_CACHE_ENTRIES:
            self._plans.popitem(last=False)
        return plan

    # -- the operator --------------------------------------------------------------------------------
    def merged_spmv_launch(self, *args, **kwargs):
        a = self._bind(args, kwargs)
        nv, ni = len(self.value_names), len(self.index_names)
        values: List[torch.Tensor] = a[:nv]
        indices: List[torch.Tensor] = a[nv:nv + ni]
        row_end_offsets, num_rows, num_cols = a[nv + ni], int(a[nv + ni + 1]), int(a[nv + ni + 2])
        for n, t in zip(self.arg_names, values + indices + [row_end_offsets]):
            if not isinstance(t, torch.Tensor):
                raise TypeError(f"{n} must be a torch.Tensor")
            if not t.is_cuda:
                raise FlexSpmvError(f"{n} must be a CUDA tensor")
            if not t.is_contiguous():
                raise FlexSpmvError(f"{n} must be contiguous")
        dispatch = values[0]
        dt = dispatch.dtype
        syms = self.symbols(dt)
        for n, t in zip(self.value_names, values):
            if t.dtype != dt:
                raise FlexSpmvError(f"{n} dtype mismatch")
        for n, t in zip(self.index_names, indices):
            if t.dtype != torch.int32:
                raise FlexSpmvError(f"{n}_idx dtype mismatch")
        ne = int(indices[0].numel()) if indices else num_cols
        if ne <= 0:
            raise FlexSpmvError("selector index must be non-empty")
        has_red = self.ir.has_reducer
        if has_red:
            if row_end_offsets.dtype not in (torch.int32, torch.int64):
                raise FlexSpmvError("row_end_offsets dtype mismatch")
            if row_end_offsets.numel() != num_rows + 1:
                raise FlexSpmvError("row_end_offsets must have length num_rows + 1")
        device = dispatch.device
        desc = self._desc(syms, values, row_end_offsets, num_rows, ne, num_cols, indices)
        outputs: List[torch.Tensor] = []
        for o in self.ir.outputs:
            d = dim_of(o["shape"])
            tgt = str(o["target"])
            if tgt == "reducer":
                shape = (num_rows,) if d == 1 else (num_rows, d)
            elif "sum" in tgt:
                shape = (d,)
            else:
                shape = (ne,) if d == 1 else (ne, d)
            outputs.append(torch.empty(shape, dtype=dt, device=device))
        with torch.cuda.device(device):
            plan = self._workspace(syms, desc, row_end_offsets if has_red else None, device, indices)
            _raise_if_failed(self.lib, plan, "merged_spmv_launch")
            vp = (ctypes.c_void_p * max(nv, 1))(*[t.data_ptr() for t in values])
            ip = (ctypes.c_void_p * max(ni, 1))(*[t.data_ptr() for t in indices])
            op = (ctypes.c_void_p * max(len(outputs), 1))(*[t.data_ptr() for t in outputs])
            st = syms.launch(ctypes.byref(desc), vp, ip,
                             ctypes.c_void_p(row_end_offsets.data_ptr() if has_red else 0), op,
                             ctypes.c_void_p(plan.ws.data_ptr()), ctypes.c_size_t(plan.nbytes), _stream_ptr())
        check(self.lib, st, "merged_spmv_launch")
        self.launches += 1
        if _CHECK_EVERY_CALL:
            self.check()
        if not outputs:
            return None
        return tuple(outputs)

    __call__ = merged_spmv_launch

    def launch_into(self, values: Sequence[torch.Tensor], indices: Sequence[torch.Tensor],
                    row_end_offsets: Optional[torch.Tensor], outputs: Sequence[torch.Tensor],
                    num_rows: int, num_edges: int, num_cols: int = 0) -> None:
        """Same fused pass as ``merged_spmv_launch`` but into caller-provided output tensors (any
        tensor or slice whose storage is large enough; e.g. the owned part of the next iteration's
        vector).  No allocation, no checks beyond the C ABI's own; one kernel launch."""
        dt = values[0].dtype
        syms = self.symbols(dt)
        has_red = self.ir.has_reducer
        device = values[0].device
        desc = self._desc(syms, values, row_end_offsets, num_rows, num_edges, num_cols, indices)
        with torch.cuda.device(device):
            plan = self._workspace(syms, desc, row_end_offsets if has_red else None, device, indices)
            _raise_if_failed(self.lib, plan, "launch_into")
            vp = (ctypes.c_void_p * max(len(values), 1))(*[t.data_ptr() for t in values])
            ip = (ctypes.c_void_p * max(len(indices), 1))(*[t.data_ptr() for t in indices])
            op = (ctypes.c_void_p * max(len(outputs), 1))(*[t.data_ptr() for t in outputs])
            st = syms.launch(ctypes.byref(desc), vp, ip,
                             ctypes.c_void_p(row_end_offsets.data_ptr() if has_red else 0), op,
                             ctypes.c_void_p(plan.ws.data_ptr()), ctypes.c_size_t(plan.nbytes), _stream_ptr())
        check(self.lib, st, "launch_into")
        self.launches += 1
        if _CHECK_EVERY_CALL:
            self.check()

    def prepare(self, values: Sequence[torch.Tensor], indices: Sequence[torch.Tensor],
                row_end_offsets: Optional[torch.Tensor], outputs: Sequence[torch.Tensor],
                num_rows: int, num_edges: int, num_cols: int = 0) -> "PreparedLaunch":
        """Binds one fixed set of tensors once (plan, workspace, C argument arrays) so that every later
        ``launch()`` is a single foreign call on the current stream: the form for time-stepping loops, where
        the reference wrapper re-marshals every argument on every call
        (python_wrapper/dynamic_replace_submodule.py:147-199).  The row offsets must not change while the
        object is in use; the value / index / output tensors may be rewritten in place."""
        dt = values[0].dtype
        syms = self.symbols(dt)
        has_red = self.ir.has_reducer
        device = values[0].device
        desc = self._desc(syms, values, row_end_offsets, num_rows, num_edges, num_cols, indices)
        with torch.cuda.device(device):
            plan = self._workspace(syms, desc, row_end_offsets if has_red else None, device, indices)
        return PreparedLaunch(self, syms, desc, list(values), list(indices), row_end_offsets if has_red else None,
                              list(outputs), plan)

    def device_status(self, dtype: torch.dtype, row_end_offsets: Optional[torch.Tensor] = None) -> int:
        """Reads back the status word of the most recently used workspace (synchronises)."""
        if not self._plans:
            return 0
        ws = next(reversed(self._plans.values())).ws
        out = torch.zeros(1, dtype=torch.int32, device=ws.device)
        syms = self.symbols(dtype)
        with torch.cuda.device(ws.device):
            check(self.lib, syms.device_status(ctypes.c_void_p(ws.data_ptr()), ctypes.c_void_p(out.data_ptr()), _stream_ptr()),
                  "device_status")
        return int(out.item())

    def check(self) -> None:
        """Waits for the work enqueued so far on every device this object planned for, then raises
        FlexSpmvError if a kernel gave up on any of its cached workspaces (a bounded wait ran out, or a
        launch met a workspace that was not planned for its problem).  Call it after a timed region or a
        time-stepping loop; the launch path itself only looks at the host-side copy of the status."""
        plans = list(self._plans.values())
        for dev in {p.ws.device for p in plans}:
            torch.cuda.synchronize(dev)
        for p in plans:
            _raise_if_failed(self.lib, p, "check")


class PreparedLaunch:
    """One graph bound to one set of device tensors (see ``GraphExtension.prepare``)."""

    def __init__(self, ext: GraphExtension, syms: _Symbols, desc: Desc, values, indices, ro, outputs, plan: _Plan):
        self.ext, self._syms, self._desc = ext, syms, desc
        ws, ws_bytes = plan.ws, plan.nbytes
        self._plan = plan
        self._keep = (values, indices, ro, outputs, ws)       # the raw pointers below borrow these tensors
        self._device = ws.device.index
        self._planned = torch.cuda.Event()                    # the plan kernels were enqueued on this stream
        self._planned.record(torch.cuda.current_stream(ws.device))
        self._ordered = {torch.cuda.current_stream(ws.device).cuda_stream}
        vp = (ctypes.c_void_p * max(len(values), 1))(*[t.data_ptr() for t in values])
        ip = (ctypes.c_void_p * max(len(indices), 1))(*[t.data_ptr() for t in indices])
        op = (ctypes.c_void_p * max(len(outputs), 1))(*[t.data_ptr() for t in outputs])
        self._args = (ctypes.byref(desc), vp, ip, ctypes.c_void_p(ro.data_ptr() if ro is not None else 0), op,
                      ctypes.c_void_p(ws.data_ptr()), ctypes.c_size_t(ws_bytes))
        self._fn = syms.launch

    def launch(self) -> None:
        """Enqueues the fused pass on the current stream of the tensors' device.  The workspace carries
        per-launch state, so launches of one prepared object must be stream-ordered with one another:
        launching from a second stream needs a second prepared object."""
        if torch.cuda.current_device() != self._device:
            with torch.cuda.device(self._device):
                return self.launch()
        if self._plan._flag_view[0]:
            _raise_if_failed(self.ext.lib, self._plan, "launch")
        stream = torch.cuda.current_stream()
        if stream.cuda_stream not in self._ordered:           # first use on another stream: after the plan
            if torch.cuda.is_current_stream_capturing():
                # an event recorded outside a capture cannot be waited on inside it
                raise FlexSpmvError("first launch of a prepared object on a stream that is being captured: launch it "
                                    "once on that stream before the capture begins")
            stream.wait_event(self._planned)
            self._ordered.add(stream.cuda_stream)
        st = self._fn(*self._args, ctypes.c_void_p(stream.cuda_stream))
        if st != 0:
            check(self.ext.lib, st, "launch")
        self.ext.launches += 1
        if _CHECK_EVERY_CALL:
            self.ext.check()

    __call__ = launch


def load_builtin(name: str, **kw) -> GraphExtension:
    """Extension object for one of the graphs compiled into libflexspmv_b200.so."""
    from .graphs import ALL_GRAPHS
    return GraphExtension(ALL_GRAPHS[name](), **kw)
