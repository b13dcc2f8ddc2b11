"""Row-block partitioned SpMV across the GPUs of one node: one process per GPU, rows split into
nnz-balanced contiguous blocks, each rank holding its block as a local CSR whose column indices point
into a local vector laid out ``[halo_below | owned | halo_above]``, and a nearest-neighbour halo
exchange of the vector entries each iteration over NCCL (NVLink / NVSwitch) -- or gloo on CPU for the
index-logic tests.  The reference has no multi-GPU code of its own (its drivers only forward a
``--comm_backend`` flag to the third-party ``easier`` runtime: easier_spmv.py:142,
test_full/easier_full.py:46); the partition search is the same lower-bound family as its
MergePathSearch (include/merged_spmv_kernels.cuh:19-50).

Only matrices whose out-of-block columns fall inside the neighbouring blocks (banded / stencil
matrices, e.g. the 7-point Laplacian split into z-slabs) are supported: the exchange is two
send/recv pairs per rank, no gather lists.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch


def balanced_row_blocks(row_offsets: torch.Tensor, parts: int, snap: int = 1) -> torch.Tensor:
    """first_row[k] = lower_bound(row_offsets, k*nnz/parts) rounded to a multiple of ``snap`` rows;
    torch restatement used on CPU tensors (tests, gloo ranks).  On CUDA tensors the C-ABI kernel
    ``flexspmv_row_blocks`` is used."""
    n = row_offsets.numel() - 1
    if row_offsets.is_cuda:
        from .binding import check, load_library
        lib = load_library()
        out = torch.empty(parts + 1, dtype=torch.int64, device=row_offsets.device)
        bits = 64 if row_offsets.dtype == torch.int64 else 32
        with torch.cuda.device(row_offsets.device):
            st = lib.flexspmv_row_blocks(ctypes.c_void_p(row_offsets.data_ptr()), bits, ctypes.c_int64(n), parts,
                                         ctypes.c_int64(snap), ctypes.c_void_p(out.data_ptr()),
                                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        check(lib, st, "flexspmv_row_blocks")
        return out
    ro = row_offsets.to(torch.int64)
    nnz = int(ro[-1])
    first = [0]
    for k in range(1, parts):
        target = (nnz * k) // parts
        lo = int(torch.searchsorted(ro, torch.tensor([target], dtype=torch.int64), right=False)[0])
        if snap > 1:
            lo = ((lo + snap // 2) // snap) * snap
        lo = min(lo, n)
        lo = max(lo, first[-1])
        first.append(lo)
    first.append(n)
    return torch.tensor(first, dtype=torch.int64)


@dataclass
class HaloPlan:
    """Index logic of one rank's block (pure integers; identical on CPU and GPU)."""
    rank: int
    world: int
    row_begin: int
    row_end: int
    halo_lo: int      # entries needed from the block below (global columns [row_begin-halo_lo, row_begin))
    halo_hi: int      # entries needed from the block above (global columns [row_end, row_end+halo_hi))
    send_lo: int      # entries the rank below needs from the head of this block
    send_hi: int      # entries the rank above needs from the tail of this block

    @property
    def rows(self) -> int:
        return self.row_end - self.row_begin

    @property
    def local_len(self) -> int:
        return self.halo_lo + self.rows + self.halo_hi

    @property
    def col_shift(self) -> int:
        """global column - col_shift = index into the local vector"""
        return self.row_begin - self.halo_lo


class _CHaloPlan(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("row_begin", "row_end", "halo_lo", "halo_hi", "send_lo", "send_hi")]


def make_halo_plans(first_row: List[int], min_col: List[int], max_col: List[int]) -> List[HaloPlan]:
    """first_row: world+1 block boundaries; min_col/max_col: smallest / largest global column
    referenced by each block's rows (for an empty block pass row_begin / row_begin-1).  The integer logic
    is the library's host-only ``flexspmv_halo_plan``."""
    from .binding import check, load_library
    world = len(first_row) - 1
    lib = load_library()
    arr = lambda v: (ctypes.c_int64 * len(v))(*[int(x) for x in v])
    out = (_CHaloPlan * world)()
    lib.flexspmv_halo_plan.restype = ctypes.c_int
    st = lib.flexspmv_halo_plan(arr(first_row), arr(min_col), arr(max_col), ctypes.c_int32(world), out)
    if st == -4:     # FLEXSPMV_ERR_TOO_LARGE
        raise NotImplementedError("halo reaches beyond the neighbouring block (matrix is not banded enough)")
    check(lib, st, "halo_plan")
    return [HaloPlan(r, world, p.row_begin, p.row_end, p.halo_lo, p.halo_hi, p.send_lo, p.send_hi)
            for r, p in enumerate(out)]


def exchange_halos(x_local: torch.Tensor, plan: HaloPlan, group=None) -> None:
    """One halo exchange of the local vector (in place): the head / tail of the owned part go to the
    neighbours' halo regions.  NCCL send/recv pairs batched in one group (or gloo on CPU)."""
    for w in start_halo_exchange(x_local, plan, group):
        w.wait()


def start_halo_exchange(x_local: torch.Tensor, plan: HaloPlan, group=None) -> list:
    """Starts the exchange and returns the outstanding requests (``wait()`` makes the current stream
    wait for them), so that work which does not touch the halos can be enqueued in between."""
    import torch.distributed as dist
    if plan.world == 1:
        return []
    lo, rows = plan.halo_lo, plan.rows
    owned = x_local[lo:lo + rows]
    ops = []
    if plan.rank > 0:
        if plan.send_lo:
            ops.append(dist.P2POp(dist.isend, owned[:plan.send_lo], plan.rank - 1, group))
        if plan.halo_lo:
            ops.append(dist.P2POp(dist.irecv, x_local[:lo], plan.rank - 1, group))
    if plan.rank < plan.world - 1:
        if plan.send_hi:
            ops.append(dist.P2POp(dist.isend, owned[rows - plan.send_hi:], plan.rank + 1, group))
        if plan.halo_hi:
            ops.append(dist.P2POp(dist.irecv, x_local[lo + rows:], plan.rank + 1, group))
    return dist.batch_isend_irecv(ops) if ops else []


# ----------------------------------------------------------------------------------------------
# config 4 built per rank on the device
# ----------------------------------------------------------------------------------------------

def poisson3d_planes_device(n: int, z_begin: int, z_end: int, device, value_dtype=torch.float64,
                            offset_dtype=torch.int64, col_shift: int = 0, chunk_planes: int = 16):
    """CSR of the rows of z-planes [z_begin, z_end) of the 7-point Laplacian on an n^3 grid (x
    fastest, Dirichlet, 6 / -1), built on ``device`` in chunks of planes.  Column indices are global
    minus ``col_shift``.  Same matrix as problems.poisson3d (tests compare them)."""
    n2 = n * n
    rows = (z_end - z_begin) * n2
    counts = torch.empty(rows, dtype=torch.int64, device=device)
    cols_parts, vals_parts = [], []
    diag = torch.tensor([-1.0, -1.0, -1.0, 6.0, -1.0, -1.0, -1.0], dtype=value_dtype, device=device)
    steps = torch.tensor([-n2, -n, -1, 0, 1, n, n2], dtype=torch.int64, device=device)
    for zb in range(z_begin, z_end, chunk_planes):
        ze = min(z_end, zb + chunk_planes)
        idx = torch.arange(zb * n2, ze * n2, dtype=torch.int64, device=device)
        k = idx // n2
        r = idx - k * n2
        j = r // n
        i = r - j * n
        valid = torch.stack([k > 0, j > 0, i > 0, torch.ones_like(i, dtype=torch.bool), i < n - 1, j < n - 1, k < n - 1], dim=1)
        cand = idx[:, None] + steps[None, :]
        counts[(zb - z_begin) * n2:(ze - z_begin) * n2] = valid.sum(dim=1)
        cols_parts.append((cand[valid] - col_shift).to(torch.int32))
        vals_parts.append(diag.expand(idx.numel(), 7)[valid].contiguous())
        del idx, k, r, j, i, valid, cand
    ro = torch.zeros(rows + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, dim=0, out=ro[1:])
    del counts
    cols = torch.cat(cols_parts) if len(cols_parts) > 1 else cols_parts[0]
    del cols_parts
    vals = torch.cat(vals_parts) if len(vals_parts) > 1 else vals_parts[0]
    del vals_parts
    return ro.to(offset_dtype), cols, vals


def poisson3d_row_offsets(n: int, device, offset_dtype=torch.int64, chunk_planes: int = 64) -> torch.Tensor:
    """Row offsets (leading 0) of the whole n^3 7-point Laplacian, from the closed-form row lengths
    7 - (number of grid faces the point touches); used to choose the slab boundaries."""
    n2 = n * n
    counts = torch.empty(n * n2, dtype=torch.int64, device=device)
    for zb in range(0, n, chunk_planes):
        ze = min(n, zb + chunk_planes)
        idx = torch.arange(zb * n2, ze * n2, dtype=torch.int64, device=device)
        k = idx // n2
        r = idx - k * n2
        j = r // n
        i = r - j * n
        c = 7 - (k == 0).to(torch.int64) - (k == n - 1).to(torch.int64) - (j == 0).to(torch.int64) \
            - (j == n - 1).to(torch.int64) - (i == 0).to(torch.int64) - (i == n - 1).to(torch.int64)
        counts[zb * n2:ze * n2] = c
    ro = torch.zeros(n * n2 + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, dim=0, out=ro[1:])
    return ro.to(offset_dtype)


def poisson3d_slab_bounds(n: int, world: int, device) -> List[int]:
    """z-plane boundaries of the nnz-balanced slabs: the row-block search (C-ABI kernel on CUDA, its
    torch restatement on CPU) on the global row offsets, snapped to whole planes (snap = n^2 rows)."""
    ro = poisson3d_row_offsets(n, device)
    first = balanced_row_blocks(ro, world, snap=n * n)
    return [int(v) // (n * n) for v in first.cpu().tolist()]


class PartitionedSpmv:
    """One rank's share of y = A x for a row-block partitioned banded matrix, iterated as
    x <- A x: the local vector is double-buffered ([halo_lo | owned | halo_hi] each) so an
    iteration is "exchange halos of the current buffer, fused SpMV into the owned part of the other
    buffer".

    With ``overlap`` the rows are split once into the few that read a halo (first / last rows of the block) and the
    interior, and an iteration becomes: one small launch over BOTH boundary row groups (their results are exactly
    what the neighbours need next) -> the send / receive of those results into the neighbours' halos of the next
    buffer, on NCCL's stream -> the interior launch on the compute stream, concurrently with the transfer.  The
    halos of iteration k + 1 thus travel while iteration k's interior is computed.  The interior launch leaves a
    few CTA slots free (``overlap_spare_ctas``): the kernel runs persistent CTAs over static tile runs, so a CTA
    that finds no free slot because a communication kernel sits on its SM would double the launch time."""

    def __init__(self, plan: HaloPlan, row_offsets: torch.Tensor, cols_local: torch.Tensor, vals: torch.Tensor,
                 x_owned: torch.Tensor, group=None, ext=None, overlap: Optional[bool] = None,
                 overlap_spare_ctas: int = 16):
        from .binding import load_builtin
        self.plan, self.group = plan, group
        self.ro, self.cols, self.vals = row_offsets, cols_local, vals
        self.ext = ext or load_builtin("spmv")
        dev = vals.device
        self.buf = [torch.zeros(plan.local_len, dtype=vals.dtype, device=dev) for _ in range(2)]
        self.cur = 0
        self.buf[0][plan.halo_lo:plan.halo_lo + plan.rows] = x_owned
        self.nnz = int(cols_local.numel())
        self.overlap = bool(overlap) and plan.world > 1
        self._prepared = {}
        self.graph, self.graph_error = None, None
        self._halos_valid = False        # overlap mode: the current buffer's halos already hold the neighbours' values
        if self.overlap:
            lo_rows, hi_rows = boundary_rows(row_offsets, cols_local, plan)
            if lo_rows + hi_rows >= plan.rows or lo_rows + hi_rows == 0:      # block too thin to have an interior
                self.overlap = False
        if self.overlap:
            from .binding import GraphExtension
            rows = plan.rows
            self.lo_rows, self.hi_rows = lo_rows, hi_rows
            # interior rows: views of the block's arrays
            self.interior = (lo_rows, rows - hi_rows) + sub_csr(row_offsets, cols_local, vals, lo_rows, rows - hi_rows)
            # both boundary row groups as ONE small CSR (lower group first), results into one scratch vector
            ro64 = row_offsets.to(torch.int64)
            e_lo, e_hi0 = int(ro64[lo_rows]), int(ro64[rows - hi_rows])
            ro_b = torch.cat([ro64[:lo_rows + 1], ro64[rows - hi_rows + 1:] - e_hi0 + e_lo]).to(row_offsets.dtype).contiguous()
            self.boundary = (ro_b, torch.cat([cols_local[:e_lo], cols_local[e_hi0:]]).contiguous(),
                             torch.cat([vals[:e_lo], vals[e_hi0:]]).contiguous())
            self.boundary_out = torch.empty(lo_rows + hi_rows, dtype=vals.dtype, device=dev)
            props = torch.cuda.get_device_properties(dev)
            info = self.ext.symbols(vals.dtype).graph_info
            resident = max(1, min(2048 // (info.block_threads + 32), (227 * 1024) // max(info.smem_bytes, 1)))
            self.ext_interior = GraphExtension(self.ext.ir, lib_path=self.ext._lib_path,
                                               max_ctas=max(1, props.multi_processor_count * resident - int(overlap_spare_ctas)),
                                               random_gather=False)

    def owned(self, which: Optional[int] = None) -> torch.Tensor:
        b = self.buf[self.cur if which is None else which]
        return b[self.plan.halo_lo:self.plan.halo_lo + self.plan.rows]

    def refresh_halos(self) -> None:
        """Exchanges the halos of the current buffer now (after the owned part was rewritten from outside)."""
        exchange_halos(self.buf[self.cur], self.plan, self.group)
        self._halos_valid = True

    def _prepared_launch(self, ext, key, values, indices, ro, outputs, rows, nnz):
        prepared = self._prepared.get(key)
        if prepared is None:       # bound once per ping-pong direction; later steps are one foreign call
            prepared = self._prepared[key] = ext.prepare(values, indices, ro, outputs, rows, nnz, self.plan.local_len)
        prepared.launch()

    def step(self) -> torch.Tensor:
        """One iteration: y = A_local x_local; y becomes the next iteration's owned vector."""
        plan = self.plan
        x = self.buf[self.cur]
        nxt = self.buf[1 - self.cur]
        y = self.owned(1 - self.cur)
        if not self.overlap:
            exchange_halos(x, plan, self.group)
            self._prepared_launch(self.ext, ("all", self.cur), [self.vals, x], [self.cols], self.ro, [y], plan.rows, self.nnz)
        else:
            if not self._halos_valid:
                self.refresh_halos()
            lo_rows, hi_rows, rows = self.lo_rows, self.hi_rows, plan.rows
            ro_b, cols_b, vals_b = self.boundary
            # (i) the rows that read a halo: the first / last rows of the block, one launch
            self._prepared_launch(self.ext, ("boundary", self.cur), [vals_b, x], [cols_b], ro_b, [self.boundary_out],
                                  lo_rows + hi_rows, int(cols_b.numel()))
            if lo_rows:
                y[:lo_rows].copy_(self.boundary_out[:lo_rows])
            if hi_rows:
                y[rows - hi_rows:].copy_(self.boundary_out[lo_rows:])
            # (ii) their results are the neighbours' halos of the next iteration: sent now, on NCCL's stream
            reqs = start_halo_exchange(nxt, plan, self.group)
            # (iii) the interior rows read no halo entry: computed while the transfer is in flight
            r0, r1, ro_i, cols_i, vals_i = self.interior
            self._prepared_launch(self.ext_interior, ("interior", self.cur), [vals_i, x], [cols_i], ro_i, [y[r0:r1]],
                                  r1 - r0, int(cols_i.numel()))
            for w in reqs:           # the next iteration's first launch waits for the halos, not this one's interior
                w.wait()
        self.cur = 1 - self.cur
        return y

    @property
    def launches_per_step(self) -> int:
        return 2 if self.overlap else 1

    def capture_pair(self) -> bool:
        """Captures two consecutive iterations (the buffers ping-pong, so two steps return to the same
        state) into one CUDA graph: halo send/recv and the fused launches replay without any host work
        between them.  At 8 GPUs an iteration is ~0.4 ms, the same order as the host-side cost of
        enqueueing the NCCL group from Python.  Plans must exist (run a step first).  Returns False
        and stays eager if the capture is refused."""
        if self.cur != 0:
            self.step()
        self.graph, self.graph_error = None, None
        try:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                # one eager pair on the capture stream first: a prepared launch orders its first use on a new
                # stream after its plan with an event wait, which is not allowed inside a capture
                self.step()
                self.step()
                side.synchronize()
                with torch.cuda.graph(g, stream=side):
                    self.step()
                    self.step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.graph = g
            return True
        except Exception as e:      # eager path keeps working; the reason is kept for the caller to report
            self.graph = None
            self.graph_error = repr(e)
            torch.cuda.synchronize()
            return False

    def step_pair(self) -> None:
        """Two iterations: one graph replay when captured, else two eager steps."""
        if getattr(self, "graph", None) is not None:
            self.graph.replay()
        else:
            self.step()
            self.step()


def boundary_rows(row_offsets: torch.Tensor, cols_local: torch.Tensor, plan: HaloPlan) -> Tuple[int, int]:
    """(number of leading rows that read the lower halo, number of trailing rows that read the upper
    halo) of a block whose columns index the local vector [halo_lo | owned | halo_hi]."""
    ro = row_offsets.to(torch.int64)
    lo_rows = hi_rows = 0
    if plan.halo_lo:
        e = torch.nonzero(cols_local < plan.halo_lo).flatten()
        if e.numel():
            lo_rows = int(torch.searchsorted(ro, e.max().reshape(1), right=True)[0])        # row of the last such edge, + 1
    if plan.halo_hi:
        e = torch.nonzero(cols_local >= plan.halo_lo + plan.rows).flatten()
        if e.numel():
            first_row = int(torch.searchsorted(ro, e.min().reshape(1), right=True)[0]) - 1
            hi_rows = plan.rows - first_row
    return lo_rows, hi_rows


def sub_csr(row_offsets: torch.Tensor, cols: torch.Tensor, vals: torch.Tensor, r0: int, r1: int):
    """CSR of rows [r0, r1) as (offsets starting at 0, column view, value view); views are copied only
    when their start is not 16-byte aligned (the kernels stage these arrays with bulk copies)."""
    e0, e1 = int(row_offsets[r0]), int(row_offsets[r1])
    ro = (row_offsets[r0:r1 + 1] - row_offsets[r0]).contiguous()
    c, v = cols[e0:e1], vals[e0:e1]
    if c.data_ptr() % 16:
        c = c.clone()
    if v.data_ptr() % 16:
        v = v.clone()
    return ro, c, v
