"""IR -> CUDA: turns the reference tracer's 6-tuple into one translation unit that plugs the fused
per-edge map into the hand-written sm_100a kernels (csrc/flex_tile_kernel.cuh for graphs with a
reduce-by-row, csrc/flex_edge_kernel.cuh for the aggregator / map-only flavour) and exports the five
C-ABI symbols of ``FLEXSPMV_DECLARE_GRAPH`` (include/flexspmv.h).

This is the counterpart of the reference's GPU emitter (codegen/merged_gen_gpu.py:17-465), which
string-substitutes selector / map / reducer snippets into CUB-derived templates.  The op vocabulary
and its meaning are the reference's (trace/graph_trace.py:229-276, codegen/merged_gen_core.py:122-236);
what differs is the target: instead of relying on C++ overload resolution over ``Tensor<ValueT,Dim>``
(data_struct_shared.cuh) the emitter resolves, per operation, which overload the reference code would
select (equal widths / broadcast / scalar on either side) and emits an explicitly named call from
csrc/flex_tensor.cuh.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

from ..graphs import GraphIR, dim_of, operator_signature

CTYPE = {"float32": ("float", "f32"), "float64": ("double", "f64"), "int64": ("long long", "i64")}
VBYTES = {"float32": 4, "float64": 8, "int64": 8}

_BIN = {"add": "Add", "sub": "Sub", "mul": "Mul", "pow": "Pow", "truediv": "Div", "lt": "Lt", "gt": "Gt"}
_SCALAR_FN = {"add": "vadd", "sub": "vsub", "mul": "vmul", "truediv": "vdiv"}


class Var:
    def __init__(self, kind: str, dim: int, expr: str):
        self.kind, self.dim, self.expr = kind, dim, expr   # kind: 'vec' | 'scalar'


def _lit(a) -> str:
    return f"V({repr(a)})"


def stage_values(ir: GraphIR) -> bool:
    """Whether the edge TENSORS (values, attributes) go through the bulk-copy stages like the index arrays and
    the row-end offsets, or are read straight from global memory with coalesced loads issued together with
    the gathers (they are not on the index -> gather dependency chain).  Measured on B200: for graphs reduced
    in two phases (plain SpMV) staging wins, 67 % against 53 % of the HBM peak on the 7-point fp64 SpMV -- a
    direct value load is a DRAM round trip inside the tile, longer than the L2-hit gather it travels with;
    for graphs that run fused, one thread per row (row-identity selectors: spring-mass, Rusanov), the direct
    loads win (33 % against 30 %), because the stage goes back to the producer only at the end of the tile and
    a smaller stage is refilled sooner -- unless the graph reads three or more separate edge tensors per edge
    (the shallow-water model's alpha, sx, sy: 38.8 % staged against 35.3 % direct), where one staged window per
    tensor replaces three uncoalesced-per-thread loads -- or one edge tensor of three or more values (the Rusanov
    face record).  FLEXSPMV_STAGE_VALUES=0/1 overrides."""
    import os
    env = os.environ.get("FLEXSPMV_STAGE_VALUES")
    if env in ("0", "1"):
        return env == "1"
    fused = any(s_.get("selector") == 1 and s_.get("row_identity") for s_ in ir.selector_register)
    edge_tensors = {s_["target"]: dim_of(s_["shape"]) for s_ in ir.selector_register if s_.get("selector") != 1}
    # fused graphs: staged from three values per edge on, in one tensor or several (Rusanov's (nx, ny, len) record:
    # 37.4 % staged against 33.6 % direct once the row-mode layout had given up its product buffer)
    return (not fused) or sum(edge_tensors.values()) >= 3


def _stream_bytes_per_edge(ir: GraphIR, vb: int) -> Tuple[int, int]:
    """(bytes staged per edge, number of staged streams): every distinct edge tensor plus one int32
    index array per distinct non-row-identity selector."""
    seen, total = set(), 0
    for s in ir.selector_register:
        if stage_values(ir) and s.get("selector") != 1 and s["target"] not in seen:
            seen.add(s["target"])
            total += vb * dim_of(s["shape"])
    for s in ir.selector_register:
        if s.get("selector") == 1 and not s.get("row_identity") and ("idx:" + s["selector_name"]) not in seen:
            seen.add("idx:" + s["selector_name"])
            total += 4
    return total, len(seen)


def direct_loads(ir: GraphIR, dtype: str) -> bool:
    """True when every per-edge record is 4, 8 or 16 bytes wide: a warp then reads 128-512 contiguous
    bytes per load instruction straight from global memory and staging through shared memory would only
    add traffic on the L1 data pipe.  Wider records (edge tensors of 3 or 6 values, ...) are staged by bulk
    copies so that the global side stays one contiguous transfer.  Measured on B200 (config 4, fp64
    SpMV): without the bulk-copy prefetch the direct path exposes the whole coordinate -> index -> gather
    latency chain per tile and reaches 44-47% of the HBM peak against 67% staged, so staging is the
    default for every graph and this path is only built with FLEXSPMV_DIRECT_LOADS=1."""
    import os
    if os.environ.get("FLEXSPMV_DIRECT_LOADS") != "1":
        return False
    vb = VBYTES[dtype]
    for s_ in ir.selector_register:
        if s_.get("selector") != 1 and vb * dim_of(s_["shape"]) not in (4, 8, 16):
            return False
    return True


def smem_bytes(ir: GraphIR, dtype: str, block: int, ipt: int, stages: int) -> int:
    """Upper bound of the tile kernel's dynamic shared memory (mirrors TileSmemLayout in
    csrc/flex_tile_kernel.cuh for 64-bit row offsets, the larger of the two instantiations)."""
    vb = VBYTES[dtype]
    per_edge, ns = _stream_bytes_per_edge(ir, vb)
    acc = max(1, sum(dim_of(o["shape"]) for o in ir.outputs if str(o["target"]) == "reducer"))
    tile = block * ipt
    stage = 0 if direct_loads(ir, dtype) else -(-(tile * max(8, per_edge) + 32 * (ns + 1) + 16) // 128) * 128
    fixed = 8 * stages + (32 + 4 * max(ns, 1) + 16) * stages + 4 * (block + 1) + 4 * (block // 32) \
        + vb * acc * (block // 32) + vb * acc * 2 + 16 + 8 * 16 + 128
    needs_row = any(s_.get("selector") == 1 and s_.get("row_identity") for s_ in ir.selector_register)
    buffers = 1   # 2 only when the kernel is built with tile pipelining (TileCfg::kPipeline)
    # row-mode graphs reduce in registers: no product buffer
    return fixed + 4 * (tile + 1) * buffers + (0 if needs_row else vb * acc * tile * buffers) + stages * stage


def choose_config(ir: GraphIR, dtype: str) -> Tuple[int, int, int, int]:
    """(consumer threads, merge items per thread, stages, min CTAs per SM).  The kernel is bound by
    latency per tile rather than by bytes in flight, so the heuristic prefers many resident CTAs (4,
    then 3, then 2 per SM) over big tiles: it takes the largest odd items-per-thread in [3, 5] whose
    shared-memory carve-up still lets that many CTAs share the 228 KB of one SM."""
    block, stages = 256, 2
    for ctas in (4, 3, 2):
        limit = (227 * 1024) // ctas - 1024
        for ipt in (5, 3):
            if smem_bytes(ir, dtype, block, ipt, stages) <= limit:
                return block, ipt, stages, ctas
    ipt = 1
    while block > 64 and smem_bytes(ir, dtype, block, ipt, stages) > 110 * 1024:
        block //= 2
    return block, ipt, stages, 2


# Tile configurations measured on B200 for the built-in benchmark graphs (block, items per thread, stages,
# min CTAs per SM[, pipelined tiles, edges per register batch of the fused row mode]); graphs not listed use the
# heuristic of choose_config.  In the fused row mode one more resident CTA beats a wider register batch: the
# other warps hide the gather latency better than more loads in flight per thread do.
TUNED_CONFIGS = {
    "spmv_f64": (256, 5, 2, 4),          # 7-point fp64 SpMV: 70 % of the HBM peak; 3 stages / bigger CTAs / 3 or 5 CTAs all lower
    "spmv_f32": (256, 5, 2, 4),
    "spmv_i64": (256, 5, 2, 4),
    # warm / L2-flushed % of the HBM peak:
    "spring_mass_f32": (256, 8, 2, 4, 0, 2),   # 35.5 / 31.2: 2048-item tiles hold ~228 rows of 8 edges, one per thread (batch 4: 34.9 / 31.2, batch 1 x 5 CTAs: 36.1 / 29.2, batch 8: 25)
    "rusanov_f64": (256, 4, 2, 3, 0, 1),       # 33.1 / 30.9: 1024-item tiles hold 256 rows of 3 edges (batch 2: 29.4 / 27.6, batch 3: 27.3 / 25.9, batch 1 x 4 CTAs: 30.3 / 28.7)
    "swe_delta_f64": (256, 3, 2, 3, 0, 1),     # 52.7 / 45.3 with staged edge tensors ((256,4,2,3) batch 1: 48.7 / 39.8, direct: 35.3 / 32.2; heuristic (256,3,2,4) batch 2: 33.8 / 31.5)
}


# Configuration of the warp kernel for matrices whose gathers have no locality (csrc/flex_warp_kernel.cuh):
# (threads per CTA, merge items per lane, min CTAs per SM).  It is built for graphs whose gathers all depend on the
# edge and whose accumulator is at most 16 bytes wide (its one shared-memory buffer holds a product per item, and
# the point of the kernel is to leave the shared-memory / L1 array to the gathers).
# Measured on the power-law matrix (fp32, % of the HBM peak): one CTA of 1024 threads per SM 27.6, 2 x 512 26.9, 4 x 256 26.1,
# 8 x 128 24.3, 16 x 64 23.0 (the same 32 warps per SM every time; the driver sizes the shared-memory carve-out for the
# largest number of CTAs the kernel could have resident, so few large CTAs leave the most L1); 6 / 7 items per lane 27.6 / 25.5.
LEAN_CONFIG = (1024, 5, 1)
# 8-byte values need more than the 64 registers a 1024-thread CTA leaves a thread (the kernel spills: 160 G gathers/s on
# the power-law matrix in fp64); 768 threads (85 registers) reach 195, 512 threads 172, cuSPARSE 188.
LEAN_CONFIG_WIDE = (768, 5, 1)
TUNED_LEAN_CONFIGS = {
}


def lean_eligible(ir: GraphIR, dtype: str) -> bool:
    if not ir.has_reducer or ir.aggregator_operations:
        return False
    if any(s_.get("selector") == 1 and s_.get("row_identity") for s_ in ir.selector_register):
        return False
    acc = sum(dim_of(o["shape"]) for o in ir.outputs if str(o["target"]) == "reducer")
    return acc * VBYTES[dtype] <= 16


# Tile configurations of the gather-window variant (its stages also hold the window area).
TUNED_WIN_CONFIGS = {
}


def _override(symbol: str):
    """Tuning hook: FLEXSPMV_CFG_OVERRIDE="spmv_f64=256,7,2,3;rusanov_f64=128,5,3,4" replaces the
    heuristic tile configuration (block, items per thread, stages, min CTAs per SM[, pipelined tiles 0|1[, edges per
    register batch of the fused row mode]]) at build time."""
    import os
    for part in os.environ.get("FLEXSPMV_CFG_OVERRIDE", "").split(";"):
        if "=" in part:
            k, v = part.split("=", 1)
            if k.strip() == symbol:
                return tuple(int(x) for x in v.split(","))
    return None


def _with_node_names(ir: GraphIR) -> GraphIR:
    """torch.fx gives a placeholder the node name ``l`` and the target ``L`` for an argument called ``L``; the
    tracer records both (edge-tensor registers carry the target, everything else the name).  The emitter works
    on node names only, so edge-tensor registers are renamed here when the two differ."""
    alias = {i["target"]: i["name"] for i in ir.inputs if i["dtype"] != "int" and i["target"] != i["name"]}
    if not any(s.get("selector") != 1 and s["target"] in alias for s in ir.selector_register):
        return ir
    import copy
    ir = copy.copy(ir)
    ir.selector_register = [dict(s, target=alias.get(s["target"], s["target"])) if s.get("selector") != 1 else s
                            for s in ir.selector_register]
    return ir


def emit_graph(ir: GraphIR, dtype: str, symbol: str | None = None, config=None, static_scratch_bytes: int = 0,
               windows: bool = True) -> str:
    """One translation unit for ``ir`` compiled for ``dtype``.  ``windows=False`` leaves out the gather-window
    variant of the tile kernel (half the kernel instantiations: the form the torch-extension shim is built in)."""
    ir = _with_node_names(ir)
    cty, sfx = CTYPE[dtype]
    symbol = symbol or f"{ir.name}_{sfx}"
    # measured configurations are keyed by graph and value type, whatever symbol prefix the unit is emitted under
    cfg = tuple(config or _override(symbol) or TUNED_CONFIGS.get(f"{ir.name}_{sfx}") or choose_config(ir, dtype))
    block, ipt, stages, min_ctas = cfg[:4]
    pipeline = len(cfg) > 4 and bool(cfg[4])     # fifth field: software-pipelined tiles (TileCfg::kPipeline)
    batch_override = cfg[5] if len(cfg) > 5 else 0   # sixth field: edges per register batch in the fused row mode
    import os
    win_bytes = int(os.environ.get("FLEXSPMV_WIN_BYTES", 1024 * VBYTES[dtype]))
    non_gather, gathers, index_names = operator_signature(ir)
    value_names = non_gather + gathers
    in_dims = {i["name"]: dim_of(i["shape"]) for i in ir.inputs if i["dtype"] != "int"}
    has_reducer = ir.has_reducer
    if has_reducer and ir.aggregator_operations:
        raise ValueError("a graph with a reducer cannot also hold a `sum` aggregator "
                         "(the reference's reducer template has no aggregator slot either)")

    # ---- streams (staged per-edge arrays) ---------------------------------------------------------
    streams: List[Tuple[str, str, int]] = []      # (param field, element C type, bytes per edge)
    stream_of: Dict[str, int] = {}
    staged_values = stage_values(ir)
    inplace_targets = {op_["args"][0] for op_ in ir.map_operations if op_["op"] in ("add_", "copy_", "setitem")}
    for s in ir.selector_register:
        if staged_values and s.get("selector") != 1 and s["target"] not in stream_of:
            stream_of[s["target"]] = len(streams)
            streams.append((s["target"], "V", f"int(sizeof(V)) * {dim_of(s['shape'])}"))
    for s in ir.selector_register:
        if s.get("selector") == 1 and not s.get("row_identity"):
            key = "idx:" + s["selector_name"]
            if key not in stream_of:
                stream_of[key] = len(streams)
                streams.append((s["selector_name"] + "_idx", "int", "4"))

    # ---- outputs ------------------------------------------------------------------------------------
    reducers, aggs, map_outs = [], [], []
    acc_off = agg_off = 0
    for oi, o in enumerate(ir.outputs):
        d = dim_of(o["shape"])
        tgt = str(o["target"])
        if tgt == "reducer":
            reducers.append((o["name"], d, acc_off, oi))
            acc_off += d
        elif "sum" in tgt:
            aggs.append((o["name"], d, agg_off, oi))
            agg_off += d
        else:
            map_outs.append((o["name"], d, oi))
    red_by_name = {r[0]: r for r in reducers}
    agg_by_name = {a[0]: a for a in aggs}

    L: List[str] = []
    w = L.append
    w(f"// GENERATED by flexspmv_b200.codegen.emit_cuda -- graph '{ir.name}' ({dtype}), digest {ir.digest()}")
    w('#include "flex_graph_api.cuh"')
    w("namespace {")
    w(f"namespace gen_{symbol} {{      // several generated units may share one translation unit")
    w("struct Graph {")
    w(f"  using V = {cty};")
    w(f"  static constexpr int kNumValues = {len(value_names)}, kNumIndices = {len(index_names)}, kNumOutputs = {len(ir.outputs)};")
    w(f"  static constexpr bool kHasReducer = {'true' if has_reducer else 'false'};")
    w(f"  static constexpr int kNumReducers = {len(reducers)}, kAccDim = {max(acc_off, 1)}, kAggDim = {agg_off};")
    w(f"  static constexpr int kNumStreams = {len(streams)};")
    w(f"  static constexpr bool kDirectLoads = {'true' if direct_loads(ir, dtype) else 'false'};")
    needs_row = any(s.get("selector") == 1 and s.get("row_identity") for s in ir.selector_register)
    w(f"  static constexpr bool kGatherNeedsRow = {'true' if needs_row else 'false'};")
    w("  static constexpr int kStreamBytesPerEdge = 0" + "".join(f" + {b}" for _, _, b in streams) + ";")
    w("  struct Params {")
    for n in value_names:
        w(f"    V* {n};")
    for n in index_names:
        w(f"    const int* {n}_idx;")
    for o in ir.outputs:
        w(f"    V* out_{o['name']};")
    w("  };")
    w("  static Params make_params(const void* const* values, const void* const* indices, void* const* outputs) {")
    w("    Params p{};")
    for i, n in enumerate(value_names):
        w(f"    p.{n} = static_cast<V*>(const_cast<void*>(values[{i}]));")
    for i, n in enumerate(index_names):
        w(f"    p.{n}_idx = static_cast<const int*>(indices[{i}]);")
    for i, o in enumerate(ir.outputs):
        w(f"    p.out_{o['name']} = static_cast<V*>(outputs[{i}]);")
    w("    (void)values; (void)indices; (void)outputs;")
    w("    return p;")
    w("  }")
    # alignment: streamed arrays 16 B, gather sources to their vector chunk
    w("  static bool pointers_aligned(const Params& p) {")
    w("    bool ok = true;")
    for f, _, _ in streams:
        w(f"    ok = ok && (reinterpret_cast<uintptr_t>(p.{f}) % 16 == 0);")
    seen = set()
    for s in ir.selector_register:
        if s.get("selector") == 1 and s["target"] not in seen:
            seen.add(s["target"])
            w(f"    ok = ok && (reinterpret_cast<uintptr_t>(p.{s['target']}) % fx::VecIO<V, {dim_of(s['shape'])}>::kChunk == 0);")
        if s.get("selector") != 1 and not staged_values and s["target"] not in seen:
            seen.add(s["target"])
            w(f"    ok = ok && (reinterpret_cast<uintptr_t>(p.{s['target']}) % fx::VecIO<V, {dim_of(s['shape'])}>::kChunk == 0);")
    w("    (void)p; return ok;")
    w("  }")
    w("  template <int I> __host__ __device__ static constexpr int stream_bytes() {")
    for i, (_, _, b) in enumerate(streams):
        w(f"    if constexpr (I == {i}) return {b};")
    w("    return 0;")
    w("  }")
    w("  template <int I> __device__ __forceinline__ static const char* stream_ptr(const Params& p) {")
    for i, (f, _, _) in enumerate(streams):
        w(f"    if constexpr (I == {i}) return reinterpret_cast<const char*>(p.{f});")
    w("    (void)p; return nullptr;")
    w("  }")
    w("  template <int R> __host__ __device__ static constexpr int red_dim() {")
    for i, (_, d, _, _) in enumerate(reducers):
        w(f"    if constexpr (R == {i}) return {d};")
    w("    return 1;")
    w("  }")
    w("  template <int R> __host__ __device__ static constexpr int red_off() {")
    for i, (_, _, off, _) in enumerate(reducers):
        w(f"    if constexpr (R == {i}) return {off};")
    w("    return 0;")
    w("  }")
    w("  template <int R> __device__ __forceinline__ static V* red_out(const Params& p) {")
    for i, (n, _, _, _) in enumerate(reducers):
        w(f"    if constexpr (R == {i}) return p.out_{n};")
    w("    (void)p; return nullptr;")
    w("  }")
    w("  __device__ __forceinline__ static void store_aggregate(const Params& p, int i, V s) {")
    for n, d, off, _ in aggs:
        w(f"    if (i >= {off} && i < {off + d}) p.out_{n}[i - {off}] = s;")
    w("    (void)p; (void)i; (void)s;")
    w("  }")

    # ---- gather: what depends only on the row (row-identity selectors) and what depends on the edge ----
    gsel = [s for s in ir.selector_register if s.get("selector") == 1]
    row_sel = [s for s in gsel if s.get("row_identity")]
    edge_sel = [s for s in gsel if not s.get("row_identity")]
    w("  struct GRow {")
    for s in row_sel:
        w(f"    fx::Vec<V, {dim_of(s['shape'])}> {s['name']};")
    w("@@GROW_FIELDS@@")
    if not row_sel:
        w("    int unused;")
    w("  };")
    w("  struct GEdge {")
    for s in edge_sel:
        w(f"    fx::Vec<V, {dim_of(s['shape'])}> {s['name']};")
    if not edge_sel:
        w("    int unused;")
    w("  };")
    w("  __device__ __forceinline__ static void gather_row(const Params& p, long long row, GRow& g) {")
    for s in row_sel:
        d = dim_of(s["shape"])
        w(f"    g.{s['name']} = fx::ldg_vec<V, {d}>(p.{s['target']} + row * {d});")
    w("@@GROW_BODY@@")
    w("    (void)p; (void)row; (void)g;")
    w("  }")
    # per-edge data that comes out of the staged arrays: copied to registers first, so that the stage can
    # be handed back to the producer before the gathers are even issued
    edge_regs_list = [s_ for s_ in ir.selector_register if s_.get("selector") != 1]
    idx_names = list(dict.fromkeys(s_["selector_name"] for s_ in edge_sel))   # calls of one Selector share its index
    w("  struct EReg {")
    for n_ in idx_names:
        w(f"    int idx_{n_};")
    seen_e = set()
    for s_ in edge_regs_list:
        if s_["selector_name"] not in seen_e:
            seen_e.add(s_["selector_name"])
            w(f"    fx::Vec<V, {dim_of(s_['shape'])}> {s_['selector_name']};")
    if not edge_sel and not edge_regs_list:
        w("    int unused;")
    w("  };")
    w("  template <class Tile, class IdxT>")
    w("  __device__ __forceinline__ static void load_edge(const Params& p, const Tile& t, IdxT le, long long e, EReg& r) {")
    for n_ in idx_names:
        si = stream_of["idx:" + n_]
        w(f"    r.idx_{n_} = *t.template stream<{si}, int>(le);")
    w("    load_edge_vals(p, t, le, e, r);")
    w("  }")
    w("  template <class Tile, class IdxT>")
    w("  __device__ __forceinline__ static void load_edge_vals(const Params& p, const Tile& t, IdxT le, long long e, EReg& r) {")
    seen_e = set()
    for s_ in edge_regs_list:
        if s_["selector_name"] not in seen_e:
            seen_e.add(s_["selector_name"])
            d_ = dim_of(s_["shape"])
            if staged_values:
                si = stream_of[s_["target"]]
                w(f"    r.{s_['selector_name']} = fx::ld_vec<V, {d_}>(t.template stream<{si}, V>(le));")
            elif s_["target"] in inplace_targets:   # written through the same pointer by this kernel: no read-only path
                w(f"    r.{s_['selector_name']} = fx::ld_vec<V, {d_}>(p.{s_['target']} + e * {d_});")
            else:
                w(f"    r.{s_['selector_name']} = fx::ldg_vec<V, {d_}>(p.{s_['target']} + e * {d_});")
    w("    (void)p; (void)t; (void)le; (void)e; (void)r;")
    w("  }")
    # edge tensors that are NOT staged are read straight from global memory by the consumers; the producer warp
    # prefetches the tile's part of them into L2 when it stages the tile, STAGES tiles ahead of their use
    w("  __device__ __forceinline__ static void prefetch_direct(const Params& p, long long nz0, long long nz1, int lane) {")
    seen_e = set()
    for s_ in edge_regs_list:
        if s_["selector_name"] not in seen_e and not staged_values:
            seen_e.add(s_["selector_name"])
            d_ = dim_of(s_["shape"])
            w(f"    fx::prefetch_l2_range(p.{s_['target']} + nz0 * {d_}, p.{s_['target']} + nz1 * {d_}, lane);")
    w("    (void)p; (void)nz0; (void)nz1; (void)lane;")
    w("  }")
    w(f"  static constexpr bool kHasDirectEdgeTensors = {'true' if (edge_regs_list and not staged_values) else 'false'};")
    # L1 prefetch of what gather_edge will read, issued by the producer warp one tile ahead
    w("  template <class Tile, class IdxT>")
    w("  __device__ __forceinline__ static void prefetch_edge(const Params& p, const Tile& t, IdxT le) {")
    for s_ in edge_sel:
        d = dim_of(s_["shape"])
        si = stream_of["idx:" + s_["selector_name"]]
        w(f"    fx::prefetch_l1<V, {d}>(p.{s_['target']} + (long long)(*t.template stream<{si}, int>(le)) * {d});")
    w("    (void)p; (void)t; (void)le;")
    w("  }")
    w(f"  static constexpr bool kHasEdgeGather = {'true' if edge_sel else 'false'};")
    w("  __device__ __forceinline__ static void gather_edge(const Params& p, const EReg& r, GEdge& g) {")
    for s_ in edge_sel:
        d = dim_of(s_["shape"])
        w(f"    g.{s_['name']} = fx::ldg_vec<V, {d}>(p.{s_['target']} + (long long)r.idx_{s_['selector_name']} * {d});")
    w("    (void)p; (void)r; (void)g;")
    w("  }")
    # gather windows: a two-phase graph with exactly one index array and one gathered tensor whose record is a
    # power of two bytes can take its gathers from segments of that tensor staged in shared memory
    win_ok = has_reducer and not needs_row and staged_values and len(idx_names) == 1 and len(edge_sel) == 1 \
        and not direct_loads(ir, dtype)
    if win_ok:
        gs = edge_sel[0]
        rec = dim_of(gs["shape"]) * VBYTES[dtype]
        win_ok = rec in (4, 8, 16, 32) and gs["target"] not in inplace_targets
    w(f"  static constexpr bool kWindowGather = {'true' if win_ok else 'false'};")
    if win_ok:
        gs = edge_sel[0]
        d = dim_of(gs["shape"])
        w(f"  static constexpr int kIdxStream = {stream_of['idx:' + idx_names[0]]};")
        w(f"  static constexpr int kGatherRecBytes = {d} * int(sizeof(V));")
        w(f"  static constexpr int kWinBytes = {win_bytes};      // window area per stage")
        w(f"  __host__ __device__ static const void* gather_base(const Params& p) {{ return p.{gs["target"]}; }}")
        w("  __device__ __forceinline__ static void gather_edge_win(const unsigned char* xw, unsigned pos, GEdge& g) {")
        w(f"    g.{gs['name']} = fx::ld_vec<V, {d}>(reinterpret_cast<const V*>(xw) + pos * {d});")
        w("  }")

    # ---- map ----------------------------------------------------------------------------------------
    env: Dict[str, Var] = {}
    # Operations whose operands are only the row's own records (row-identity gathers), literals and other such
    # operations depend on the row, not on the edge: they are evaluated once per row in gather_row (same operations
    # in the same order, so bit-identical) and their results travel in GRow.  FLEXSPMV_HOIST=0 keeps them per edge.
    import os as _os
    hoisting = _os.environ.get("FLEXSPMV_HOIST", "1") != "0"
    row_only = {s_["name"] for s_ in ir.selector_register if s_.get("selector") == 1 and s_.get("row_identity")}
    pure_kinds = set(_BIN) | {"neg", "exp", "abs", "sign", "norm", "getitem", "clone", "where"}
    body: List[str] = []
    row_body: List[str] = []
    grow_fields: List[str] = []
    target = [body]

    def b(line: str):
        target[0].append(line)

    for s_ in ir.selector_register:
        if s_.get("selector") == 1 and s_.get("row_identity"):
            row_body.append(f"    const fx::Vec<V, {dim_of(s_['shape'])}>& {s_['name']} = g.{s_['name']};")
    for s in ir.selector_register:
        d = dim_of(s["shape"])
        if s.get("selector") == 1:
            src = "gr" if s.get("row_identity") else "ge"
            b(f"    const fx::Vec<V, {d}>& {s['name']} = {src}.{s['name']};")
            env[s["name"]] = Var("vec", d, s["name"])
        else:
            b(f"    fx::Vec<V, {d}> {s['selector_name']} = r.{s['selector_name']};")
            env[s["selector_name"]] = Var("vec", d, s["selector_name"])

    def operand(a):
        if isinstance(a, str):
            if a not in env:
                raise ValueError(f"graph '{ir.name}': operand '{a}' is not defined before use")
            return env[a]
        return Var("lit", 0, _lit(a))

    for op in ir.map_operations:
        kind, name, args = op["op"], op["name"], op["args"]
        d = dim_of(op["shape"])
        names_used = [a_ for a_ in args if isinstance(a_, str)]
        hoist = hoisting and kind in pure_kinds and names_used and all(a_ in row_only for a_ in names_used)
        target[0] = row_body if hoist else body
        if hoist:
            row_only.add(name)
        if kind in _BIN:
            A, B = operand(args[0]), operand(args[1])
            if A.kind == "vec" and B.kind == "vec":
                opn = _BIN[kind]
                if kind == "truediv" and A.dim == B.dim:
                    opn = "DivGuard"        # member operator/ of equal widths guards a zero divisor
                b(f"    const auto {name} = fx::zip({A.expr}, {B.expr}, fx::{opn}{{}});")
                env[name] = Var("vec", max(A.dim, B.dim), name)
            elif A.kind == "vec":
                opn = _BIN[kind]
                if kind == "pow" and B.kind == "lit" and not isinstance(args[1], str) and float(args[1]) == 0.5 \
                        and dtype != "int64":
                    opn = "PowHalf"     # x ^ 0.5: one exactly rounded sqrt instead of the library pow
                b(f"    const auto {name} = fx::zip_vs({A.expr}, {B.expr}, fx::{opn}{{}});")
                env[name] = Var("vec", A.dim, name)
            elif B.kind == "vec":
                if kind in ("lt", "gt"):
                    raise ValueError("scalar on the left of lt/gt has no overload in the reference")
                opn = "DivGuard" if kind == "truediv" else _BIN[kind]
                b(f"    const auto {name} = fx::zip_sv({A.expr}, {B.expr}, fx::{opn}{{}});")
                env[name] = Var("vec", B.dim, name)
            else:
                if kind not in _SCALAR_FN or (A.kind == "lit" and B.kind == "lit"):
                    raise ValueError(f"unsupported scalar-scalar op {kind}")
                b(f"    const fx::Vec<V, 1> {name}{{{{ fx::{_SCALAR_FN[kind]}(V({A.expr}), V({B.expr})) }}}};")
                env[name] = Var("vec", 1, name)
        elif kind == "neg":
            A = operand(args[0])
            b(f"    const auto {name} = fx::neg({A.expr});")
            env[name] = Var("vec", A.dim, name)
        elif kind in ("exp", "abs", "sign"):
            A = operand(args[0])
            b(f"    const auto {name} = fx::vec_{kind}({A.expr});")
            env[name] = Var("vec", A.dim, name)
        elif kind == "norm":
            A = operand(args[0])
            b(f"    const V {name} = fx::norm({A.expr});")
            env[name] = Var("scalar", 1, name)
        elif kind == "getitem":
            A = operand(args[0])
            b(f"    const auto {name} = fx::item({A.expr}, {int(args[1][1])});")
            env[name] = Var("vec", 1, name)
        elif kind == "clone":
            A = operand(args[0])
            if A.kind == "vec":
                b(f"    const auto {name} = {A.expr};")
                env[name] = Var("vec", A.dim, name)
            else:
                b(f"    const fx::Vec<V, 1> {name}{{{{ {A.expr} }}}};")
                env[name] = Var("vec", 1, name)
        elif kind == "where":
            C, X, Y = operand(args[0]), operand(args[1]), operand(args[2])
            b(f"    const auto {name} = fx::where3({C.expr}, {X.expr}, {Y.expr});")
            env[name] = Var("vec", max([C.dim] + [v.dim for v in (X, Y) if v.kind == "vec"]), name)
        elif kind == "copy_":
            S = operand(args[1])
            b(f"    fx::st_vec(p.{args[0]} + (long long)e * {d}, {S.expr});")
        elif kind == "setitem":
            S = operand(args[2])
            b(f"    fx::st_vec(p.{args[0]} + (long long)e * {d}, {S.expr});")
            b(f"    {args[0]} = {S.expr};")
        elif kind == "add_":
            A, B = operand(args[0]), operand(args[1])
            if B.kind == "vec":
                b(f"    {A.expr} = fx::zip({A.expr}, {B.expr}, fx::Add{{}});")
            else:
                b(f"    {A.expr} = fx::zip_vs({A.expr}, {B.expr}, fx::Add{{}});")
            b(f"    fx::st_vec(p.{args[0]} + (long long)e * {d}, {A.expr});")
        elif kind == "reducer":
            A = operand(args[0])
            _, rd, off, _ = red_by_name[name]
            if A.kind == "vec":
                if A.dim != rd:
                    raise ValueError(f"reducer {name}: width {A.dim} != {rd}")
                b(f"    fx::accumulate<{off}>(acc, {A.expr});")
            else:
                b(f"    fx::accumulate_scalar<{off}, {rd}>(acc, {A.expr});")
        elif kind == "sum":
            A = operand(args[0])
            _, ad, off, _ = agg_by_name[name]
            if A.kind == "vec":
                b(f"    fx::accumulate<{off}>(acc, {A.expr});")
            else:
                b(f"    fx::accumulate_scalar<{off}, {ad}>(acc, {A.expr});")
        else:
            raise ValueError(f"Operation {kind} not supported")
        if hoist:
            v_ = env[name]
            if v_.kind == "scalar":
                grow_fields.append(f"    V {name};")
                body.append(f"    const V {name} = gr.{name};")
            else:
                grow_fields.append(f"    fx::Vec<V, {v_.dim}> {name};")
                body.append(f"    const fx::Vec<V, {v_.dim}>& {name} = gr.{name};")
            row_body.append(f"    g.{name} = {name};")
    target[0] = body
    for n, d, _ in map_outs:
        v = operand(n)
        if v.kind == "vec":
            b(f"    fx::st_vec(p.out_{n} + (long long)e * {d}, {v.expr});")
        else:
            b(f"    p.out_{n}[(long long)e] = {v.expr};")

    w("  __device__ __forceinline__ static void map(const Params& p, const EReg& r, long long e, const GRow& gr, const GEdge& ge, V* acc) {")
    L.extend(body)
    w("    (void)p; (void)r; (void)e; (void)gr; (void)ge; (void)acc;")
    w("  }")
    w("};")
    # registers one edge keeps live in the fused thread-per-row loop: its staged record (indices + edge
    # tensors) and its gathered vertex data; the batch is the largest of 8/4/3/2 edges that stays under ~28
    words = VBYTES[dtype] // 4
    per_edge_regs = sum(dim_of(s_["shape"]) * words for s_ in ir.selector_register
                        if not (s_.get("selector") == 1 and s_.get("row_identity")))
    per_edge_regs += len({s_["selector_name"] for s_ in ir.selector_register
                          if s_.get("selector") == 1 and not s_.get("row_identity")})
    batch = next((b_ for b_ in (8, 4, 3, 2) if b_ * max(per_edge_regs, 1) <= 28), 2)
    batch = batch_override or batch
    w(f"using Cfg = flex::TileCfg<{block}, {ipt}, {stages}, {min_ctas}, {batch}, {'true' if pipeline else 'false'}>;")
    wb_, wi_, ws_, wm_ = tuple(_override(symbol + "_win") or TUNED_WIN_CONFIGS.get(symbol) or (block, ipt, stages, min_ctas))[:4]
    if windows:
        w(f"using CfgWin = flex::TileCfg<{wb_}, {wi_}, {ws_}, {wm_}, {batch}, false>;   // the gather-window variant of the kernel")
    else:
        w("using CfgWin = flex::NoWindows;      // built without the gather-window variant of the kernel")
    if lean_eligible(ir, dtype):
        lean_default = LEAN_CONFIG_WIDE if VBYTES[dtype] == 8 else LEAN_CONFIG
        lb, li, lm = tuple(_override(symbol + "_lean") or TUNED_LEAN_CONFIGS.get(f"{ir.name}_{sfx}") or lean_default)[:3]
        w(f"using CfgLean = flex::WarpCfg<{lb}, {li}, {lm}>;      // the warp kernel for matrices with random columns")
    else:
        w("using CfgLean = flex::NoLean;")
    w(f"}}  // namespace gen_{symbol}")
    w("}  // namespace")
    for i_, line in enumerate(L):
        if line == "@@GROW_FIELDS@@":
            L[i_] = "\n".join(grow_fields) if grow_fields else "    // (no row-only intermediate values)"
        elif line == "@@GROW_BODY@@":
            L[i_] = "\n".join(row_body) if grow_fields else "    // (nothing to evaluate per row)"
    ns = f"gen_{symbol}::"
    w(f"FLEXSPMV_DEFINE_GRAPH({symbol}, {ns}Graph, {ns}Cfg, {ns}CfgWin, {ns}CfgLean)")
    if static_scratch_bytes:
        w(f"FLEXSPMV_DEFINE_STATIC_SCRATCH_LAUNCH({symbol}, {ns}Graph, {ns}Cfg, {int(static_scratch_bytes)})")
    return "\n".join(L) + "\n"
