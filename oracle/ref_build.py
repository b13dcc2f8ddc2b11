"""CPU ORACLE -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Builds the REFERENCE'S OWN generated CPU operator for each graph, from the reference's sources where
they lie, into ``oracle/_ref/`` (git-ignored; only shared objects and a manifest are written there).

Recipe (the reference's own flow, codegen/merged_gen_cpu.py:18-151, minus the ``easier`` tracer that
produces the IR): feed the hand-built IR lists (flexspmv_b200/graphs.py) to the reference emitters
``codegen.merged_gen_core.{declarations_gen, map_gen, reducer_gen, aggregator_gen}``, substitute the
snippets into ``cpu_template/merged_spmv_template_{reducer,aggregator}.h`` with ``string.Template``
exactly as merged_gen_cpu.py does, and compile the resulting ``OmpMergeSystem<ValueT,int>`` with
``g++ -O3 -fopenmp`` (the flags of test_full/easier_full.py:476; no -march so the object runs on any
x86-64 host) behind a three-line ``extern "C"`` trampoline written here.  The reference's torch
binding (merged_binding_cpu.cpp) is a thin shim over the same function and is not needed.
The trampoline also exports the header's own free function ``MergePathSearch``
(cpu_template/merged_spmv_template_reducer.h:27-51) as ``ref_merge_path_search`` so that partition
coordinates can be compared with the reference's search itself.

The reference's Makefile compiles with ``-march=native`` (Makefile:18).  The machine that times the CPU
arm is not the machine that compiles it (the reference tree is only present on the latter), so a
second object of the plain SpMV graph is built with ``-march=x86-64-v3`` (AVX2 + FMA, what every recent
x86-64 server has); the benchmark times both and keeps the faster.  The tests use the portable one.

No reference source text is copied into the repository: the generated header lives in a temporary
directory and only the compiled object is kept.  Requires the reference tree: FLEXSPMV_REFERENCE_DIR, or
a directory called ``reference`` beside the repository; when it is absent this script does nothing and
the prebuilt objects already in oracle/_ref are used.
"""
from __future__ import annotations

import json
import os
import re
import string
import subprocess
import sys
import tempfile

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.environ.get("FLEXSPMV_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
OUT_DIR = os.path.join(_HERE, "_ref")
CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"

RECIPE = 2      # bumped when the trampoline or the compile commands change, so that existing objects are rebuilt

_CTYPE = {"float32": ("float", "f32"), "float64": ("double", "f64"), "int64": ("long", "i64")}


def reference_available() -> bool:
    return os.path.isfile(os.path.join(REF_DIR, "codegen", "merged_gen_core.py"))


def _join(x):
    return "".join(x) if x else ""


def generate_header(ir) -> tuple[str, list]:
    """Returns (merged_spmv.h text, parameter list [(kind, name)]) for one graph."""
    sys.dont_write_bytecode = True
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    from codegen.merged_gen_core import declarations_gen, map_gen, reducer_gen, aggregator_gen  # reference module

    inputs, outputs, selreg, mapops, reducers, aggs = ir.as_tuple()
    (input_parameters_code, input_agent_tenosrs_code, output_agent_tenosrs_code,
     output_agent_forloop_code, selector_code) = declarations_gen(inputs, outputs, selreg)
    map_code, map_agent_tenosrs_code = map_gen(mapops)
    (r_init, r_for, r_add, p_init, p_for, p_carry, p_fix) = reducer_gen(reducers)
    (a_fix, a_for, a_search, a_carry) = aggregator_gen(aggs)
    tag = "reducer" if reducers else "aggregator"
    with open(os.path.join(REF_DIR, "cpu_template", f"merged_spmv_template_{tag}.h")) as f:
        template = f.read()
    text = string.Template(template).substitute(
        input_parameters_code=_join(input_parameters_code),
        input_agent_tenosrs_code=_join(input_agent_tenosrs_code),
        output_agent_tenosrs_code=_join(output_agent_tenosrs_code),
        output_agent_forloop_code=_join(output_agent_forloop_code),
        selector_code=_join(selector_code),
        map_code=_join(map_code),
        map_agent_tenosrs_code=_join(map_agent_tenosrs_code),
        reducer_consume_init_code=_join(r_init),
        reducer_consume_forloop_code=_join(r_for),
        reducer_consume_forloop_add_code=_join(r_add),
        reducer_partial_init_code=_join(p_init),
        reducer_partial_forloop_code=_join(p_for),
        reducer_partial_carry_code=_join(p_carry),
        reducer_partial_carry_fixup_code=_join(p_fix),
        aggregator_partial_carry_fixup_code=_join(a_fix),
        aggregator_partial_forloop_code=_join(a_for),
        aggregator_diagonal_code_search=_join(a_search),
        aggregator_tenosrs_carry_out_code=_join(a_carry),
    )
    params = []
    for line in input_parameters_code:
        m = re.search(r"(OffsetT|ValueT) \*__restrict (\w+)_ptr", line)
        params.append(("index" if m.group(1) == "OffsetT" else "value", m.group(2)))
    return text, params


def build_graph(ir, dtypes) -> dict:
    text, params = generate_header(ir)
    os.makedirs(OUT_DIR, exist_ok=True)
    has_rows = ir.has_reducer
    with tempfile.TemporaryDirectory(prefix="flexspmv_ref_") as tmp:
        with open(os.path.join(tmp, "merged_spmv.h"), "w") as f:
            f.write(text)
        tramp = ['#include "merged_spmv.h"', 'extern "C" {']
        for dt in dtypes:
            cty, sfx = _CTYPE[dt]
            args = ", ".join(
                f"static_cast<{'int' if k == 'index' else cty}*>(p[{i}])" for i, (k, _) in enumerate(params))
            ro = "row_offsets, " if has_rows else ""
            tramp.append(
                f"void ref_run_{sfx}(int num_threads, int* row_offsets, void** p, int num_rows, int nnz) {{\n"
                f"  OmpMergeSystem<{cty}, int>(num_threads, {ro}{args}{', ' if args else ''}num_rows, nnz);\n}}")
        if has_rows:   # the reducer template defines the search; `a` = row END offsets (the callee's shifted pointer)
            tramp.append(
                "void ref_merge_path_search(int diagonal, int* row_end_offsets, int num_rows, int nnz, int* xy) {\n"
                "  int2 c; CountingInputIterator<int> nz(0);\n"
                "  MergePathSearch(diagonal, row_end_offsets, nz, num_rows, nnz, c);\n"
                "  xy[0] = c.x; xy[1] = c.y;\n}")
        tramp.append("}")
        with open(os.path.join(tmp, "trampoline.cpp"), "w") as f:
            f.write("\n".join(tramp) + "\n")
        so = os.path.join(OUT_DIR, f"libref_{ir.name}.so")
        base = [CXX, "-O3", "-fopenmp", "-fPIC", "-shared", "-w", "-I", REF_DIR, "-I", tmp,
                os.path.join(tmp, "trampoline.cpp")]
        subprocess.check_call(base + ["-o", so])
        ent = {"so": os.path.basename(so), "params": params, "dtypes": list(dtypes), "has_rows": has_rows}
        if ir.name == "spmv":      # the graph the benchmark's CPU arm times
            so3 = os.path.join(OUT_DIR, f"libref_{ir.name}_x86_64_v3.so")
            subprocess.check_call(base + ["-march=x86-64-v3", "-o", so3])
            ent["so_x86_64_v3"] = os.path.basename(so3)
    return ent


def build_all(force: bool = False) -> bool:
    """Build every graph's reference object; returns False when the reference tree is absent."""
    if not reference_available():
        return False
    sys.path.insert(0, os.path.dirname(_HERE))
    from flexspmv_b200.graphs import ALL_GRAPHS, GRAPH_DTYPES
    manifest_path = os.path.join(OUT_DIR, "manifest.json")
    manifest = {}
    if os.path.exists(manifest_path) and not force:
        with open(manifest_path) as f:
            manifest = json.load(f)
    changed = False
    for name, make in ALL_GRAPHS.items():
        ir = make()
        ent = manifest.get(name)
        if (not force and ent and ent.get("digest") == ir.digest() and ent.get("recipe") == RECIPE
                and os.path.exists(os.path.join(OUT_DIR, ent["so"]))):
            continue
        ent = build_graph(ir, GRAPH_DTYPES[name])
        ent["digest"] = ir.digest()
        ent["recipe"] = RECIPE
        manifest[name] = ent
        changed = True
    if changed:
        with open(manifest_path, "w") as f:
            json.dump(manifest, f, indent=1)
    return True


if __name__ == "__main__":
    ok = build_all(force="--force" in sys.argv)
    print("reference CPU operators built into", OUT_DIR if ok else "(skipped: reference tree absent)")
