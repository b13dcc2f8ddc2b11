"""The C-ABI library loads without a GPU and exports every symbol include/flexspmv.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "flexspmv.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    syms = set(re.findall(r"\b(flexspmv_[a-z0-9_]+)\s*\(", text))
    for g in re.findall(r"^FLEXSPMV_DECLARE_GRAPH\((\w+)\)", text, flags=re.M):
        for fn in ("info", "workspace_bytes", "plan", "launch", "device_status"):
            syms.add(f"flexspmv_{g}_{fn}")
    syms.discard("flexspmv_")
    return sorted(s for s in syms if "##" not in s)


@pytest.fixture(scope="module")
def lib():
    from flexspmv_b200.binding import load_library
    return load_library()


def test_every_declared_symbol_is_exported(lib):
    syms = declared_symbols()
    assert len(syms) >= 6 + 18 * 5
    missing = [s for s in syms if not hasattr(lib, s)]
    assert not missing, missing


def test_header_graph_list_matches_registry():
    from flexspmv_b200 import graphs
    from flexspmv_b200.codegen.emit_cuda import CTYPE
    text = open(HEADER).read()
    declared = set(re.findall(r"^FLEXSPMV_DECLARE_GRAPH\((\w+)\)", text, flags=re.M))
    expected = {f"{g}_{CTYPE[dt][1]}" for g in graphs.ALL_GRAPHS for dt in graphs.GRAPH_DTYPES[g]}
    assert declared == expected


def test_host_only_entry_points(lib):
    from flexspmv_b200.binding import Desc, GraphInfo
    assert lib.flexspmv_abi_version() == 1
    lib.flexspmv_error_string.restype = ctypes.c_char_p
    assert b"success" in lib.flexspmv_error_string(0)
    assert b"aligned" in lib.flexspmv_error_string(-2)
    assert b"static scratch" in lib.flexspmv_error_string(-8)
    n = ctypes.c_size_t()
    assert lib.flexspmv_partition_bytes(ctypes.c_int64(10), ctypes.c_int64(90), 32, 10, ctypes.byref(n)) == 0 and n.value == 11 * 8
    assert lib.flexspmv_partition_bytes(ctypes.c_int64(10), ctypes.c_int64(90), 64, 10, ctypes.byref(n)) == 0 and n.value == 11 * 16
    assert lib.flexspmv_partition_bytes(ctypes.c_int64(10), ctypes.c_int64(90), 16, 10, ctypes.byref(n)) == -1
    gi = GraphInfo()
    assert lib.flexspmv_spmv_f64_info(ctypes.byref(gi)) == 0
    assert (gi.num_values, gi.num_indices, gi.num_outputs, gi.has_reducer, gi.value_bytes) == (2, 1, 1, 1, 8)
    assert gi.default_tile_items == gi.block_threads * gi.items_per_thread and gi.smem_bytes <= 227 * 1024
    assert lib.flexspmv_edge_sum_f32_info(ctypes.byref(gi)) == 0 and gi.has_reducer == 0 and gi.acc_dim == 2
    d = Desc(1000, 9000, 1000, 32, 0, 0, 0)
    assert lib.flexspmv_spmv_f64_workspace_bytes(ctypes.byref(d), ctypes.byref(n)) == 0 and n.value > 256
    d_bad = Desc(1000, 9000, 1000, 48, 0, 0, 0)
    assert lib.flexspmv_spmv_f64_workspace_bytes(ctypes.byref(d_bad), ctypes.byref(n)) == -1
    d_big = Desc(1 << 30, 1 << 31, 1, 32, 0, 0, 0)
    assert lib.flexspmv_spmv_f64_workspace_bytes(ctypes.byref(d_big), ctypes.byref(n)) == -4
    assert lib.flexspmv_spmv_f64_plan(ctypes.byref(d), None, None, ctypes.c_size_t(0), None) == -3     # no workspace


def test_missing_library_fails_loudly(tmp_path):
    from flexspmv_b200.binding import FlexSpmvError, load_library
    with pytest.raises(FlexSpmvError):
        load_library(str(tmp_path / "nope.so"))


def test_header_is_plain_c_and_links(tmp_path):
    """include/flexspmv.h must be usable from a C translation unit (the drop-in boundary is a C ABI): a C99
    program that includes it and calls a host-only entry point compiles with -pedantic, links against the
    library and runs without a GPU."""
    import shutil
    import subprocess
    from flexspmv_b200.binding import DEFAULT_LIB
    gcc = shutil.which("gcc") or "/usr/bin/gcc"
    src = tmp_path / "use_abi.c"
    src.write_text(
        '#include <stdio.h>\n#include "flexspmv.h"\n'
        "int main(void) {\n"
        "  flexspmv_desc d = {1000, 7000, 1000, 32, 0, 0, 0};\n"
        "  size_t bytes = 0;\n"
        "  flexspmv_graph_info gi;\n"
        "  if (flexspmv_spmv_f64_info(&gi) != 0 || gi.has_reducer != 1) return 2;\n"
        "  if (flexspmv_spmv_f64_workspace_bytes(&d, &bytes) != 0 || bytes == 0) return 3;\n"
        '  printf("%d %zu %s\\n", flexspmv_abi_version(), bytes, flexspmv_error_string(FLEXSPMV_ERR_TIMEOUT));\n'
        "  return 0;\n}\n")
    exe = tmp_path / "use_abi"
    lib_dir = os.path.dirname(DEFAULT_LIB)
    inc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", inc, str(src), "-o", str(exe),
                    "-L", lib_dir, "-lflexspmv_b200", f"-Wl,-rpath,{lib_dir}"], check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert int(out[0]) >= 1 and int(out[1]) > 0
