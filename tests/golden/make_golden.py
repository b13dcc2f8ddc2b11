"""Generates tests/golden/*.npz by running the REFERENCE'S OWN generated CPU operator (compiled from
the reference tree into oracle/_ref by oracle/ref_build.py) on small seeded problems.  The reference
ships no golden vectors of its own, so these fixtures are what pins the oracle on machines where the
reference tree is absent.  Each file holds the inputs, the thread count and the reference outputs.

    python tests/golden/make_golden.py [name ...]     # needs the reference tree; no name = all fixtures
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from flexspmv_b200 import graphs, problems  # noqa: E402
from oracle import ref_build, ref_run  # noqa: E402

CASES = [
    # name, graph, dtype, problem factory, threads
    ("spmv_f64_poisson2d_24", "spmv", np.float64, lambda ir: problems.poisson2d(24), 5),
    ("spmv_f32_cut_rows", "spmv", np.float32, lambda ir: problems.random_problem(ir, 311, 311, 5000, 7, np.float32), 7),
    ("spmv_i64_cut_rows", "spmv", np.int64, lambda ir: problems.random_problem(ir, 97, 97, 3000, 8, np.int64), 3),
    ("spmv_f64_poisson3d_10", "spmv", np.float64, lambda ir: problems.poisson3d(10, offset_dtype=np.int32), 8),
    ("spring_mass_f32_lattice_20", "spring_mass", np.float32, lambda ir: problems.spring_mass(20), 8),
    ("rusanov_f64_mesh_12", "rusanov", np.float64, lambda ir: problems.shallow_water(12), 6),
    ("swe_delta_f64_mesh_12", "swe_delta", np.float64, lambda ir: problems.swe_mesh(12), 6),
    ("swe_delta_f32_cut_rows", "swe_delta", np.float32, lambda ir: problems.random_problem(ir, 200, 200, 4000, 14, np.float32), 5),
    ("swe_boundary_f64_cut_rows", "swe_boundary", np.float64, lambda ir: problems.random_problem(ir, 400, 400, 150, 15, np.float64), 4),
    ("swe_components_i64_mesh_10", "swe_components", np.int64, lambda ir: problems.swe_components_mesh(10), 4),
    ("swe_init_edges_f64_mesh_10", "swe_init_edges", np.float64, lambda ir: problems.swe_init_mesh(10), 4),
    ("swe_init_cells_f64_mesh_10", "swe_init_cells", np.float64, lambda ir: problems.swe_init_cells_mesh(10), 4),
    ("swe_init_boundary_f64_mesh_10", "swe_init_boundary", np.float64, lambda ir: problems.swe_init_boundary_mesh(10), 4),
    ("mixed_dims_f64", "mixed_dims", np.float64, lambda ir: problems.random_problem(ir, 150, 90, 2500, 9, np.float64), 4),
    ("mixed_dims_i64", "mixed_dims", np.int64, lambda ir: problems.random_problem(ir, 150, 90, 2500, 10, np.int64), 4),
    ("ops_zoo_f64", "ops_zoo", np.float64, lambda ir: problems.random_problem(ir, 120, 80, 2000, 11, np.float64), 4),
    ("edge_sum_f32", "edge_sum", np.float32, lambda ir: problems.random_problem(ir, 64, 64, 3000, 12, np.float32), 8),
    ("edge_copy_i64", "edge_copy", np.int64, lambda ir: problems.random_problem(ir, 64, 64, 1000, 13, np.int64), 8),
]


def main():
    if not ref_build.build_all():
        raise SystemExit("reference tree not found: cannot generate golden fixtures")
    only = set(sys.argv[1:])
    for name, gname, dt, make, threads in CASES:
        if only and name not in only:
            continue
        ir = graphs.ALL_GRAPHS[gname]()
        prob = make(ir)
        outs, written = ref_run.run_graph(ir, prob, dt, num_threads=threads)
        blob = {"num_rows": prob.num_rows, "num_cols": prob.num_cols, "threads": threads, "graph": gname,
                "dtype": np.dtype(dt).name}
        for k, v in prob.values.items():
            blob["val_" + k] = v.astype(dt)
        for k, v in prob.indices.items():
            blob["idx_" + k] = v
        if prob.row_offsets is not None:
            blob["row_offsets"] = prob.row_offsets
        for i, o in enumerate(outs):
            blob[f"out_{i}"] = o
        for k, v in written.items():
            blob["written_" + k] = v
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **blob)
        print("wrote", name)


if __name__ == "__main__":
    main()
