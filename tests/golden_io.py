"""Loads a tests/golden fixture back into a Problem plus the reference outputs."""
import glob
import os

import numpy as np

from flexspmv_b200.problems import Problem

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load(path):
    z = np.load(path)
    values = {k[4:]: z[k] for k in z.files if k.startswith("val_")}
    indices = {k[4:]: z[k] for k in z.files if k.startswith("idx_")}
    ro = z["row_offsets"] if "row_offsets" in z.files else None
    prob = Problem(str(z["graph"]), values, indices, ro, int(z["num_rows"]), int(z["num_cols"]))
    outs = [z[f"out_{i}"] for i in range(len([k for k in z.files if k.startswith("out_")]))]
    written = {k[8:]: z[k] for k in z.files if k.startswith("written_")}
    return prob, np.dtype(str(z["dtype"])), int(z["threads"]), outs, written
