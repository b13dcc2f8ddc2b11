"""Parity metric shared by the tests.

Floating-point rows are compared per row (and per component) as
    |gpu - ref| / max(sum_j |term_ij|, tiny)
i.e. relative to the sum of the magnitudes of the row's per-edge terms, the quantity that bounds the
effect of a different summation order (rows such as 4x - sum(x) cancel, so |y_i| itself is not a
meaningful scale).  Tolerances: 1e-12 (float64), 1e-5 (float32).  Integer outputs, partition
coordinates and per-edge outputs of exactly rounded operations must be bit-identical.
"""
import numpy as np

TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-12}


def row_error(gpu: np.ndarray, ref: np.ndarray, abs_sums: np.ndarray) -> float:
    gpu = np.asarray(gpu, np.float64)
    ref = np.asarray(ref, np.float64)
    finite = np.isfinite(ref)
    if not np.array_equal(np.isfinite(gpu), finite):
        return float("inf")
    if not finite.any():
        return 0.0
    tiny = np.finfo(np.float64).tiny
    scale = np.maximum(np.asarray(abs_sums, np.float64).reshape(ref.shape), tiny)
    err = np.abs(gpu - ref)[finite] / scale[finite]
    return float(err.max()) if err.size else 0.0


def assert_outputs_match(ir, gpu_outs, ref_outs, abs_sums, dtype, what=""):
    dt = np.dtype(dtype)
    assert len(gpu_outs) == len(ref_outs)
    for o, g, r, s in zip(ir.outputs, gpu_outs, ref_outs, abs_sums):
        g = np.asarray(g)
        assert g.shape == r.shape, f"{what} output {o['name']}: shape {g.shape} != {r.shape}"
        if dt.kind == "i":
            assert np.array_equal(g, r), f"{what} output {o['name']}: integer outputs must be bit-exact"
            continue
        tgt = str(o["target"])
        if tgt == "reducer" or "sum" in tgt:
            e = row_error(g, r, s)
            assert e <= TOL[dt], f"{what} output {o['name']}: row error {e:.3e} > {TOL[dt]:.0e}"
        else:
            e = row_error(g, r, np.maximum(np.abs(r.astype(np.float64)), 1e-30))
            assert e <= TOL[dt], f"{what} per-edge output {o['name']}: error {e:.3e}"
