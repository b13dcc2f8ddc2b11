"""TEST INFRASTRUCTURE ONLY: numpy restatement of one time step of the reference's shallow-water model,
``ShallowWaterEquation.forward`` with ``face_reconstruct`` and ``delta``
(shallow_water_equation/swe_main.py:83-146), with ``esr.Selector`` as fancy indexing and ``esr.Reducer``
as an unordered scatter-add.  Parity unpinned at the model level: the reference model needs the
third-party ``easier`` package and its HDF5 meshes, neither of which is available; the two fused graphs
inside it (graphs.swe_delta_graph, graphs.swe_boundary_graph) are pinned separately against the
reference's generated CPU operator."""
import numpy as np


def _scatter(idx, values, n):
    out = np.zeros(n, dtype=values.dtype)
    np.add.at(out, idx, values)
    return out


def delta(m, h, uh, vh):
    """swe_main.py:86-119"""
    src, dst, b, nc = m["src"], m["dst"], m["bcells"], m["area"].shape[0]
    rec = lambda phi: (1.0 - m["alpha"]) * phi[src] + m["alpha"] * phi[dst]      # face_reconstruct, :83-85
    h_f, uh_f, vh_f = rec(h), rec(uh), rec(vh)
    u_f, v_f = uh_f / h_f, vh_f / h_f
    h_f_square = 0.5 * h_f * h_f
    uh_f_times_sx, vh_f_times_sy = uh_f * m["sx"], vh_f * m["sy"]
    gather_b_h_square = 0.5 * h[b] ** 2
    delta_h = -(_scatter(dst, uh_f_times_sx + vh_f_times_sy, nc)) / m["area"]
    delta_uh = -(_scatter(dst, (u_f * uh_f + h_f_square) * m["sx"] + u_f * vh_f_times_sy, nc)
                 + _scatter(b, gather_b_h_square * m["bsx"], nc)) / m["area"]
    delta_vh = -(_scatter(dst, v_f * uh_f_times_sx + (v_f * vh_f + h_f_square) * m["sy"], nc)
                 + _scatter(b, gather_b_h_square * m["bsy"], nc)) / m["area"]
    return delta_h, delta_uh, delta_vh


def forward(m, h, uh, vh, dt=0.005):
    """One classical Runge-Kutta step, swe_main.py:121-146.  Returns the new (h, uh, vh)."""
    d1 = delta(m, h, uh, vh)
    d2 = delta(m, h + 0.5 * dt * d1[0], uh + 0.5 * dt * d1[1], vh + 0.5 * dt * d1[2])
    d3 = delta(m, h + 0.5 * dt * d2[0], uh + 0.5 * dt * d2[1], vh + 0.5 * dt * d2[2])
    d4 = delta(m, h + dt * d3[0], uh + dt * d3[1], vh + dt * d3[2])
    return tuple(x + dt / 6 * (a + b + c + d) for x, a, b, c, d in zip((h, uh, vh), d1, d2, d3, d4))
