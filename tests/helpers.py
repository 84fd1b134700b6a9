"""Shared helpers for the parity tests: seeded inputs, error metrics, problem lists."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from openequivariance_b200.core import problems as P  # noqa: E402
from openequivariance_b200.core.problem import TPProblem  # noqa: E402

# Tolerances.  north_star: relative L2 <= 1e-5 (fp32) / 1e-12 (fp64) against the fp64 oracle; the reference's own
# absolute L-infinity thresholds on uniform[0,1) inputs (tests/batch_test.py:30-36, tests/conv_test.py:50-56) are
# checked in addition for first and second order.
REL_L2 = {np.float32: 1e-5, np.float64: 1e-12}
ABS_LINF = {"fwd": 1e-5, "bwd": 3e-4, "dbl": 3e-4, "triple": 5e-4}


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    denom = np.linalg.norm(b.ravel())
    return float(np.linalg.norm((a - b).ravel()) / denom) if denom > 0 else float(np.linalg.norm(a.ravel()))


def uniform_inputs(problem, batch, seed=12345, n_rows=None):
    """uniform[0,1) buffers in the style of the reference's test_buffers.py (x rows = n_rows for convolutions)."""
    rng = np.random.default_rng(seed)
    dt = problem.irrep_dtype
    nx = batch if n_rows is None else n_rows
    x = rng.uniform(size=(nx, problem.irreps_in1.dim)).astype(dt)
    y = rng.uniform(size=(batch, problem.irreps_in2.dim)).astype(dt)
    wshape = (problem.weight_numel,) if problem.shared_weights else (batch, problem.weight_numel)
    w = rng.uniform(size=wshape).astype(dt)
    g = rng.uniform(size=(nx, problem.irreps_out.dim)).astype(dt)
    x2 = rng.uniform(size=x.shape).astype(dt)
    y2 = rng.uniform(size=y.shape).astype(dt)
    w2 = rng.uniform(size=w.shape).astype(dt)
    return x, y, w, g, x2, y2, w2


def with_dtype(problem, dt):
    q = problem.clone()
    q.irrep_dtype = dt
    q.weight_dtype = dt
    return q


def single(in1, in2, out, mode, shared=False, layout="mul_ir"):
    return TPProblem(in1, in2, out, [(0, 0, 0, mode, True)], shared_weights=shared, internal_weights=False,
                     layout=layout, label=f"{in1} x {in2} -> {out} {mode}")


def tp_problem_matrix():
    """(id, problem) pairs covering the reference's batch-test matrix (tests/batch_test.py:130-283) in reduced form."""
    out = []
    out.append(("readme", P.readme_problem()))
    for tag, (m1, m2, m3) in {"m1": (1, 1, 1), "m2": (2, 1, 2), "m5": (5, 1, 5), "m32": (32, 1, 32), "m33v3": (33, 3, 33),
                              "m70v2": (70, 2, 70), "m16v5": (16, 5, 16)}.items():
        out.append((f"uvu_{tag}", single(f"{m1}x2e", f"{m2}x1o", f"{m3}x3o", "uvu")))
    for l1, l2, l3 in [(1, 1, 1), (2, 2, 2), (4, 3, 1), (5, 2, 5), (7, 2, 5)]:
        p1, p2 = "e", "e"
        out.append((f"uvu_l{l1}{l2}{l3}", single(f"8x{l1}e", f"1x{l2}e", f"8x{l3}e", "uvu")))
    for tag, (m1, m2, m3) in {"m1": (1, 1, 1), "m4": (4, 2, 3), "m32": (32, 1, 32), "m40": (40, 3, 33), "m64": (64, 1, 64)}.items():
        out.append((f"uvw_{tag}", single(f"{m1}x1o", f"{m2}x2e", f"{m3}x1o", "uvw")))
    for l1, l2, l3 in [(2, 2, 2), (4, 3, 1), (5, 2, 5)]:
        out.append((f"uvw_l{l1}{l2}{l3}", single(f"6x{l1}e", f"2x{l2}e", f"5x{l3}e", "uvw")))
    out.append(("uvu_shared", single("20x1e", "1x1e", "20x1e", "uvu", shared=True)))
    out.append(("uvw_shared", single("12x1e", "2x1e", "9x1e", "uvw", shared=True)))
    out.append(("uvu_ir_mul", single("24x2e", "2x1o", "24x3o", "uvu", layout="ir_mul")))
    out.append(("uvu_ir_mul_fast", single("64x2e", "1x1o", "64x3o", "uvu", layout="ir_mul")))
    ctpp_ir_mul = P.nequip_problems()[4].clone()
    ctpp_ir_mul.layout = "ir_mul"
    out.append(("ctpp_ir_mul", ctpp_ir_mul))
    out.append(("multi_out", TPProblem("6x1o+4x2e", "1x1o+1x0e", "6x1o+6x2e+4x2e",
                                       [(0, 0, 1, "uvu", True), (0, 1, 0, "uvu", True, 0.7), (1, 1, 2, "uvu", True),
                                        (0, 0, 1, "uvu", True, 0.5)], shared_weights=False, internal_weights=False)))
    out.append(("mace_like", P.mace_like_problem()))
    out.append(("mace_medium", P.mace_problems()[1]))
    out.append(("nequip_like", P.nequip_like_problem()))
    out.append(("nequip_water_uvu", P.nequip_problems()[4]))
    out.append(("diffdock1", P.diffdock_problems()[0]))
    out.append(("tetris_poly2", P.e3nn_torch_tetris_poly_problems()[1]))
    return out


def small_graph(n_nodes=40, mean_degree=6.0, seed=3, isolated=(5, 17)):
    """Small symmetric periodic graph with a few isolated nodes (empty receiver segments)."""
    from openequivariance_b200.core.graph import periodic_radius_graph, sort_edges
    g = periodic_radius_graph(n_nodes, mean_degree=mean_degree, cutoff=2.0, seed=seed)
    rows, cols, vec = g["rows"], g["cols"], g["vec"]
    keep = torch.ones(rows.numel(), dtype=torch.bool)
    for node in isolated:
        keep &= (rows != node) & (cols != node)
    rows, cols, vec = rows[keep], cols[keep], vec[keep]
    order, perm = sort_edges(rows, cols)
    return {"n_nodes": n_nodes, "rows": rows[order].contiguous(), "cols": cols[order].contiguous(),
            "vec": vec[order].contiguous(), "transpose_perm": perm.contiguous()}
