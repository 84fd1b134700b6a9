"""Outputs of the unmodified reference (its JIT CUDA kernels, run once on a B200 by tests/golden/make_reference_gpu_golden.py)
pin the CPU oracle -- this is the contraction itself, weight reordering included -- and, on a GPU, this library's kernels."""
import os

import numpy as np
import pytest
import torch

from helpers import rel_l2
from openequivariance_b200.core import problems as P
from openequivariance_b200.core.irreps import Irreps
from openequivariance_b200.core.problem import TPProblem
from oracle import tp_oracle

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_gpu.npz"))


def _get(prefix, key):
    return GOLD[f"{prefix}__{key}".replace("/", "__")]


TP_CASES = {
    "readme": lambda: TPProblem(Irreps("1x2e"), Irreps("1x3e"), Irreps("1x2e"), [(0, 0, 0, "uvu", True)],
                                shared_weights=False, internal_weights=False),
    "uvu_16x1e_3x1e": lambda: P.SingleInstruction("16x1e", "3x1e", "16x1e", "uvu"),
    "uvw_40_3_33": lambda: P.SingleInstruction("40x1o", "3x2e", "33x1o", "uvw"),
    "ctpp_32": lambda: P.ChannelwiseTPP("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e"),
    "fc_shared": lambda: P.FullyConnectedTPProblem("8x0e+8x1o+8x1e", "1x0e+1x1o", "8x0e+8x1o+8x1e", shared_weights=True),
}
# the fixtures are fp32 results of the reference's kernels: agreement with the fp64 oracle is limited by their rounding
TOL = 2e-6


@pytest.mark.parametrize("name", list(TP_CASES))
def test_oracle_matches_reference_kernels_tp(name):
    p = TP_CASES[name]()
    x, y, w, g = (_get(f"tp/{name}", k) for k in ("x", "y", "w", "g"))
    assert rel_l2(tp_oracle.forward(p, x, y, w), _get(f"tp/{name}", "z")) <= TOL
    dx, dy, dw = tp_oracle.backward(p, x, y, w, g)
    assert rel_l2(dx, _get(f"tp/{name}", "dx")) <= TOL
    assert rel_l2(dy, _get(f"tp/{name}", "dy")) <= TOL
    assert rel_l2(dw, _get(f"tp/{name}", "dw")) <= TOL


def _conv_problem():
    return P.ChannelwiseTPP("32x0e+32x1o", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e")


@pytest.mark.parametrize("mode", ["atomic", "det"])
def test_oracle_matches_reference_kernels_conv(mode):
    p = _conv_problem()
    x, y, w, g, rows, cols = (_get("conv", k) for k in ("x", "y", "w", "g", "rows", "cols"))
    z = tp_oracle.forward(p, x, y, w, graph=(rows, cols))
    assert rel_l2(z, _get(f"conv/{mode}", "z")) <= TOL
    dx, dy, dw = tp_oracle.backward(p, x, y, w, g, graph=(rows, cols))
    for mine, key in ((dx, "dx"), (dy, "dy"), (dw, "dw")):
        assert rel_l2(mine, _get(f"conv/{mode}", key)) <= TOL * 2


def test_coord_graph_fixture_is_consistent():
    from openequivariance_b200.core.graph import transpose_permutation
    rows, cols, perm = (_get("conv", k) for k in ("rows", "cols", "perm"))
    assert np.array_equal(transpose_permutation(rows, cols), perm)


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(TP_CASES))
def test_kernels_match_reference_kernels_tp(name):
    import openequivariance_b200 as oeq
    p = TP_CASES[name]()
    tp = oeq.TensorProduct(p)
    x, y, w, g = (_get(f"tp/{name}", k) for k in ("x", "y", "w", "g"))
    z = np.zeros_like(_get(f"tp/{name}", "z"))
    tp.forward_cpu(x, y, z, w)
    assert rel_l2(z, _get(f"tp/{name}", "z")) <= TOL
    dx, dy, dw = np.zeros_like(x), np.zeros_like(y), np.zeros_like(w)
    tp.backward_cpu(x, dx, y, dy, g, w, dw)
    for mine, key in ((dx, "dx"), (dy, "dy"), (dw, "dw")):
        assert rel_l2(mine, _get(f"tp/{name}", key)) <= TOL * 2


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["atomic", "det"])
def test_kernels_match_reference_kernels_conv(mode):
    import openequivariance_b200 as oeq

    class G:
        pass

    graph = G()
    graph.rows, graph.cols, graph.transpose_perm = (_get("conv", k) for k in ("rows", "cols", "perm"))
    p = _conv_problem()
    conv = oeq.TensorProductConv(p, deterministic=mode == "det")
    x, y, w, g = (_get("conv", k) for k in ("x", "y", "w", "g"))
    z = np.zeros_like(_get(f"conv/{mode}", "z"))
    conv.forward_cpu(x, y, w, z, graph)
    assert rel_l2(z, _get(f"conv/{mode}", "z")) <= TOL
    dx, dy, dw = np.zeros_like(x), np.zeros_like(y), np.zeros_like(w)
    conv.backward_cpu(x, dx, y, dy, w, dw, g, graph)
    for mine, key in ((dx, "dx"), (dy, "dy"), (dw, "dw")):
        assert rel_l2(mine, _get(f"conv/{mode}", key)) <= TOL * 2


# ---- second order, on the benchmark signatures themselves ------------------------------------------------------------
# tests/golden/reference_gpu_second_order.npz (made by make_reference_gpu_golden.py --second-order): forward, backward and
# double backward of the MACE-like and the NequIP-like problem (and a smaller channelwise one) as the unmodified reference's
# kernels computed them on a B200.

GOLD2 = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_gpu_second_order.npz"))
TP2_CASES = {
    "mace_like": lambda: P.mace_like_problem(),
    "nequip_like": lambda: P.nequip_like_problem(),
    "ctpp_32": lambda: P.ChannelwiseTPP("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e"),
}
# fp32 results of the reference's kernels against the fp64 oracle (measured: at most 1.7e-7 over all cases and orders)
TOL2 = 1e-6


def _get2(name, key):
    return GOLD2[f"tp2__{name}__{key}"]


@pytest.mark.parametrize("name", list(TP2_CASES))
def test_oracle_matches_reference_kernels_second_order(name):
    p = TP2_CASES[name]()
    x, y, w, g, x2, y2, w2 = (_get2(name, k) for k in ("x", "y", "w", "g", "x2", "y2", "w2"))
    assert rel_l2(tp_oracle.forward(p, x, y, w), _get2(name, "z")) <= TOL2
    for mine, key in zip(tp_oracle.backward(p, x, y, w, g), ("dx", "dy", "dw")):
        assert rel_l2(mine, _get2(name, key)) <= TOL2, key
    for mine, key in zip(tp_oracle.double_backward(p, x, y, w, g, x2, y2, w2), ("ddx", "ddy", "ddw", "ddg")):
        assert rel_l2(mine, _get2(name, key)) <= TOL2, key


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(TP2_CASES))
def test_kernels_match_reference_kernels_second_order(name):
    import openequivariance_b200 as oeq
    p = TP2_CASES[name]()
    tp = oeq.TensorProduct(p)
    shared = p.shared_weights
    x, y, w, g, x2, y2, w2 = (_get2(name, k) for k in ("x", "y", "w", "g", "x2", "y2", "w2"))
    wk, w2k = tp.reorder_weights_from_e3nn(w, not shared), tp.reorder_weights_from_e3nn(w2, not shared)
    got = tp.double_backward_cpu(x, y, g, wk, w2k, x2, y2)           # kernel-order weights in and out
    got = (got[0], got[1], tp.reorder_weights_to_e3nn(got[2], not shared), got[3])
    for mine, key in zip(got, ("ddx", "ddy", "ddw", "ddg")):
        assert rel_l2(mine, _get2(name, key)) <= TOL2 * 2, key      # two fp32 implementations against each other
