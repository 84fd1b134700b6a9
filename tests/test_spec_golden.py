"""Spec layer and oracle inputs pinned against fixtures generated from the reference's own classes
(tests/golden/make_golden.py)."""
import json
import os

import numpy as np
import pytest

from openequivariance_b200.core import problems as P
from openequivariance_b200.core.graph import CoordGraph
from openequivariance_b200.core.irreps import Irrep, Irreps
from openequivariance_b200.core.problem import TPProblem
from openequivariance_b200.core.weights import oeq_weight_permutation, reorder_weights
from openequivariance_b200.core.wigner import wigner_3j

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_wigner_3j_matches_reference_generator():
    gold = np.load(os.path.join(GOLD, "wigner_3j.npz"))
    assert len(gold.files) > 100
    for key in gold.files:
        l1, l2, l3 = (int(t) for t in key.split("_"))
        mine = wigner_3j(l1, l2, l3)
        assert mine.shape == gold[key].shape
        np.testing.assert_allclose(mine, gold[key], rtol=0, atol=1e-14, err_msg=key)


def _build(spec):
    cls, args, kwargs = spec["cls"], spec["args"], spec["kwargs"]
    if cls == "TPProblem":
        return TPProblem(args[0], args[1], args[2], [tuple(i) for i in args[3]], **kwargs)
    return getattr(P, cls)(*args, **kwargs)


with open(os.path.join(GOLD, "problems.json")) as _f:
    _PROBLEMS = json.load(_f)


@pytest.mark.parametrize("spec", _PROBLEMS["problems"], ids=[s["name"] for s in _PROBLEMS["problems"]])
def test_problem_matches_reference(spec):
    p = _build(spec)
    assert p.irreps_in1.dim == spec["L1_dim"]
    assert p.irreps_in2.dim == spec["L2_dim"]
    assert p.irreps_out.dim == spec["L3_dim"]
    assert str(p.irreps_out) == spec["irreps_out"]
    assert p.weight_numel == spec["weight_numel"]
    assert bool(p.shared_weights) == spec["shared_weights"]
    assert len(p.instructions) == len(spec["instructions"])
    for mine, ref in zip(p.instructions, spec["instructions"]):
        assert [mine.i_in1, mine.i_in2, mine.i_out, mine.connection_mode, bool(mine.has_weight)] == ref[:5]
        assert mine.path_weight == pytest.approx(ref[5], rel=1e-15)
        assert list(mine.path_shape) == ref[6]
    perm = oeq_weight_permutation(p)
    ref_perm = spec["oeq_from_e3nn_perm"]
    if ref_perm == "identity":
        ref_perm = list(range(p.weight_numel))
    assert perm.tolist() == ref_perm
    # round trip, numpy and torch, batched and flat
    w = np.random.default_rng(0).normal(size=(3, p.weight_numel))
    there = reorder_weights(p, w, "forward", perm)
    np.testing.assert_array_equal(there, w[:, perm])
    np.testing.assert_array_equal(reorder_weights(p, there, "backward", perm), w)
    import torch
    wt = torch.from_numpy(w[0].copy())
    back = reorder_weights(p, reorder_weights(p, wt, "forward", perm), "backward", perm)
    assert isinstance(back, torch.Tensor) and torch.equal(back, wt)


def test_normalisation_variants():
    ref = _PROBLEMS["norm_path_case"]
    p = TPProblem("4x1o+2x2e", "2x1o+1x0e", "4x1o+4x2e+4x0e",
                  [(0, 0, 1, "uvu", True, 2.0), (0, 1, 0, "uvu", True), (0, 0, 2, "uvu", True, 0.5), (1, 1, 1, "uvw", True)],
                  irrep_normalization="norm", path_normalization="path", in1_var=[1.0, 2.0], in2_var=[0.5, 1.5],
                  out_var=[1.0, 3.0, 0.25])
    assert p.weight_numel == ref["weight_numel"]
    np.testing.assert_allclose([i.path_weight for i in p.instructions], ref["path_weights"], rtol=1e-15)


def test_coord_graph_matches_reference():
    with open(os.path.join(GOLD, "coord_graph.json")) as f:
        ref = json.load(f)
    g = CoordGraph(np.zeros((ref["n"], 3)), np.array(ref["rows_in"]), np.array(ref["cols_in"]), "g")
    assert g.rows.tolist() == ref["rows"]
    assert g.cols.tolist() == ref["cols"]
    assert g.transpose_perm.tolist() == ref["transpose_perm"]


def test_irreps_behaviour():
    ir = Irreps("128x0e + 3x1o+2e")
    assert str(ir) == "128x0e+3x1o+1x2e" and ir.dim == 128 + 9 + 5 and ir.lmax == 2
    assert [s.start for s in ir.slices()] == [0, 128, 137]
    assert Irrep("3y") == Irrep(3, -1) and Irrep("2y") == Irrep(2, 1)
    assert list(Irrep("1o") * Irrep("2e")) == [Irrep("1o"), Irrep("2o"), Irrep("3o")]
    srt = Irreps("2x2e+1x0e+3x1o").sort()
    assert str(srt.irreps) == "1x0e+3x1o+2x2e" and srt.p == (2, 0, 1) and srt.inv == (1, 2, 0)
    assert str(Irreps("2x1o+3x1o+0x2e+1x0e").simplify()) == "5x1o+1x0e"
    assert Irrep("1o") in ir and Irrep("1e") not in ir and ir.count("1o") == 3
    assert str(Irreps.spherical_harmonics(2)) == "1x0e+1x1o+1x2e"
    with pytest.raises(ValueError):
        Irreps("3x-1e")
    with pytest.raises(ValueError):
        Irrep("1x")
    its = Irrep.iterator(1)
    assert [str(next(its)) for _ in range(4)] == ["0e", "0o", "1o", "1e"]
