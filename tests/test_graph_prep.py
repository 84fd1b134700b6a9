"""Device-side graph preparation against the NumPy ``CoordGraph`` (the reference's ordering, pinned by
``tests/golden/coord_graph.json``): index arrays must be identical, for shuffled input, duplicate edges, int32 ids."""
import numpy as np
import pytest
import torch

from openequivariance_b200 import CoordGraph, prepare_graph


def _random_edges(n_nodes, n_edges, seed, dtype):
    rng = np.random.default_rng(seed)
    rows = rng.integers(0, n_nodes, n_edges).astype(dtype)
    cols = rng.integers(0, n_nodes, n_edges).astype(dtype)
    return rows, cols


def _check(device, dtype):
    n_nodes = 97
    rows, cols = _random_edges(n_nodes, 1500, 3, dtype)      # many duplicate (row, col) pairs
    want = CoordGraph(np.zeros((n_nodes, 3)), rows, cols, "t")
    got = prepare_graph(torch.tensor(rows, device=device), torch.tensor(cols, device=device), n_nodes)
    assert got["rows"].dtype == torch.tensor(rows).dtype
    assert np.array_equal(got["rows"].cpu().numpy(), want.rows)
    assert np.array_equal(got["cols"].cpu().numpy(), want.cols)
    # duplicates make the permutation ambiguous in principle; both sides sort stably, so it must match exactly
    assert np.array_equal(got["transpose_perm"].cpu().numpy(), want.transpose_perm)
    assert np.array_equal(got["order"].cpu().numpy(), want.edge_order)
    # the permutation lists the sorted edges in (col, row) order
    r, c, p = got["rows"].cpu().numpy(), got["cols"].cpu().numpy(), got["transpose_perm"].cpu().numpy()
    keys = list(zip(c[p].tolist(), r[p].tolist()))
    assert keys == sorted(keys)


@pytest.mark.parametrize("dtype", [np.int64, np.int32])
def test_prepare_graph_cpu(dtype):
    _check("cpu", dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.int64, np.int32])
def test_prepare_graph_gpu(dtype):
    _check("cuda", dtype)


@pytest.mark.gpu
def test_prepared_graph_drives_the_deterministic_conv():
    """Shuffled edges -> prepare_graph -> deterministic conv equals the conv on the generator's own sorted list."""
    import openequivariance_b200 as oeq
    from helpers import tp_problem_matrix
    from openequivariance_b200.core.graph import periodic_radius_graph, spherical_harmonics

    dev = torch.device("cuda", 0)
    problem = dict(tp_problem_matrix())["mace_medium"]
    n_nodes = 300
    g = periodic_radius_graph(n_nodes, mean_degree=10.0, cutoff=2.0, seed=4, device=dev)
    E = g["rows"].numel()
    gen = torch.Generator(device=dev).manual_seed(1)
    X = torch.randn(n_nodes, problem.irreps_in1.dim, device=dev, generator=gen)
    Y = spherical_harmonics(3, g["vec"]).float().contiguous()
    W = torch.randn(E, problem.weight_numel, device=dev, generator=gen)
    conv = oeq.TensorProductConv(problem, deterministic=True)
    Z_ref = conv(X, Y, W, g["rows"], g["cols"], g["transpose_perm"])
    shuffle = torch.randperm(E, device=dev, generator=gen)
    prep = prepare_graph(g["rows"][shuffle], g["cols"][shuffle], n_nodes)
    o = prep["order"]
    Z = conv(X, Y[shuffle][o].contiguous(), W[shuffle][o].contiguous(), prep["rows"], prep["cols"], prep["transpose_perm"])
    assert torch.equal(Z, Z_ref)
