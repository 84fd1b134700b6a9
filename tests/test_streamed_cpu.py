"""Host logic of the streamed convolution: the chunk plans partition the receiver-sorted edge list, renumber each chunk's
senders densely, and their sender-major permutations list every chunk edge exactly once in (sender, receiver) order."""
import numpy as np
import pytest
import torch

from openequivariance_b200.core.graph import periodic_radius_graph
from openequivariance_b200.streamed import plan_chunks


@pytest.mark.parametrize("chunk_nodes", [1, 37, 200, 10_000])
def test_chunk_plans_cover_the_graph(chunk_nodes):
    n_nodes = 400
    g = periodic_radius_graph(n_nodes, mean_degree=8.0, cutoff=2.0, seed=11)
    rows, cols = g["rows"], g["cols"]
    E = rows.numel()
    plans = plan_chunks(rows, cols, n_nodes, chunk_nodes)
    assert plans[0].n0 == 0 and plans[-1].n1 == n_nodes
    assert plans[0].e0 == 0 and plans[-1].e1 == E
    for a, b in zip(plans[:-1], plans[1:]):
        assert a.n1 == b.n0 and a.e1 == b.e0
    for p in plans:
        r, c = rows[p.e0:p.e1], cols[p.e0:p.e1]
        assert p.n1 - p.n0 <= chunk_nodes
        if p.e1 > p.e0:
            assert int(r.min()) >= p.n0 and int(r.max()) < p.n1
        # dense sender numbering maps back to the global ids
        assert torch.equal(p.senders[p.cols_local], c)
        assert torch.equal(p.rows_local + p.n0, r)
        assert torch.equal(torch.unique(p.senders), p.senders)
        # sender-major permutation: a permutation of the chunk's edges, sorted by (sender, receiver), stable
        perm = p.perm_local.numpy()
        assert sorted(perm.tolist()) == list(range(p.e1 - p.e0))
        keys = [(int(p.cols_local[k]), int(p.rows_local[k])) for k in perm]
        assert keys == sorted(keys)


def test_empty_receivers_and_empty_graph():
    rows = torch.tensor([2, 2, 5], dtype=torch.int64)
    cols = torch.tensor([0, 7, 2], dtype=torch.int64)
    plans = plan_chunks(rows, cols, 8, 2)          # receivers 0-1, 6-7 have no edges
    assert [(p.e0, p.e1) for p in plans] == [(0, 0), (0, 2), (2, 3), (3, 3)]
    assert plans[0].senders.numel() == 0 and plans[1].senders.tolist() == [0, 7]
    empty = torch.zeros(0, dtype=torch.int64)
    plans = plan_chunks(empty, empty, 3, 2)
    assert [(p.n0, p.n1, p.e0, p.e1) for p in plans] == [(0, 2, 0, 0), (2, 3, 0, 0)]


def test_drivers_refuse_other_precisions_and_index_widths():
    """fp64 problems and int32 index arrays would make the kernels read the drivers' fp32 / int64 buffers past their
    end; both constructors must refuse them before anything is launched."""
    import types

    import numpy as np
    import pytest
    import torch

    from openequivariance_b200.partition import PartitionedConv, build_plan
    from openequivariance_b200.streamed import StreamedConv

    def fake_conv(dt):
        return types.SimpleNamespace(deterministic=True, config=types.SimpleNamespace(irrep_dtype=dt, weight_dtype=dt))

    rows = torch.tensor([0, 0, 1, 2, 2, 3], dtype=torch.int64)
    cols = torch.tensor([1, 2, 0, 0, 3, 2], dtype=torch.int64)
    plan = build_plan(rows, cols, 4, 1, 0)
    with pytest.raises(TypeError, match="float32"):
        PartitionedConv(fake_conv(np.float64), plan, "cpu")
    with pytest.raises(TypeError, match="float32"):
        StreamedConv(fake_conv(np.float64), rows, cols, 4, 2, "cpu")
    with pytest.raises(TypeError, match="int64"):
        StreamedConv(fake_conv(np.float32), rows.int(), cols.int(), 4, 2, "cpu")
    plan.cols_local = plan.cols_local.int()
    with pytest.raises(TypeError, match="int64"):
        PartitionedConv(fake_conv(np.float32), plan, "cpu")
