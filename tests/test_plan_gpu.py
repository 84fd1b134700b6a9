"""The device-side planner of the partitioned / streamed drivers (csrc/partition_plan.cuh) against the torch restatement
it replaces: identical index arrays for every rank of several world sizes, for chunk plans, and for degenerate cases."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _graph(n_nodes, seed, degree=12.0):
    from openequivariance_b200.core.graph import periodic_radius_graph
    g = periodic_radius_graph(n_nodes, mean_degree=degree, cutoff=5.0, seed=seed, device=torch.device("cuda", 0))
    return g["rows"], g["cols"]


def _same_plan(dev_plan, cpu_plan):
    for name in ("n0", "n1", "e0", "e1", "recv_counts", "interior", "interior_edges"):
        assert getattr(dev_plan, name) == getattr(cpu_plan, name), name
    for name in ("halo_ids", "rows_local", "cols_local", "perm_local", "rows_mid", "rows_right"):
        assert torch.equal(getattr(dev_plan, name).cpu(), getattr(cpu_plan, name)), name
    assert len(dev_plan.send_ids) == len(cpu_plan.send_ids)
    for a, b in zip(dev_plan.send_ids, cpu_plan.send_ids):
        assert torch.equal(a.cpu(), b)


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_device_partition_plan_equals_host_plan(world):
    from openequivariance_b200 import native
    from openequivariance_b200.partition import build_plan
    rows, cols = _graph(3000, seed=world)
    for rank in range(world):
        before = native.launch_count()
        dev_plan = build_plan(rows, cols, 3000, world, rank)
        assert native.launch_count() > before          # the library's kernels did the work
        _same_plan(dev_plan, build_plan(rows.cpu(), cols.cpu(), 3000, world, rank))


def test_device_partition_plan_without_edges_into_a_rank():
    """A rank whose receivers have no edges, and a graph without any halo (two disconnected halves)."""
    from openequivariance_b200.partition import build_plan
    rows = torch.tensor([0, 0, 1, 2, 2, 3], device="cuda")
    cols = torch.tensor([1, 0, 0, 3, 2, 2], device="cuda")
    for world, n in ((2, 4), (2, 8), (4, 8)):
        for rank in range(world):
            _same_plan(build_plan(rows, cols, n, world, rank), build_plan(rows.cpu(), cols.cpu(), n, world, rank))


@pytest.mark.parametrize("chunk_nodes", [700, 3000, 5000])
def test_device_chunk_plans_equal_host_plans(chunk_nodes):
    from openequivariance_b200.streamed import plan_chunks
    rows, cols = _graph(3000, seed=7)
    dev_plans, cpu_plans = plan_chunks(rows, cols, 3000, chunk_nodes), plan_chunks(rows.cpu(), cols.cpu(), 3000, chunk_nodes)
    assert len(dev_plans) == len(cpu_plans)
    for d, c in zip(dev_plans, cpu_plans):
        assert (d.n0, d.n1, d.e0, d.e1) == (c.n0, c.n1, c.e0, c.e1)
        for name in ("senders", "rows_local", "cols_local", "perm_local"):
            assert torch.equal(getattr(d, name).cpu(), getattr(c, name)), name
