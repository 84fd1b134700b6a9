"""Host logic of the receiver-partitioned convolution on CPU ranks (gloo, world sizes 2 and 3): the partition plan,
the halo exchange of sender rows and the return of halo gradients.  The local tensor product is done by the CPU oracle
here; the GPU kernels are exercised by the gpu-marked tests."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import ROOT, single

sys.path.insert(0, ROOT)


def _problem():
    return single("5x2e", "1x1o", "5x3o", "uvu")


def _inputs(n_nodes, seed=0):
    from openequivariance_b200.core.graph import periodic_radius_graph
    p = _problem()
    g = periodic_radius_graph(n_nodes, mean_degree=8.0, cutoff=2.0, seed=seed)
    gen = torch.Generator().manual_seed(seed)
    E = g["rows"].numel()
    X = torch.randn(n_nodes, p.irreps_in1.dim, generator=gen, dtype=torch.float64)
    Y = torch.randn(E, p.irreps_in2.dim, generator=gen, dtype=torch.float64)
    W = torch.randn(E, p.weight_numel, generator=gen, dtype=torch.float64)
    G = torch.randn(n_nodes, p.irreps_out.dim, generator=gen, dtype=torch.float64)
    return p, g, X, Y, W, G


def _rank_main(rank, world, port, n_nodes, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from openequivariance_b200.partition import build_plan, exchange_halo, return_halo_gradients
        from oracle import tp_oracle
        p, g, X, Y, W, G = _inputs(n_nodes)
        plan = build_plan(g["rows"], g["cols"], n_nodes, world, rank)
        x_local = torch.zeros(plan.n_owned + plan.n_halo, X.shape[1], dtype=torch.float64)
        x_local[:plan.n_owned] = X[plan.n0:plan.n1]
        exchange_halo(plan, x_local)
        assert torch.equal(x_local[plan.n_owned:], X[plan.halo_ids])          # halo rows arrived, in the planned order
        Yl, Wl = Y[plan.e0:plan.e1], W[plan.e0:plan.e1]
        xl = x_local.clone().requires_grad_(True)
        yl, wl = Yl.clone().requires_grad_(True), Wl.clone().requires_grad_(True)
        msgs = tp_oracle.tp_forward(p, xl[plan.cols_local], yl, wl)
        Z = torch.zeros(plan.n_owned, msgs.shape[1], dtype=torch.float64).index_add(0, plan.rows_local, msgs)
        Z.backward(G[plan.n0:plan.n1])
        dX = return_halo_gradients(plan, xl.grad.clone())
        a, b = plan.interior
        ea, eb = plan.interior_edges
        interior_ok = bool((plan.cols_local[ea:eb] < plan.n_owned).all())
        torch.save({"Z": Z.detach(), "dX": dX, "dY": yl.grad, "dW": wl.grad, "range": (plan.n0, plan.n1, plan.e0, plan.e1),
                    "interior_ok": interior_ok, "interior": (a, b), "n_halo": plan.n_halo},
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_partitioned_conv_matches_global(world, tmp_path):
    n_nodes = 90
    port = 29600 + world + (os.getpid() % 200)
    mp.spawn(_rank_main, args=(world, port, n_nodes, str(tmp_path)), nprocs=world, join=True)
    from oracle import tp_oracle
    p, g, X, Y, W, G = _inputs(n_nodes)
    x, y, w = X.clone().requires_grad_(True), Y.clone().requires_grad_(True), W.clone().requires_grad_(True)
    Z = tp_oracle.conv_forward(p, x, y, w, g["rows"], g["cols"])
    Z.backward(G)
    covered_nodes, covered_edges, halo_total = 0, 0, 0
    for r in range(world):
        part = torch.load(os.path.join(tmp_path, f"rank{r}.pt"))
        n0, n1, e0, e1 = part["range"]
        covered_nodes += n1 - n0
        covered_edges += e1 - e0
        halo_total += part["n_halo"]
        assert part["interior_ok"]
        torch.testing.assert_close(part["Z"], Z.detach()[n0:n1], rtol=1e-12, atol=1e-12)
        torch.testing.assert_close(part["dX"], x.grad[n0:n1], rtol=1e-12, atol=1e-12)
        torch.testing.assert_close(part["dY"], y.grad[e0:e1], rtol=1e-12, atol=1e-12)
        torch.testing.assert_close(part["dW"], w.grad[e0:e1], rtol=1e-12, atol=1e-12)
    assert covered_nodes == n_nodes and covered_edges == g["rows"].numel() and halo_total > 0


def test_plan_single_rank_has_no_halo():
    from openequivariance_b200.partition import build_plan
    p, g, X, Y, W, G = _inputs(60)
    plan = build_plan(g["rows"], g["cols"], 60, 1, 0)
    assert plan.n_halo == 0 and plan.n_owned == 60 and plan.n_local_edges == g["rows"].numel()
    assert plan.interior == (0, 60)
    assert torch.equal(plan.cols_local, g["cols"]) and torch.equal(plan.rows_local, g["rows"])
