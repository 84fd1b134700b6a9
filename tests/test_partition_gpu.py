"""GPU kernels under the receiver partition, all ranks played by one process on one GPU (halo rows copied directly
instead of travelling over NCCL): the forward must be bit-identical to the single-GPU deterministic result for every
world size, dY/dW too, and dX must agree to fp32 rounding (bit-identical away from the partition boundaries)."""
import numpy as np
import pytest
import torch

from helpers import rel_l2, tp_problem_matrix

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [1, 2, 3])
def test_partitioned_kernels_match_single_gpu(world):
    import openequivariance_b200 as oeq
    from openequivariance_b200.core.graph import periodic_radius_graph, spherical_harmonics
    from openequivariance_b200.partition import PartitionedConv, build_plan

    dev = torch.device("cuda", 0)
    problem = dict(tp_problem_matrix())["mace_medium"]
    n_nodes = 600
    g = periodic_radius_graph(n_nodes, mean_degree=10.0, cutoff=2.0, seed=2, device=dev)
    rows, cols, perm = g["rows"], g["cols"], g["transpose_perm"]
    E = rows.numel()
    gen = torch.Generator(device=dev).manual_seed(0)
    X = torch.randn(n_nodes, problem.irreps_in1.dim, device=dev, generator=gen)
    Y = spherical_harmonics(3, g["vec"]).float().contiguous()
    W = torch.randn(E, problem.weight_numel, device=dev, generator=gen)
    G = torch.randn(n_nodes, problem.irreps_out.dim, device=dev, generator=gen)
    conv = oeq.TensorProductConv(problem, deterministic=True)
    ops = torch.ops.libtorch_tp_jit
    Z_ref = ops.jit_conv_forward(conv.kernel, conv.hash, X, Y, W, conv.L3_dim, rows, cols, conv.workspace_buffer, perm)
    dX_ref, dY_ref, dW_ref = ops.jit_conv_backward(conv.kernel, conv.hash, X, Y, W, G, rows, cols, conv.workspace_buffer, perm)

    def copy_halo(pl, x_local):
        if pl.n_halo:
            x_local[pl.n_owned:].copy_(X[pl.halo_ids])
        return []

    plans = [build_plan(rows, cols, n_nodes, world, r) for r in range(world)]
    parts, dx_locals = [], []
    for plan in plans:
        pc = PartitionedConv(conv, plan, dev,
                             exchange=copy_halo,
                             give_back=lambda pl, dx: dx)          # keep the local dX; combined below in rank order
        Z = pc.forward(X[plan.n0:plan.n1], Y[plan.e0:plan.e1].contiguous(), W[plan.e0:plan.e1].contiguous())
        dx_local, dY, dW = pc.backward(G[plan.n0:plan.n1].contiguous())
        torch.cuda.synchronize()
        assert torch.equal(Z, Z_ref[plan.n0:plan.n1])
        assert torch.equal(dY, dY_ref[plan.e0:plan.e1])
        assert torch.equal(dW, dW_ref[plan.e0:plan.e1])
        dx_locals.append(dx_local)
        parts.append(plan)
    dX = torch.zeros_like(X)
    for plan, dxl in zip(parts, dx_locals):                        # owners first, then halo partials in rank order
        dX[plan.n0:plan.n1] += dxl[:plan.n_owned]
    for plan, dxl in zip(parts, dx_locals):
        if plan.n_halo:
            dX.index_add_(0, plan.halo_ids, dxl[plan.n_owned:])
    assert rel_l2(dX.cpu().numpy(), dX_ref.cpu().numpy()) <= 1e-6
    if world == 1:
        assert torch.equal(dX, dX_ref)
