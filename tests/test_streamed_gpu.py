"""Chunk-by-chunk ("streamed") convolution against one resident call of the same deterministic kernels and against the
fp64 oracle.  Z, dY and dW must be bit-identical to the resident result whatever the chunk size; dX is a sum of one
partial per chunk and must agree to fp32 rounding (bit-identical with a single chunk)."""
import numpy as np
import pytest
import torch

from helpers import rel_l2, tp_problem_matrix

pytestmark = pytest.mark.gpu


def _setup(n_nodes, seed):
    import openequivariance_b200 as oeq
    from openequivariance_b200.core.graph import periodic_radius_graph, spherical_harmonics

    dev = torch.device("cuda", 0)
    problem = dict(tp_problem_matrix())["mace_medium"]
    g = periodic_radius_graph(n_nodes, mean_degree=10.0, cutoff=2.0, seed=seed, device=dev)
    gen = torch.Generator(device=dev).manual_seed(seed)
    E = g["rows"].numel()
    X = torch.randn(n_nodes, problem.irreps_in1.dim, device=dev, generator=gen)
    Y = spherical_harmonics(3, g["vec"]).float().contiguous()
    W = torch.randn(E, problem.weight_numel, device=dev, generator=gen)
    conv = oeq.TensorProductConv(problem, deterministic=True)
    return dev, problem, g, X, Y, W, conv


@pytest.mark.parametrize("chunk_nodes", [10_000, 257, 64])
def test_streamed_matches_resident(chunk_nodes):
    from openequivariance_b200.streamed import StreamedConv

    n_nodes = 700
    dev, problem, g, X, Y, W, conv = _setup(n_nodes, 3)
    rows, cols, perm = g["rows"], g["cols"], g["transpose_perm"]
    ops = torch.ops.libtorch_tp_jit
    Z_ref = ops.jit_conv_forward(conv.kernel, conv.hash, X, Y, W, conv.L3_dim, rows, cols, conv.workspace_buffer, perm)
    G = 0.5 * Z_ref            # cotangent of the separable loss 0.25 * |Z|^2
    dX_ref, dY_ref, dW_ref = ops.jit_conv_backward(conv.kernel, conv.hash, X, Y, W, G, rows, cols, conv.workspace_buffer, perm)

    sc = StreamedConv(conv, rows, cols, n_nodes, chunk_nodes, dev)
    Z, dW, dY, dX = torch.empty_like(Z_ref), torch.empty_like(W), torch.empty_like(Y), torch.empty_like(X)

    def weights(c, out):
        p = sc.plans[c]
        out.copy_(W[p.e0:p.e1])

    def cotangent(c, Z_c):
        Z_c.mul_(0.5)          # in place: the chunk's Z buffer now holds G
        return Z_c

    def on_chunk(c, p, Z_c, dW_c):
        Z[p.n0:p.n1] = Z_c * 2.0   # exact: undo the halving
        dW[p.e0:p.e1] = dW_c

    sc.step(X, Y, weights, cotangent, dX, dY, on_chunk)
    torch.cuda.synchronize()
    assert torch.equal(Z, Z_ref)
    assert torch.equal(dY, dY_ref)
    assert torch.equal(dW, dW_ref)
    assert rel_l2(dX.cpu().numpy(), dX_ref.cpu().numpy()) <= 1e-6
    if len(sc.plans) == 1:
        assert torch.equal(dX, dX_ref)


def test_streamed_against_oracle_fp64_subbox():
    """The accuracy pass of the large configuration: a sub-box of the graph, streamed in chunks, against the fp64 oracle."""
    from oracle import tp_oracle
    from openequivariance_b200.streamed import StreamedConv

    n_nodes = 300
    dev, problem, g, X, Y, W, conv = _setup(n_nodes, 5)
    rows, cols = g["rows"], g["cols"]
    sc = StreamedConv(conv, rows, cols, n_nodes, 97, dev)
    Z = torch.empty(n_nodes, problem.irreps_out.dim, device=dev)
    dX, dY, dW = torch.empty_like(X), torch.empty_like(Y), torch.empty_like(W)

    def on_chunk(c, p, Z_c, dW_c):
        Z[p.n0:p.n1] = Z_c
        dW[p.e0:p.e1] = dW_c

    sc.step(X, Y, lambda c, out: out.copy_(W[sc.plans[c].e0:sc.plans[c].e1]), lambda c, Z_c: Z_c, dX, dY, on_chunk)
    torch.cuda.synchronize()
    Xd, Yd, Wd = (t.double().cpu().requires_grad_(True) for t in (X, Y, W))
    Zo = tp_oracle.conv_forward(problem, Xd, Yd, Wd, rows.cpu(), cols.cpu())
    (0.5 * Zo.square().sum()).backward()    # dL/dZ = Z, the cotangent used above
    for got, want in ((Z, Zo.detach()), (dX, Xd.grad), (dY, Yd.grad), (dW, Wd.grad)):
        assert rel_l2(got.cpu().numpy(), want.numpy()) <= 1e-5
