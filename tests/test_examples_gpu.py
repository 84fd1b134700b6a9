"""The reference's README / tutorial snippets (tests/example_test.py:5-82) with this package: a tensor product from
irreps strings, the atomic convolution on an explicit edge list, and the deterministic convolution after sorting the edges
by receiver (plain ``argsort`` in place of torch_geometric's ``EdgeIndex.sort_by``), each checked against the oracle."""
import numpy as np
import pytest
import torch

from helpers import rel_l2
from oracle import tp_oracle

pytestmark = pytest.mark.gpu


def test_tutorial_snippets():
    import openequivariance_b200 as oeq
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    batch_size = 1000
    X_ir, Y_ir, Z_ir = oeq.Irreps("1x2e"), oeq.Irreps("1x3e"), oeq.Irreps("1x2e")
    X = torch.rand(batch_size, X_ir.dim, device="cuda", generator=gen)
    Y = torch.rand(batch_size, Y_ir.dim, device="cuda", generator=gen)
    instructions = [(0, 0, 0, "uvu", True)]
    problem = oeq.TPProblem(X_ir, Y_ir, Z_ir, instructions, shared_weights=False, internal_weights=False)
    W = torch.rand(batch_size, problem.weight_numel, device="cuda", generator=gen)
    tp_fast = oeq.TensorProduct(problem)
    Z = tp_fast(X, Y, W)
    assert Z.shape == (batch_size, Z_ir.dim)
    want = tp_oracle.forward(problem, X.cpu().numpy(), Y.cpu().numpy(), tp_fast.reorder_weights_to_e3nn(W.cpu().numpy()))
    assert rel_l2(Z.cpu().numpy(), want) <= 1e-5

    # graph convolution: receivers, senders of a message-passing network, in no particular order
    node_ct, nonzero_ct = 3, 4
    receivers = torch.tensor([1, 0, 2, 1], device="cuda", dtype=torch.long)
    senders = torch.tensor([2, 1, 1, 0], device="cuda", dtype=torch.long)
    X = torch.rand(node_ct, X_ir.dim, device="cuda", generator=gen)
    Y = torch.rand(nonzero_ct, Y_ir.dim, device="cuda", generator=gen)
    W = torch.rand(nonzero_ct, problem.weight_numel, device="cuda", generator=gen)
    tp_conv = oeq.TensorProductConv(problem, deterministic=False)
    Z_atomic = tp_conv.forward(X, Y, W, receivers, senders)
    assert Z_atomic.shape == (node_ct, Z_ir.dim)
    want = tp_oracle.forward(problem, X.cpu().numpy(), Y.cpu().numpy(), tp_conv.reorder_weights_to_e3nn(W.cpu().numpy()),
                             graph=(receivers.cpu().numpy(), senders.cpu().numpy()))
    assert rel_l2(Z_atomic.cpu().numpy(), want) <= 1e-5

    # the deterministic algorithm wants the edges sorted by receiver and the sender-major permutation of that list
    receiver_perm = torch.argsort(receivers, stable=True)
    rows, cols = receivers[receiver_perm], senders[receiver_perm]
    sender_perm = torch.argsort(cols, stable=True)
    tp_det = oeq.TensorProductConv(problem, deterministic=True)
    Z_det = tp_det.forward(X, Y[receiver_perm], W[receiver_perm], rows, cols, sender_perm)
    assert rel_l2(Z_det.cpu().numpy(), want) <= 1e-5
    assert np.allclose(Z_det.cpu().numpy(), Z_atomic.cpu().numpy(), atol=1e-6)
