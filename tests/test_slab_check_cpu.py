"""The slab checker used for full-size graphs (oracle/slab_check.py) against the oracle run on the whole of a small
graph: cutting node slabs out of a convolution must reproduce exactly the rows the whole-graph oracle gives, for a
sorted and for a shuffled edge list, first and second order."""
import numpy as np
import torch

from helpers import single, small_graph
from oracle import slab_check, tp_oracle


def test_slabs_reproduce_the_whole_graph_oracle():
    p = single("6x1o", "1x2e", "6x1o", "uvu")
    g = small_graph(n_nodes=60, mean_degree=7.0, seed=9)
    rows, cols, N = g["rows"], g["cols"], g["n_nodes"]
    E = rows.numel()
    gen = torch.Generator().manual_seed(1)
    X, X2 = (torch.randn(N, p.irreps_in1.dim, generator=gen, dtype=torch.float64) for _ in range(2))
    Y, Y2 = (torch.randn(E, p.irreps_in2.dim, generator=gen, dtype=torch.float64) for _ in range(2))
    W, W2 = (torch.randn(E, p.weight_numel, generator=gen, dtype=torch.float64) for _ in range(2))
    G = torch.randn(N, p.irreps_out.dim, generator=gen, dtype=torch.float64)
    for order in (torch.arange(E), torch.randperm(E, generator=gen)):
        r, c, y, w, y2, w2 = rows[order], cols[order], Y[order], W[order], Y2[order], W2[order]
        graph = (r.numpy(), c.numpy())
        Z = tp_oracle.forward(p, X.numpy(), y.numpy(), w.numpy(), graph=graph)
        dX, dY, dW = tp_oracle.backward(p, X.numpy(), y.numpy(), w.numpy(), G.numpy(), graph=graph)
        outs = {k: torch.tensor(v) for k, v in (("Z", Z), ("dX", dX), ("dY", dY), ("dW", dW))}
        err = slab_check.check_slabs(p, X, y, w, G, r, c, outs, [(0, 9), (30, 41)])
        assert max(err.values()) < 1e-13, err
        # a wrong row must be seen
        outs["Z"][3] += 1e-3
        assert slab_check.check_slabs(p, X, y, w, G, r, c, outs, [(0, 9)])["Z"] > 1e-6
        d2 = tp_oracle.double_backward(p, X.numpy(), y.numpy(), w.numpy(), G.numpy(), X2.numpy(), y2.numpy(), w2.numpy(),
                                       graph=graph)
        outs2 = {k: torch.tensor(v) for k, v in zip(("dX", "dY", "dW", "dG"), d2)}
        err = slab_check.check_slabs(p, X, y, w, G, r, c, outs2, [(5, 20)], second=(X2, y2, w2))
        assert max(err.values()) < 1e-13, err
