"""Spot checks of a large convolution against the fp64 oracle on small node slabs.

TEST INFRASTRUCTURE ONLY (like ``tp_oracle.py``): used by ``tests/`` and by ``bench.py`` after its timed region, as
the checker.  A full-size graph (millions of edges) is far too large for the CPU oracle, but the convolution is local:

* ``Z[r]``, ``dY[e]``, ``dW[e]`` (and the second-order ``dG[r]``) of a *receiver slab* ``[r0, r1)`` depend only on the
  edges whose receiver lies in the slab, on the sender rows of those edges and on the slab's cotangent rows;
* ``dX[c]`` of a *sender slab* ``[c0, c1)`` depends only on the edges whose sender lies in the slab.

So each slab becomes a small stand-alone graph (nodes renumbered) that the oracle finishes in seconds, and the
device results are compared on exactly the rows that the sub-graph determines completely.  The edge list may be in
any order (the atomic variant's is shuffled): slabs are cut with masks, not with ranges.
"""

from __future__ import annotations

import numpy as np
import torch

from . import tp_oracle


def _rel(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    d = np.linalg.norm(b.ravel())
    return float(np.linalg.norm((a - b).ravel()) / d) if d > 0 else float(np.linalg.norm(a.ravel()))


def _subgraph(rows, cols, edge_ids):
    """Renumbers the nodes touched by ``edge_ids``; returns (node ids, local rows, local cols) as CPU int64 tensors."""
    r, c = rows[edge_ids].cpu(), cols[edge_ids].cpu()
    nodes = torch.unique(torch.cat([r, c]))
    return nodes, torch.searchsorted(nodes, r), torch.searchsorted(nodes, c)


def _np(t, idx=None):
    t = t if idx is None else t[idx.to(t.device)]
    return t.detach().double().cpu().numpy()


def check_slabs(problem, X, Y, W, G, rows, cols, outputs, slabs, second=None, to_e3nn=None, from_e3nn=None):
    """Largest relative L2 error per output over the given slabs.

    ``X [N, L1]``, ``Y [E, L2]``, ``W [E, wn]``, ``G [N, L3]``, ``rows``/``cols [E]`` torch tensors on any device, weights
    in kernel order (``to_e3nn`` / ``from_e3nn`` map a numpy weight array to and from the oracle's order; identity when
    omitted).  ``outputs``: dict with any of ``Z, dX, dY, dW`` (first order) or, when ``second = (X2, Y2, W2)`` is
    given, ``dX, dY, dW, dG`` of the double-backward pass.  ``slabs``: list of ``(lo, hi)`` node ranges, each used
    both as a receiver slab and as a sender slab.
    """
    ident = (lambda a: a)
    to_e3nn, from_e3nn = to_e3nn or ident, from_e3nn or ident
    worst = {k: 0.0 for k in outputs}
    for lo, hi in slabs:
        # ---- receiver slab: Z / dG rows, dY and dW of its edges
        eid = torch.nonzero((rows >= lo) & (rows < hi)).flatten()
        if eid.numel() > 0:
            nodes, rl, cl = _subgraph(rows, cols, eid)
            x, y, w, g = _np(X, nodes), _np(Y, eid), to_e3nn(_np(W, eid)), _np(G, nodes)
            recv = torch.nonzero((nodes >= lo) & (nodes < hi)).flatten().numpy()
            graph = (rl.numpy(), cl.numpy())
            if second is None:
                if "Z" in outputs:
                    want = tp_oracle.forward(problem, x, y, w, graph=graph)
                    worst["Z"] = max(worst["Z"], _rel(_np(outputs["Z"], nodes)[recv], want[recv]))
                if "dY" in outputs or "dW" in outputs:
                    # cotangent rows outside the slab do not reach these edges: zero them so the sub-graph is exact
                    gz = np.zeros_like(g)
                    gz[recv] = g[recv]
                    _, wdy, wdw = tp_oracle.backward(problem, x, y, w, gz, graph=graph)
                    if "dY" in outputs:
                        worst["dY"] = max(worst["dY"], _rel(_np(outputs["dY"], eid), wdy))
                    if "dW" in outputs:
                        worst["dW"] = max(worst["dW"], _rel(_np(outputs["dW"], eid), from_e3nn(wdw)))
            else:
                X2, Y2, W2 = second
                gz = np.zeros_like(g)
                gz[recv] = g[recv]
                _, wdy, wdw, wdg = tp_oracle.double_backward(problem, x, y, w, gz, _np(X2, nodes), _np(Y2, eid),
                                                             to_e3nn(_np(W2, eid)), graph=graph)
                if "dY" in outputs:
                    worst["dY"] = max(worst["dY"], _rel(_np(outputs["dY"], eid), wdy))
                if "dW" in outputs:
                    worst["dW"] = max(worst["dW"], _rel(_np(outputs["dW"], eid), from_e3nn(wdw)))
                if "dG" in outputs:
                    worst["dG"] = max(worst["dG"], _rel(_np(outputs["dG"], nodes)[recv], wdg[recv]))
        # ---- sender slab: dX rows
        if "dX" in outputs:
            eid = torch.nonzero((cols >= lo) & (cols < hi)).flatten()
            if eid.numel() == 0:
                continue
            nodes, rl, cl = _subgraph(rows, cols, eid)
            x, y, w, g = _np(X, nodes), _np(Y, eid), to_e3nn(_np(W, eid)), _np(G, nodes)
            send = torch.nonzero((nodes >= lo) & (nodes < hi)).flatten().numpy()
            graph = (rl.numpy(), cl.numpy())
            if second is None:
                wdx, _, _ = tp_oracle.backward(problem, x, y, w, g, graph=graph)
            else:
                X2, Y2, W2 = second
                wdx, _, _, _ = tp_oracle.double_backward(problem, x, y, w, g, _np(X2, nodes), _np(Y2, eid),
                                                         to_e3nn(_np(W2, eid)), graph=graph)
            worst["dX"] = max(worst["dX"], _rel(_np(outputs["dX"], nodes)[send], wdx[send]))
    return worst
